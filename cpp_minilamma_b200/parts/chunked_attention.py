"""Grouped-query attention whose keys and values have head sizes of their own, masked in chunks.

    q = W_q h, k = W_k h, v = W_v h                       Hq heads of d, Hk heads of d, Hk heads of dv
    q <- q / rms(q) * w_q,  k <- k / rms(k) * w_k         over the whole projection, all heads at once (optional)
    rotate the first `rotary_dims` dimensions of every q and k head by position * f_i
    score(i, j) = scale * q_i . k_j   for j <= i, j // chunk == i // chunk (chunk 0: every j <= i),
                                      and j > i - window where window > 0
    out = W_o concat_heads(softmax(score) v)

Options beyond that, each a parameter: a query temperature (q at position p times 1 + coef * ln(floor((p + 1) /
every) + 1)); a sink in the softmax (weights exp(s_j) / (1 + sum_j exp(s_j)): one more key that scores 0 and carries
no value), or a learned one (exp(c_h) in place of the 1, c_h a number per query head that no scale touches); values
that are the keys themselves as projected, before norm and rotation (no W_v; dv == d); an output gate read from the mixer's own input, one number per head (head h's output times
sigmoid(W_g h)_h) or one per element, applied before W_o; a smooth cap on the scores, s <- cap * tanh(s / cap) after the
scale; a window that keeps the sequence's first tokens (key j < keep_first stays visible whatever its distance, at its own
position); keys and values that are another layer's (`kv_shared`: the layer has queries and an output projection only and
reads the cache of the schedule entry named by its own entry's `cache_of`, with its own mask, scale and cap).

Chunks count from position 0 of the sequence, not from where a step's tokens begin.  Keys and values live in
the paged cache; a chunked layer asks the cache to keep only what its chunk can still reach (a window of one
chunk), so pages of finished chunks go back to the pool.  Every constant is a parameter; the Llama attention
of `parts/attention.py` is the case d == dv, scale 1 / sqrt(d), no chunk, no norm, all dimensions rotated,
which has kernels of its own.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, CacheNeed, KVNeed, Mixer, WeightSpec, register_part
from .linear import Linear
from .rope import shared_position_encoding


class ChunkedAttention(Mixer):
    """params:
      n_heads, n_kv_heads, head_dim, v_head_dim     sizes
      scale                                         factor on q . k
      chunk                                         0 = plain causal
      window                                        0 = none
      position                                      PartSpec of a rotary encoding over `rotary_dims` dimensions, or None
      rotary_dims                                   how many leading dimensions of a head are rotated
      qk_norm                                       None or {"q": tensor name, "k": tensor name, "eps": float}
      q_temp                                        None or {"coef": float, "every": int}: the query temperature
      sink                                          True: the softmax's denominator has one more term exp(0); a tensor
                                                    name: one more term exp(c_h), c [n_heads] loaded under that name
      values                                        "projected" (default) or "keys": v = W_k h, no names["v"]
      out_name                                      workspace name of the result (default "o"; two mixers whose results
                                                    are both pending need two)
      gate                                          None, "head" or "element": an output gate sigmoid(W_g h), names["g"]
      softcap                                       0 / None, or the cap c: score <- c * tanh(score / c) after the scale
      keep_first                                    with a window: keys at positions below this stay visible
      kv_shared                                     True: no names["k"] / ["v"]; keys and values are read from the cache
                                                    of another schedule entry (the entry's `cache_of`)
      cache_window, cache_keep_first                what the cache must keep when other layers read this layer's keys
                                                    with masks of their own (default: this layer's window / keep_first)
      names                                         {"q","k","v","o"} (and "g"): tensor names
    """

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params.get("v_head_dim") or self.d)
        self.scale = float(params["scale"])
        self.chunk = int(params.get("chunk") or 0)
        self.window = int(params.get("window") or 0)
        self.names = dict(params["names"])
        self.qk_norm = dict(params["qk_norm"]) if params.get("qk_norm") else None
        q_temp = params.get("q_temp")
        self.q_temp = (float(q_temp["coef"]), int(q_temp["every"])) if q_temp else None
        sink = params.get("sink", False)
        self.sink_name = sink if isinstance(sink, str) else None
        self.sink = bool(sink)
        self.sink_values: Optional[torch.Tensor] = None
        self.v_from_k = (params.get("values") or "projected") == "keys"
        if params.get("values") not in (None, "projected", "keys"):
            raise ValueError(f"attention: values {params.get('values')!r} are neither 'projected' nor 'keys'")
        if self.v_from_k and self.dv != self.d:
            raise ValueError(f"attention: values that are the keys have their size, got {self.dv} / {self.d}")
        self.out_name = params.get("out_name") or "o"
        self.softcap = float(params.get("softcap") or 0.0)
        self.keep_first = int(params.get("keep_first") or 0) if self.window > 0 else 0
        self.kv_shared = bool(params.get("kv_shared", False))
        self.cache_window = int(params["cache_window"]) if params.get("cache_window") is not None else self.window
        self.cache_keep_first = int(params["cache_keep_first"]) if params.get("cache_keep_first") is not None else self.keep_first
        if self.softcap < 0 or self.keep_first < 0:
            raise ValueError(f"attention: a cap of {self.softcap} or {self.keep_first} kept tokens")
        if self.keep_first and self.chunk:
            raise ValueError("attention: kept first tokens go with a window, not with chunks")
        if self.kv_shared and (self.v_from_k or params.get("qk_norm")):
            raise ValueError("attention: a layer that reads another layer's keys has no key options of its own")
        self.gate = params.get("gate") or None
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"attention: gate {self.gate!r} is neither 'head' nor 'element'")
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError(f"attention: a query temperature every {self.q_temp[1]} positions")
        self.rot = int(params.get("rotary_dims") or 0) if params.get("position") else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        if self.rot % 2 or self.rot > self.d:
            raise ValueError(f"attention: {self.rot} rotated dimensions of a head of {self.d}")
        if self.dv > 256:
            raise ValueError(f"attention: value heads of {self.dv} exceed the 256 the kernel takes")
        self.position = shared_position_encoding(params["position"], ctx) if self.rot else None
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_weight = self.k_weight = None

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        specs = [WeightSpec(self.names["q"], (self.n_heads * self.d, D))]
        if not self.kv_shared:
            specs.append(WeightSpec(self.names["k"], (self.n_kv_heads * self.d, D)))
            if not self.v_from_k:
                specs.append(WeightSpec(self.names["v"], (self.n_kv_heads * self.dv, D)))
        specs.append(WeightSpec(self.names["o"], (D, self.n_heads * self.dv)))
        if self.sink_name:
            specs.append(WeightSpec(self.sink_name, (self.n_heads,), kind="vector", init="normal"))
        if self.gate:
            specs.append(WeightSpec(self.names["g"], (self._gate_width(), D)))
        if self.qk_norm:
            specs.append(WeightSpec(self.qk_norm["q"], (self.n_heads * self.d,), kind="vector", init="norm"))
            specs.append(WeightSpec(self.qk_norm["k"], (self.n_kv_heads * self.d,), kind="vector", init="norm"))
        return specs

    def _gate_width(self) -> int:
        return self.n_heads if self.gate == "head" else self.n_heads * self.dv

    def bind(self, store) -> None:
        # the gate reads the same rows as q, k and v: its matrix rides behind theirs in the one fused product
        parts = [p for p in ("q", "k", "v", "g") if (p != "v" or not self.v_from_k) and (p != "g" or self.gate)
                 and (p == "q" or p == "g" or not self.kv_shared)]
        mats = [store.take(self.names[p]) for p in parts]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        fused = torch.cat(mats, dim=0)
        spare = -fused.shape[0] % 8  # rows of zeros up to a multiple of 8: the product's rows stay 16-byte aligned
        if spare:
            fused = torch.cat([fused, torch.zeros((spare, fused.shape[1]), dtype=fused.dtype, device=fused.device)], dim=0)
        self.qkv = Linear(fused, "+".join(self.names[p] if p == "q" else p for p in parts))
        del mats, fused
        if self.sink_name:
            self.sink_values = store.take(self.sink_name)
        self.o = Linear(store.take(self.names["o"]), self.names["o"])
        if self.qk_norm:
            self.q_weight = store.take(self.qk_norm["q"])
            self.k_weight = store.take(self.qk_norm["k"])

    def parameter_bytes(self) -> int:
        return self.qkv.parameter_bytes() + self.o.parameter_bytes()

    def cache_need(self) -> CacheNeed:
        # a query reads nothing before its chunk's first key, which lies less than `chunk` positions back
        window = self.cache_window
        reach = self.chunk if window <= 0 else (min(self.chunk, window) if self.chunk else window)
        return CacheNeed(kv=KVNeed(self.n_kv_heads, self.d, reach, self.dv if self.dv != self.d else 0,
                                   keep_first=self.cache_keep_first if reach > 0 and not self.chunk else 0))

    def _tensor_cores(self) -> bool:
        return K.local_attention_mma_supported(self.ctx.act_dtype, self.d, self.dv)

    def step_metadata_key(self):
        # prompt steps on tensor cores read a list of query tiles; layers share it whatever their sizes
        return ("chunked_attention.tiles", K.PREFILL_TILE) if self.ctx.act_dtype == torch.bfloat16 else None

    def prepare_step(self, shape):
        """Tiles of up to PREFILL_TILE query rows as (sequence, first row among the sequence's new tokens), the
        sequences with the most rows first.  Steps of single tokens need no list."""
        if shape.all_decode:
            return {}
        lists = {"tile_seq": [], "tile_row0": []}
        wide = []
        for i in sorted(range(shape.n_seqs), key=lambda i: -shape.lens[i]):
            for row0 in range(0, shape.lens[i], K.PREFILL_TILE):
                lists["tile_seq"].append(i)
                lists["tile_row0"].append(row0)
            for row0 in range(0, shape.lens[i], 2 * K.PREFILL_TILE):
                wide.append((shape.starts[i] + min(shape.lens[i], row0 + 2 * K.PREFILL_TILE), i, row0))
        # the same rows in tiles of twice as many, for the tcgen05 kernel, which walks its list from the back
        wide.sort()
        lists["wide_seq"] = [i for _, i, _ in wide]
        lists["wide_row0"] = [row0 for _, _, row0 in wide]
        return lists

    def forward(self, step, h, cache):
        T = h.shape[0]
        act = self.ctx.act_dtype
        if cache.k is None:
            raise RuntimeError("attention: the cache view has no key/value storage")
        if self.kv_shared and cache.owns_kv:
            raise RuntimeError("attention: a layer without keys of its own must read another schedule entry's cache")
        qkv = self.qkv.forward(step, h, "qkv")
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        q = step.ws.buffer("q", (T, self.n_heads * self.d), act)
        K.local_attention_prepare(qkv, self.q_weight, self.k_weight, cos, sin, step.tok_pos, step.tok_seq,
                                  step.seq_slot, cache.block_table, q, cache.k, cache.v, self.n_heads,
                                  self.n_kv_heads, self.d, self.dv, self.rot,
                                  bool(self.position.interleaved) if self.position is not None else False,
                                  float(self.qk_norm["eps"]) if self.qk_norm else 0.0, q_temp=self.q_temp,
                                  v_from_k=self.v_from_k, write_kv=not self.kv_shared)
        out = step.ws.buffer("attn", (T, self.n_heads * self.dv), act)
        self._attend(step, q, cache, out)
        if self.gate:
            gate_col = self.n_heads * self.d + (0 if self.kv_shared else
                                                self.n_kv_heads * (self.d if self.v_from_k else self.d + self.dv))
            K.heads_gate(out, qkv, gate_col, out, self.n_heads, self.dv, per_head=self.gate == "head")
        return self.o.forward(step, out, self.out_name)

    def _attend(self, step, q, cache, out) -> None:
        act = self.ctx.act_dtype
        learned = self.sink_values  # a sink with a score of its own per head, or None
        extra = {"keep_first": self.keep_first, "softcap": self.softcap}
        plain = not self.keep_first and not self.softcap  # what the Llama attention's kernels know
        if ((plain or K.attention_decode_takes_window_extras(act, self.d)) and step.all_decode and self.d == self.dv
                and self.d % 16 == 0 and 16 <= self.d <= 256
                and not (self.chunk and self.window) and act == torch.bfloat16
                and (not self.sink or K.USE_TENSOR_CORE_DECODE)):
            # single tokens, keys and values of one head size: the Llama attention's decode kernels (TMA-fed or
            # mma.sync), which take the chunk as the key range's start; one block per (sequence, kv head)
            K.attention_decode(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, cache.block_table, None, out,
                               step.n_seqs, self.n_heads, self.n_kv_heads, self.d, 1, self.window, self.scale,
                               chunk=self.chunk, sink=self.sink, sink_values=learned, **extra)
            return
        if step.all_decode and self._tensor_cores():
            # single tokens that the kernels above do not take (a sink, values of another size): the tensor-core
            # prompt kernel with a kv head's query heads as the rows of its tile
            group = self.n_heads // self.n_kv_heads
            splits = K.local_attention_heads_splits(step.n_seqs, self.n_kv_heads * -(-group // 64), self.ctx.multiprocessors)
            scratch = step.ws.buffer("attn.parts", (K.local_attention_heads_scratch(step.n_seqs, self.n_heads, self.dv, splits),),
                                     torch.float32) if splits > 1 else None
            K.local_attention_heads(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                    cache.block_table, out, step.n_seqs, self.n_heads, self.n_kv_heads, self.d, self.dv,
                                    self.chunk, self.window, self.scale, sink=self.sink, n_splits=splits, scratch=scratch,
                                    sink_values=learned, **extra)
            return
        tiles = step.meta.get(self.step_metadata_key()) if not step.all_decode else None
        if tiles and self.d == self.dv and K.attention_prefill_takes_chunks(act, self.d):
            # keys and values of one head size that the Llama attention's tcgen05 prompt kernel takes: that kernel,
            # which knows the chunk mask too
            K.attention_prefill(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                tiles["tile_seq"], tiles["tile_row0"], cache.block_table, out,
                                tiles["tile_seq"].shape[0], self.n_heads, self.n_kv_heads, self.d, self.window,
                                self.scale, wide_tiles=(tiles["wide_seq"], tiles["wide_row0"]), chunk=self.chunk,
                                sink=self.sink, sink_values=learned, **extra)
            return
        if tiles and self._tensor_cores():
            K.local_attention_tiles(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                    tiles["tile_seq"], tiles["tile_row0"], cache.block_table, out, self.n_heads,
                                    self.n_kv_heads, self.d, self.dv, self.chunk, self.window, self.scale,
                                    sink=self.sink, sink_values=learned, **extra)
            return
        K.local_attention(q, cache.k, cache.v, step.tok_pos, step.tok_seq, step.seq_slot, cache.block_table, out,
                          self.n_heads, self.n_kv_heads, self.d, self.dv, self.chunk, self.window, self.scale,
                          sink=self.sink, sink_values=learned, **extra)


register_part("mixer", "chunked_attention", ChunkedAttention)
