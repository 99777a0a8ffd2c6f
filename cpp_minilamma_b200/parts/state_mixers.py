"""Mixers that keep a matrix per sequence and head instead of keys and values.

Both run   S_t = diag(g_t) S_(t-1) + k_t u_t^T,   o_t = S_t^T q_t   (S is [d, dv], float32, zero at the start of a
sequence, carried from step to step in the cache's per-slot state), so the read-out sees the current token's
write, and both normalise every head's o by its root mean square before a gate and the output projection.

`retention`          one fixed decay per head, u = v; q and k carry rotary positions, k / sqrt(d);
                     out = W_o (o / rms(o) * silu(W_g h))
`gated_delta_rule`   a decay per head and key channel, g = exp(-exp(A) softplus(W_a2 W_a1 h + b)), and the delta
                     rule u = beta (v - S^T k) with beta = sigmoid(W_b h); q, k, v pass a short causal
                     convolution over time and silu, q and k are scaled to unit length per head, q / sqrt(d);
                     the last taps - 1 convolution inputs of a sequence are state too;
                     out = W_o (o / rms(o) * w * sigmoid(W_g2 W_g1 h))

`gated_linear_attention`  a decay per head and key channel, g = sigmoid(W_a2 W_a1 h + b)^(1 / tau), u = v, q / sqrt(d);
                     out = W_o (o / rms(o) * w * silu(W_g h))

`state_space`        (the state-space duality form) one projection W_in h = [z | x | B | C | dt]; x, B and C pass a short
                     causal convolution with a bias and silu; dt = softplus(dt + bias) per head; one decay per token
                     and head, g = exp(-exp(A_h) dt); k = B and q = C are shared by the heads of a group, u = dt x;
                     o + D_h x, times silu(z), normalised in a few equal parts of the row, times a weight, then W_o;
                     the last taps - 1 convolution inputs of a sequence are state too

What enters the recurrence is float32 (decays, step sizes, gates, unit vectors, the state); the projections are
products in the run's dtype.  Sizes, decays, tap counts and eps are parameters.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, CacheNeed, Mixer, StateNeed, WeightSpec, register_part
from .linear import Linear
from .rope import shared_position_encoding


def _pad_rows(matrix: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Zero rows up to a multiple of 8: the product's row stride then keeps 16-byte alignment."""
    spare = -matrix.shape[0] % multiple
    if not spare:
        return matrix
    return torch.cat([matrix, torch.zeros((spare, matrix.shape[1]), dtype=matrix.dtype, device=matrix.device)], dim=0)


def _same_dtype(mats):
    return [m.float() for m in mats] if len({m.dtype for m in mats}) > 1 else list(mats)


class Retention(Mixer):
    """params: n_heads, head_dim, v_head_dim, decay (one per head), eps (of the head norm),
    position (PartSpec of a rotary encoding over `rotary_dims` dimensions, or None), rotary_dims,
    names {"q","k","v","g","o"}: tensor names."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params["v_head_dim"])
        self.decay = [float(x) for x in params["decay"]]
        self.eps = float(params["eps"])
        self.names = dict(params["names"])
        self.rot = int(params.get("rotary_dims") or 0) if params.get("position") else 0
        if len(self.decay) != self.n_heads:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.n_heads} heads")
        if self.rot % 2 or self.rot > self.d:
            raise ValueError(f"retention: {self.rot} rotated dimensions of a head of {self.d}")
        self.position = shared_position_encoding(params["position"], ctx) if self.rot else None
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=ctx.device)
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        D, H = self.ctx.hidden_size, self.n_heads
        return [WeightSpec(self.names["q"], (H * self.d, D)), WeightSpec(self.names["k"], (H * self.d, D)),
                WeightSpec(self.names["v"], (H * self.dv, D)), WeightSpec(self.names["g"], (H * self.dv, D)),
                WeightSpec(self.names["o"], (D, H * self.dv))]

    def bind(self, store) -> None:
        mats = _same_dtype([store.take(self.names[p]) for p in ("q", "k", "v", "g")])
        self.proj = Linear(_pad_rows(torch.cat(mats, dim=0)), self.names["q"] + "+k+v+g")
        del mats
        self.o = Linear(store.take(self.names["o"]), self.names["o"])

    def parameter_bytes(self) -> int:
        return self.proj.parameter_bytes() + self.o.parameter_bytes()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((("S", (self.n_heads, self.d, self.dv)),)))

    def forward(self, step, h, cache):
        T, H, d, dv = h.shape[0], self.n_heads, self.d, self.dv
        ws = step.ws
        proj = self.proj.forward(step, h, "mix.proj")
        q = ws.buffer("mix.q", (T, H * d), torch.float32)
        k = ws.buffer("mix.k", (T, H * d), torch.float32)
        v = ws.buffer("mix.v", (T, H * dv), torch.float32)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        K.retention_prepare(proj, cos, sin, step.tok_pos, q, k, v, H, d, dv, self.rot,
                            bool(self.position.interleaved) if self.position is not None else False,
                            1.0 / math.sqrt(d))
        o = ws.buffer("mix.o", (T, H * dv), torch.float32)
        K.state_scan(q, k, v, None, None, self.decay_t, cache.state["S"], o, step.seq_slot, step.seq_qstart,
                     step.seq_qlen, step.n_seqs, H, H, d, dv)
        gated = ws.buffer("mix.gated", (T, H * dv), self.ctx.act_dtype)
        K.head_norm_gate(o, None, proj, gated, H, dv, self.eps, K.GATE_SILU, gate_col=H * (2 * d + dv))
        return self.o.forward(step, gated, "o")


class GatedDeltaRule(Mixer):
    """params: n_heads, n_kv_heads (q and k heads; value head h reads q/k head h // (n_heads / n_kv_heads)),
    head_dim, v_head_dim, conv (taps), eps (of the head norm), unit_eps (inside the root of the unit length),
    names: tensor names for "q","k","v" (their convolution taps are "<name>.conv"), "b", "a1", "a2", "dt_bias",
    "A_log", "g1", "g2", "norm", "o"; decay_rank, gate_rank: inner sizes of the two low-rank pairs (-1: as stored)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params["v_head_dim"])
        self.taps = int(params["conv"])
        self.eps = float(params["eps"])
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        self.decay_rank = int(params.get("decay_rank") or -1)  # -1: whatever the tensors have
        self.gate_rank = int(params.get("gate_rank") or -1)
        self.names = dict(params["names"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"delta rule: {self.n_heads} heads are not a multiple of {self.n_kv_heads} q/k heads")
        if self.taps < 1:
            raise ValueError("delta rule: the convolution needs at least one tap")
        self.channels = 2 * self.n_kv_heads * self.d + self.n_heads * self.dv
        self.proj: Optional[Linear] = None      # q, k, v, b
        self.low: Optional[Linear] = None       # a1, g1
        self.high: Optional[Linear] = None      # a2 and g2 side by side on the low ranks
        self.o: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, d, dv, n = self.ctx.hidden_size, self.n_heads, self.n_kv_heads, self.d, self.dv, self.names
        return [WeightSpec(n["q"], (G * d, D)), WeightSpec(n["q"] + ".conv", (G * d, self.taps), kind="vector"),
                WeightSpec(n["k"], (G * d, D)), WeightSpec(n["k"] + ".conv", (G * d, self.taps), kind="vector"),
                WeightSpec(n["v"], (H * dv, D)), WeightSpec(n["v"] + ".conv", (H * dv, self.taps), kind="vector"),
                WeightSpec(n["b"], (H, D)), WeightSpec(n["A_log"], (H,), kind="vector"),
                WeightSpec(n["norm"], (dv,), kind="vector", init="norm"),
                WeightSpec(n["a1"], (self.decay_rank, D)), WeightSpec(n["a2"], (H * d, self.decay_rank)),
                WeightSpec(n["dt_bias"], (H * d,), kind="vector"),
                WeightSpec(n["g1"], (self.gate_rank, D)), WeightSpec(n["g2"], (H * dv, self.gate_rank)),
                WeightSpec(n["o"], (D, H * dv))]

    def bind(self, store) -> None:
        n = self.names
        mats = _same_dtype([store.take(n[p]) for p in ("q", "k", "v", "b")])
        self.proj = Linear(_pad_rows(torch.cat(mats, dim=0)), n["q"] + "+k+v+b")
        low = _same_dtype([store.take(n["a1"]), store.take(n["g1"])])
        self.low = Linear(_pad_rows(torch.cat(low, dim=0)), n["a1"] + "+g1")
        # the second level of both low-rank pairs as one product: [[a2, 0], [0, g2]] over the columns (a1 | g1 | padding)
        a2, g2 = _same_dtype([store.take(n["a2"]), store.take(n["g2"])])
        ra, rg, width = low[0].shape[0], low[1].shape[0], self.low.out_features
        if a2.shape[1] != ra or g2.shape[1] != rg:
            raise ValueError(f"delta rule: {n['a2']} / {n['g2']} read {a2.shape[1]} / {g2.shape[1]} inputs, "
                             f"{n['a1']} / {n['g1']} give {ra} / {rg}")
        high = torch.zeros((a2.shape[0] + g2.shape[0], width), dtype=a2.dtype, device=a2.device)
        high[:a2.shape[0], :ra] = a2
        high[a2.shape[0]:, ra:ra + rg] = g2
        self.high = Linear(_pad_rows(high), n["a2"] + "+g2")
        del mats, low, a2, g2, high
        self.conv_w = torch.cat([store.take(n[p] + ".conv") for p in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = store.take(n["A_log"])
        self.dt_bias = store.take(n["dt_bias"])
        self.norm_w = store.take(n["norm"])
        self.o = Linear(store.take(n["o"]), n["o"])

    def parameter_bytes(self) -> int:
        return sum(l.parameter_bytes() for l in (self.proj, self.low, self.high, self.o))

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((("S", (self.n_heads, self.d, self.dv)),
                                          ("conv", (self.taps - 1, self.channels)))))

    def forward(self, step, h, cache):
        T, H, G, d, dv = h.shape[0], self.n_heads, self.n_kv_heads, self.d, self.dv
        ws = step.ws
        proj = self.proj.forward(step, h, "mix.proj")
        low = self.low.forward(step, h, "mix.low")
        high = self.high.forward(step, low, "mix.high", out_dtype=torch.float32)  # [T, H d (decay) + H dv (gate) + padding]
        q = ws.buffer("mix.q", (T, G * d), torch.float32)
        k = ws.buffer("mix.k", (T, G * d), torch.float32)
        v = ws.buffer("mix.v", (T, H * dv), torch.float32)
        g = ws.buffer("mix.g", (T, H * d), torch.float32)
        beta = ws.buffer("mix.beta", (T, H), torch.float32)
        K.delta_prepare(proj, high, self.conv_w, cache.state["conv"], self.a_log, self.dt_bias, step.tok_seq,
                        step.seq_slot, step.seq_qstart, q, k, v, g, beta, H, G, d, dv, self.taps, self.unit_eps)
        K.conv_state_update(proj, cache.state["conv"], step.seq_slot, step.seq_qstart, step.seq_qlen, step.n_seqs,
                            self.channels, self.taps)
        o = ws.buffer("mix.o", (T, H * dv), torch.float32)
        K.state_scan(q, k, v, g, beta, None, cache.state["S"], o, step.seq_slot, step.seq_qstart, step.seq_qlen,
                     step.n_seqs, H, G, d, dv)
        gated = ws.buffer("mix.gated", (T, H * dv), self.ctx.act_dtype)
        K.head_norm_gate(o, self.norm_w, high, gated, H, dv, self.eps, K.GATE_SIGMOID, gate_col=H * d)
        return self.o.forward(step, gated, "o")


class GatedLinearAttention(Mixer):
    """params: n_heads, head_dim, v_head_dim, tau (the decay is sigmoid(z)^(1 / tau)), eps (of the head norm),
    decay_rank (inner size of the low-rank pair, -1: as stored), out_name (workspace name of the result, default "o"),
    names: tensor names for "q", "k", "v", "g", "a1", "a2", "a2_bias", "norm", "o"."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.d = int(params["head_dim"])
        self.dv = int(params["v_head_dim"])
        self.tau = float(params["tau"])
        self.eps = float(params["eps"])
        self.decay_rank = int(params.get("decay_rank") or -1)
        self.names = dict(params["names"])
        self.out_name = params.get("out_name") or "o"
        if self.tau <= 0:
            raise ValueError(f"gated linear attention: tau {self.tau} must be positive")
        self.proj: Optional[Linear] = None   # q, k, v, g
        self.low: Optional[Linear] = None    # a1
        self.high: Optional[Linear] = None   # a2 over the columns of a1
        self.o: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        D, H, d, dv, n = self.ctx.hidden_size, self.n_heads, self.d, self.dv, self.names
        return [WeightSpec(n["q"], (H * d, D)), WeightSpec(n["k"], (H * d, D)), WeightSpec(n["v"], (H * dv, D)),
                WeightSpec(n["g"], (H * dv, D)), WeightSpec(n["a1"], (self.decay_rank, D)),
                WeightSpec(n["a2"], (H * d, self.decay_rank)), WeightSpec(n["a2_bias"], (H * d,), kind="vector"),
                WeightSpec(n["norm"], (dv,), kind="vector", init="norm"), WeightSpec(n["o"], (D, H * dv))]

    def bind(self, store) -> None:
        n = self.names
        a1 = store.take(n["a1"])
        a2 = store.take(n["a2"])
        if a2.shape[1] != a1.shape[0]:
            raise ValueError(f"gated linear attention: {n['a2']} reads {a2.shape[1]} inputs, {n['a1']} gives {a1.shape[0]}")
        mats = _same_dtype([store.take(n[p]) for p in ("q", "k", "v", "g")])
        self.proj = Linear(_pad_rows(torch.cat(mats, dim=0)), n["q"] + "+k+v+g")
        a1, a2 = _same_dtype([a1, a2])
        self.low = Linear(_pad_rows(a1), n["a1"])
        # the second level over the first level's columns (and its padding)
        high = torch.zeros((a2.shape[0], self.low.out_features), dtype=a2.dtype, device=a2.device)
        high[:, :a2.shape[1]] = a2
        self.high = Linear(_pad_rows(high), n["a2"])
        del mats, a1, a2, high
        self.bias = store.take(n["a2_bias"])
        self.norm_w = store.take(n["norm"])
        self.o = Linear(store.take(n["o"]), n["o"])

    def parameter_bytes(self) -> int:
        return sum(l.parameter_bytes() for l in (self.proj, self.low, self.high, self.o))

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((("S", (self.n_heads, self.d, self.dv)),)))

    def forward(self, step, h, cache):
        T, H, d, dv = h.shape[0], self.n_heads, self.d, self.dv
        ws = step.ws
        proj = self.proj.forward(step, h, "gla.proj")
        low = self.low.forward(step, h, "gla.low")
        rate = self.high.forward(step, low, "gla.rate", out_dtype=torch.float32)  # [T, H d (+ padding)]
        q = ws.buffer("gla.q", (T, H * d), torch.float32)
        k = ws.buffer("gla.k", (T, H * d), torch.float32)
        v = ws.buffer("gla.v", (T, H * dv), torch.float32)
        g = ws.buffer("gla.g", (T, H * d), torch.float32)
        K.channel_decay_prepare(proj, rate, self.bias, q, k, v, g, H, d, dv, 1.0 / math.sqrt(d), self.tau)
        o = ws.buffer("gla.o", (T, H * dv), torch.float32)
        K.state_scan(q, k, v, g, None, None, cache.state["S"], o, step.seq_slot, step.seq_qstart, step.seq_qlen,
                     step.n_seqs, H, H, d, dv)
        gated = ws.buffer("gla.gated", (T, H * dv), self.ctx.act_dtype)
        K.head_norm_gate(o, self.norm_w, proj, gated, H, dv, self.eps, K.GATE_SILU, gate_col=H * (2 * d + dv))
        return self.o.forward(step, gated, self.out_name)


class StateSpace(Mixer):
    """params: n_heads, n_groups (heads of one group share B and C), v_head_dim (columns of x per head), state (rows of
    the state per head: the size of B and C), conv (taps), norm_groups (equal parts of the row that are normalised
    each by itself), eps (of that norm), out_name (workspace name of the result, default "o"),
    names: tensor names for "in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o"."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.n_groups = int(params["n_groups"])
        self.dv = int(params["v_head_dim"])
        self.d = int(params["state"])
        self.taps = int(params["conv"])
        self.parts = int(params.get("norm_groups") or 1)
        self.eps = float(params["eps"])
        self.names = dict(params["names"])
        self.out_name = params.get("out_name") or "o"
        if self.n_groups < 1 or self.n_heads % self.n_groups:
            raise ValueError(f"state space: {self.n_heads} heads are not a multiple of {self.n_groups} groups")
        if self.taps < 1:
            raise ValueError("state space: the convolution needs at least one tap")
        self.inner = self.n_heads * self.dv
        if self.parts < 1 or self.inner % self.parts:
            raise ValueError(f"state space: {self.inner} columns cannot be normalised in {self.parts} equal parts")
        self.channels = self.inner + 2 * self.n_groups * self.d        # what passes the convolution: x, B, C
        self.rows = 2 * self.inner + 2 * self.n_groups * self.d + self.n_heads
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        D, H, n = self.ctx.hidden_size, self.n_heads, self.names
        return [WeightSpec(n["in"], (self.rows, D)),
                WeightSpec(n["conv"], (self.channels, self.taps), kind="vector"),
                WeightSpec(n["conv_bias"], (self.channels,), kind="vector"),
                WeightSpec(n["dt_bias"], (H,), kind="vector"), WeightSpec(n["A_log"], (H,), kind="vector"),
                WeightSpec(n["D"], (H,), kind="vector", init="norm"),
                WeightSpec(n["norm"], (self.inner,), kind="vector", init="norm"),
                WeightSpec(n["o"], (D, self.inner))]

    def bind(self, store) -> None:
        n = self.names
        self.proj = Linear(_pad_rows(store.take(n["in"])), n["in"])
        self.conv_w = store.take(n["conv"]).contiguous()
        self.conv_b = store.take(n["conv_bias"])
        self.dt_bias = store.take(n["dt_bias"])
        self.a_log = store.take(n["A_log"])
        self.skip = store.take(n["D"])
        self.norm_w = store.take(n["norm"])
        self.o = Linear(store.take(n["o"]), n["o"])

    def parameter_bytes(self) -> int:
        return self.proj.parameter_bytes() + self.o.parameter_bytes()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((("S", (self.n_heads, self.d, self.dv)),
                                          ("conv", (self.taps - 1, self.channels)))))

    def forward(self, step, h, cache):
        T, H, G, d, dv = h.shape[0], self.n_heads, self.n_groups, self.d, self.dv
        ws = step.ws
        proj = self.proj.forward(step, h, "ssd.proj")
        q = ws.buffer("ssd.q", (T, G * d), torch.float32)
        k = ws.buffer("ssd.k", (T, G * d), torch.float32)
        u = ws.buffer("ssd.u", (T, self.inner), torch.float32)
        xs = ws.buffer("ssd.x", (T, self.inner), torch.float32)
        decay = ws.buffer("ssd.decay", (T, H), torch.float32)
        K.ssd_prepare(proj, self.conv_w, self.conv_b, cache.state["conv"], self.a_log, self.dt_bias, step.tok_seq,
                      step.seq_slot, step.seq_qstart, q, k, u, xs, decay, H, G, d, dv, self.taps)
        K.conv_state_update(proj, cache.state["conv"], step.seq_slot, step.seq_qstart, step.seq_qlen, step.n_seqs,
                            self.channels, self.taps, first_column=self.inner)
        o = ws.buffer("ssd.o", (T, self.inner), torch.float32)
        K.state_scan(q, k, u, None, None, None, cache.state["S"], o, step.seq_slot, step.seq_qstart, step.seq_qlen,
                     step.n_seqs, H, G, d, dv, token_decay=decay)
        gated = ws.buffer("ssd.gated", (T, self.inner), self.ctx.act_dtype)
        K.gated_group_norm(o, xs, self.skip, proj, self.norm_w, gated, dv, self.parts, self.eps)
        return self.o.forward(step, gated, self.out_name)


register_part("mixer", "state_space", StateSpace)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "retention", Retention)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
