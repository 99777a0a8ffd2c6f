"""Token embedding and the language-model head.

x = E[token, :] (src/forward.cc:198-205) into the float32 residual stream;
logits = lm_head . norm(x), returned as float32 (src/forward.cc:415-424).  A tied head
reuses the embedding matrix (the reference's GGUF loader does so when `output.weight`
is missing, src/gguf_load.cc:406-408).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, CacheNeed, Part, StateNeed, WeightSpec, build_part, register_part
from .linear import Linear


class TokenEmbedding(Part):
    """params: vocab, name; optional `scale`: a factor on the looked-up rows (applied in float32); optional `norm`:
    PartSpec of a norm applied to the looked-up rows (on the float32 stream itself) before the first layer."""

    capturable = True

    role = "embedding"

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab"])
        self.name = params["name"]
        self.table: Optional[torch.Tensor] = None
        self.row_scale = float(params.get("scale", 1.0))
        self.norm = build_part("norm", params["norm"], ctx) if params.get("norm") else None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.name, (self.vocab, self.ctx.hidden_size))]
        return specs + (self.norm.weight_specs() if self.norm is not None else [])

    def bind(self, store) -> None:
        self.table = store.get(self.name)  # left in the store: a tied head takes it too
        if self.norm is not None:
            self.norm.bind(store)

    def cache_need(self):
        """None: nothing is carried from token to token."""
        return None

    def forward(self, step, tokens: torch.Tensor) -> torch.Tensor:
        x = step.ws.buffer("x", (tokens.shape[0], self.ctx.hidden_size), torch.float32)
        K.embedding(tokens, self.table, x, self.row_scale)
        if self.norm is not None:
            self.norm.forward_in_place(x)
        return x


class PairHashEmbedding(TokenEmbedding):
    """x = scale * E[token] + B[(mul_prev * previous token + mul_cur * token) mod buckets], and B's last row
    (row `buckets`) for a sequence's first token.  The token before a step's first one is per-sequence state, kept
    in the cache beside the mixers' (one int32 per slot), so a prompt may arrive in portions and decoding goes on
    from where the prompt ended.

    params: vocab, name, scale (default 1), pairs: None or {"name", "buckets", "mul_prev", "mul_cur"}."""

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.scale = float(params.get("scale", 1.0))
        pairs = params.get("pairs") or None
        self.pairs_name = pairs["name"] if pairs else None
        self.buckets = int(pairs["buckets"]) if pairs else 0
        self.mul_prev = int(pairs["mul_prev"]) if pairs else 0
        self.mul_cur = int(pairs["mul_cur"]) if pairs else 0
        if pairs and self.buckets < 1:
            raise ValueError(f"pair embedding: {self.buckets} buckets")
        self.pairs: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = super().weight_specs()
        if self.pairs_name:
            specs.append(WeightSpec(self.pairs_name, (self.buckets + 1, self.ctx.hidden_size)))
        return specs

    def bind(self, store) -> None:
        super().bind(store)
        if self.pairs_name:
            self.pairs = store.take(self.pairs_name)
            if self.pairs.dtype != self.table.dtype:  # one of the two stored in 32-bit: both are read as 32-bit
                self.pairs, self.table = self.pairs.float(), self.table.float()

    def cache_need(self):
        return CacheNeed(state=StateNeed((("previous", (), "int32"),)))

    def forward(self, step, tokens: torch.Tensor, cache=None) -> torch.Tensor:
        if cache is None:
            raise RuntimeError("pair embedding: the step came without the embedding's state")
        x = step.ws.buffer("x", (tokens.shape[0], self.ctx.hidden_size), torch.float32)
        K.embedding_pair(tokens, step.tok_pos, step.tok_seq, step.seq_slot, step.seq_qstart, step.seq_qlen,
                         cache.state["previous"], self.table, self.pairs, x, self.buckets, self.mul_prev, self.mul_cur,
                         self.scale)
        if self.norm is not None:
            self.norm.forward_in_place(x)
        return x


class LMHead(Part):
    """params: vocab, name, tied_to (name of the embedding tensor, or None), scale (a factor on the float32 logits,
    default 1)."""

    capturable = True

    role = "lm_head"

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab"])
        self.name = params["name"]
        self.tied_to = params.get("tied_to")
        self.scale = float(params.get("scale", 1.0))
        self.linear: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        if self.tied_to:
            return []
        return [WeightSpec(self.name, (self.vocab, self.ctx.hidden_size))]

    def bind(self, store) -> None:
        self.linear = Linear(store.get(self.tied_to) if self.tied_to else store.take(self.name),
                             self.tied_to or self.name)

    def parameter_bytes(self) -> int:
        return self.linear.parameter_bytes()

    def forward(self, step, h: torch.Tensor, out_name: str = "logits") -> torch.Tensor:
        logits = self.linear.forward(step, h, out_name, out_dtype=torch.float32)
        if self.scale != 1.0:
            K.scale_(logits, self.scale)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding)
register_part("lm_head", "linear_head", LMHead)
