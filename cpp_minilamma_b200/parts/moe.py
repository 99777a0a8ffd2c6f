"""A routed feed-forward: every token goes through `top` of E small SwiGLU experts, plus a shared one.

    z       = W_r h + b_r                          float32 router logits
    chosen  = the `top` experts with the largest z (ties: the lower index)
    weights = softmax over the chosen logits alone
    out     = sum_j weights_j * expert_{chosen_j}(h)  +  shared(h)        expert(h) = W_down (silu(W_gate h) * W_up h)

Other forms, each a parameter: scores over all experts (s = softmax(z) over every expert; the choice goes by s + a
stored correction, the weights are the chosen s over their sum, times a constant); experts without a gate,
W_down gelu(W_up h); identity experts - the router's last rows belong to experts without tensors, whose output is
their input times the weight; sigmoid scores with a choice limited to groups (s = sigmoid(z); the experts are cut into
`count` runs of consecutive experts of one length, a run is rated by its top two s added up, only experts of the `keep`
best-rated runs can be chosen; the weights are the chosen s over their sum); a gate on the shared expert, sigmoid(w_g . h), one number per token, whose row rides
behind the router's so that the routing kernel forms it.

The experts' matrices are stacked ([E, 2 I, D] gate rows then up rows, and [E, D, I]); the routing stays on the
device: the (token, choice) pairs are sorted by expert there and the two products run over tiles of one expert's
rows (csrc/moe.cu), so a step's launches follow from its number of tokens alone and decode steps replay from a
graph.  bfloat16 steps take the tensor-core kernels, float32 steps the plain ones.  The shared expert is a dense
SwiGLU feed-forward of its own width (the `swiglu` part); its output is added in the same pass that sums a token's
experts.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, FeedForward, PartSpec, WeightSpec, build_part, register_part


class RoutedFeedForward(FeedForward):
    """params:
      experts, top, intermediate      number of experts, experts per token, an expert's width
      router_bias                     True: the router has a bias
      names                           {"router", "router_bias", "expert": a pattern with {e} and {p}} where p is one of
                                      gate, up, down
      shared                          None, or the params of a feed-forward part that every token also goes through
      shared_kind                     that part's kind ("swiglu" by default)
      shared_gate                     None, or the tensor name of a [1, D] matrix: the shared output times sigmoid(w . h)
      scoring                         "chosen" (softmax over the chosen logits, the default), "all" (see above;
                                      names["correction"] is then the correction, `scale` the constant) or
                                      "sigmoid_groups" (`groups` = {"count", "keep"}; `scale` the constant)
      identity                        experts behind the `experts` real ones that hand their input on (router rows
                                      experts .. experts + identity - 1)
      expert_form                     "swiglu" (default) or "gelu" (names' p is then one of up, down)
    """

    capturable = True
    ROUTE_BY_PRODUCT = 256  # tokens from which the router's logits are a library product

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.inter = int(params["intermediate"])
        self.names = dict(params["names"])
        self.has_bias = bool(params.get("router_bias", False))
        self.identity = int(params.get("identity") or 0)
        self.routed = self.experts + self.identity  # rows of the router
        self.all_scores = (params.get("scoring") or "chosen") in ("all", "sigmoid_groups")
        if params.get("scoring") not in (None, "chosen", "all", "sigmoid_groups"):
            raise ValueError(f"routed feed-forward: scoring {params.get('scoring')!r} is none of 'chosen', 'all', 'sigmoid_groups'")
        self.groups = None
        if params.get("scoring") == "sigmoid_groups":
            groups = params.get("groups") or {"count": 1, "keep": 1}
            self.groups = (int(groups["count"]), int(groups["keep"]))
            count, keep = self.groups
            if count < 1 or self.experts % count or not 1 <= keep <= count or int(params.get("identity") or 0):
                raise ValueError(f"routed feed-forward: {self.experts} experts in {count} groups of which {keep} are kept")
            if int(params["top"]) > keep * (self.experts // count):
                raise ValueError(f"routed feed-forward: top {params['top']} exceeds the experts of {keep} groups")
        self.scale = float(params.get("scale", 1.0))
        self.gelu = (params.get("expert_form") or "swiglu") == "gelu"
        if params.get("expert_form") not in (None, "swiglu", "gelu"):
            raise ValueError(f"routed feed-forward: expert form {params.get('expert_form')!r}")
        if self.all_scores and self.has_bias:
            raise ValueError("routed feed-forward: scores over all experts take a correction, not a router bias")
        if not self.all_scores and (self.scale != 1.0 or self.identity):
            raise ValueError("routed feed-forward: a weight scale or identity experts need scoring 'all'")
        if not 1 <= self.top <= min(self.routed, 32):
            raise ValueError(f"routed feed-forward: top {self.top} of {self.routed} experts (at most 32)")
        self.shared = build_part("feed_forward", PartSpec(params.get("shared_kind") or "swiglu", dict(params["shared"])), ctx) \
            if params.get("shared") else None
        self.shared_gate_name = params.get("shared_gate") if self.shared is not None else None
        self.router: Optional[torch.Tensor] = None
        self.router_bias: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def _expert(self, e: int, p: str) -> str:
        return self.names["expert"].format(e=e, p=p)

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        specs = [WeightSpec(self.names["router"], (self.routed, D), kind="vector", init="normal")]
        if self.has_bias:
            specs.append(WeightSpec(self.names["router_bias"], (self.experts,), kind="vector", init="normal"))
        if self.all_scores and self.names.get("correction"):
            specs.append(WeightSpec(self.names["correction"], (self.routed,), kind="vector", init="normal"))
        for e in range(self.experts):
            if not self.gelu:
                specs.append(WeightSpec(self._expert(e, "gate"), (self.inter, D)))
            specs += [WeightSpec(self._expert(e, "up"), (self.inter, D)), WeightSpec(self._expert(e, "down"), (D, self.inter))]
        if self.shared_gate_name:
            specs.append(WeightSpec(self.shared_gate_name, (1, D), kind="vector", init="normal"))
        return specs + (self.shared.weight_specs() if self.shared is not None else [])

    def sub_parts(self):
        return [self.shared] if self.shared is not None else []

    def bind(self, store) -> None:
        self.router = store.take(self.names["router"])  # float32: the logits are 32-bit whatever the run's dtype
        if self.shared_gate_name:  # the shared expert's gate: one more row behind the experts'
            self.router = torch.cat([self.router, store.take(self.shared_gate_name).float()], dim=0).contiguous()
        self.router_bias = store.take(self.names["router_bias"]) if self.has_bias else None
        if self.all_scores and self.names.get("correction"):
            self.router_bias = store.take(self.names["correction"])  # corrects the choice, not the logits
        act = self.ctx.act_dtype
        gate_up, down = [], []
        for e in range(self.experts):
            up = store.take(self._expert(e, "up")).to(act)
            gate_up.append(up if self.gelu else torch.cat([store.take(self._expert(e, "gate")).to(act), up]))
            down.append(store.take(self._expert(e, "down")).to(act))
        self.gate_up = torch.stack(gate_up).contiguous()
        self.down = torch.stack(down).contiguous()
        if self.shared is not None:
            self.shared.bind(store)

    def parameter_bytes(self) -> int:
        """What a step reads at most: the router, `top` experts a token (a large batch touches them all) and the
        shared expert."""
        size = self.gate_up.element_size()
        per_expert = (self.gate_up.shape[1] * self.gate_up.shape[2] + self.down.shape[1] * self.down.shape[2]) * size
        return (self.router.numel() * 4 + self.experts * per_expert
                + (self.shared.parameter_bytes() if self.shared is not None else 0))

    def _plan(self, step, n_pairs: int, mma: bool) -> K.MoePlan:
        rows = K.moe_tile_rows(mma, n_pairs, self.routed)
        tiles = K.moe_max_tiles(n_pairs, self.routed, rows)
        ws = step.ws
        return K.MoePlan(ws.buffer("moe.order", (n_pairs,), torch.int32), ws.buffer("moe.offsets", (self.routed + 1,), torch.int32),
                         ws.buffer("moe.tile_expert", (tiles,), torch.int32), ws.buffer("moe.tile_row0", (tiles,), torch.int32),
                         ws.buffer("moe.n_tiles", (1,), torch.int32), rows, mma)

    def forward(self, step, h, into=None):
        T, D = h.shape
        ws = step.ws
        act = self.ctx.act_dtype
        n_pairs = T * self.top
        chosen = ws.buffer("moe.chosen", (T, self.top), torch.int32)
        weight = ws.buffer("moe.weight", (T, self.top), torch.float32)
        logits = None
        if T > self.ROUTE_BY_PRODUCT:
            # many tokens: the logits as one library product in float32 (the rows widened first); few: in the kernel
            if torch.backends.cuda.matmul.allow_tf32:
                raise RuntimeError("routed feed-forward: TF32 is enabled; the router's logits need true 32-bit products")
            wide = h
            if h.dtype != torch.float32:
                wide = ws.buffer("moe.h32", (T, D), torch.float32)
                K.cast(h, wide)
            logits = ws.buffer("moe.logits", (T, self.router.shape[0]), torch.float32)
            torch.mm(wide, self.router.t(), out=logits)
        shared_gate = ws.buffer("moe.shared_gate", (T,), torch.float32) if self.shared_gate_name else None
        K.moe_route(h, self.router, self.router_bias, chosen, weight, self.top, logits=logits, all_scores=self.all_scores,
                    scale=self.scale, gate_out=shared_gate, groups=self.groups)
        # bfloat16: tiles of 64 rows on tensor cores at every size - with few rows per expert the products stream each
        # touched expert's weights once, and a mostly empty tile costs nothing that memory does not hide
        mma = K.USE_TENSOR_CORE_MOE and K.moe_mma_supported(act, D, self.inter)
        plan = self._plan(step, n_pairs, mma)
        K.moe_sort(chosen, plan, self.routed, n_real=self.experts)
        hidden = ws.buffer("moe.act", (n_pairs, self.inter), act)
        K.moe_gate_up(h, self.gate_up, hidden, plan, self.top, form=K.EXPERT_GELU if self.gelu else K.EXPERT_SWIGLU,
                      n_experts=self.routed)
        y = ws.buffer("moe.y", (n_pairs, D), torch.float32)
        K.moe_down(hidden, self.down, y, weight, plan, self.top, n_experts=self.routed)
        shared = self.shared.forward(step, h) if self.shared is not None else None
        out = ws.buffer("moe.out", (T, D), act)
        if self.identity:
            K.moe_combine(y, shared, out, self.top, chosen=chosen, pair_weight=weight, h=h, n_real=self.experts,
                          other_gate=shared_gate)
        else:
            K.moe_combine(y, shared, out, self.top, other_gate=shared_gate)
        return out


register_part("feed_forward", "routed", RoutedFeedForward)
