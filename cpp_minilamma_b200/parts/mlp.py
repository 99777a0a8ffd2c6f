"""Dense SwiGLU feed-forward: down( silu(gate(h)) * up(h) ).

The reference's FfnForward (src/forward.cc:313-322) with SiLU as x / (1 + exp(-x))
(src/ops.cc:135-151).  The gate and up matrices are fused at bind time into one
[2I, D] matrix so that one product feeds the activation kernel; when I is a multiple of
8 their rows are interleaved in blocks of 8 (gate rows 0-7, up rows 0-7, gate rows
8-15, ...), which puts a gate value and its up value into the same thread of a
tensor-core accumulator tile.  With biases (not in the reference) the form is
down( silu(gate(h) + b_g) * (up(h) + b_u) ) + b_d: the gate and up biases are added in float32 inside the activation
kernel, in the fused matrix's row order.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, FeedForward, PreNormed, WeightSpec, register_part
from .linear import Linear

INTERLEAVE = 8


def fuse_gate_up(gate: torch.Tensor, up: torch.Tensor):
    """Return (fused [2I, D], block) with block = INTERLEAVE, or 0 for plain halves."""
    inter, width = gate.shape
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    if inter % INTERLEAVE:
        return torch.cat([gate, up], dim=0).contiguous(), 0
    fused = torch.stack([gate.view(inter // INTERLEAVE, INTERLEAVE, width),
                         up.view(inter // INTERLEAVE, INTERLEAVE, width)], dim=1)
    return fused.reshape(2 * inter, width).contiguous(), INTERLEAVE


class SwiGLUFeedForward(FeedForward):
    """params: intermediate, names {"gate","up","down"} (tensor name stems, ".weight" is appended; with
    `bare_names` they are the tensor names themselves); bias_names {"gate","up","down"}: tensor names of the three
    biases, or None for a feed-forward without biases; out_name: workspace name of the result (default "down")."""

    capturable = True
    takes_prenormed = True  # the gate/up product may read rows whose norm it finishes itself
    adds_residual = True    # the down product may add to the residual stream and prepare the next norm

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.inter = int(params["intermediate"])
        suffix = "" if params.get("bare_names") else ".weight"
        self.names = {k: v + suffix for k, v in dict(params["names"]).items()}
        self.bias_names = dict(params["bias_names"]) if params.get("bias_names") else None
        self.out_name = params.get("out_name") or "down"
        if self.bias_names:  # the products that fold norms away know no bias: this instance takes plain rows
            self.takes_prenormed = self.adds_residual = False
        self.gate_up_bias = self.down_bias = None
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.block = 0

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        specs = [WeightSpec(self.names["gate"], (self.inter, D)),
                 WeightSpec(self.names["up"], (self.inter, D)),
                 WeightSpec(self.names["down"], (D, self.inter))]
        if self.bias_names:
            specs += [WeightSpec(self.bias_names["gate"], (self.inter,), kind="vector"),
                      WeightSpec(self.bias_names["up"], (self.inter,), kind="vector"),
                      WeightSpec(self.bias_names["down"], (D,), kind="vector")]
        return specs

    def bind(self, store) -> None:
        if self.bias_names:
            # the two biases in the fused matrix's row order (as columns [inter, 1] they interleave like its rows)
            fused_bias, _ = fuse_gate_up(store.take(self.bias_names["gate"]).float().view(-1, 1),
                                         store.take(self.bias_names["up"]).float().view(-1, 1))
            self.gate_up_bias = fused_bias.view(-1).contiguous()
            self.down_bias = store.take(self.bias_names["down"]).float().contiguous()
        fused, self.block = fuse_gate_up(store.take(self.names["gate"]), store.take(self.names["up"]))
        self.gate_up = Linear(fused, self.names["gate"] + "+up")
        self.down = Linear(store.take(self.names["down"]), self.names["down"])

    def parameter_bytes(self) -> int:
        return self.gate_up.parameter_bytes() + self.down.parameter_bytes()

    def forward(self, step, h, into=None):
        if self.gate_up_bias is not None:
            gu = self.gate_up.forward(step, h, "gu")
            act = step.ws.buffer("act", (h.shape[0], self.inter), gu.dtype)
            K.swiglu(gu, act, self.block, bias=self.gate_up_bias)
            out = self.down.forward(step, act, self.out_name)
            K.add_bias(out, self.down_bias)
            return out
        values, row_norm = (h.values, K.RowNorm(h.sumsq, h.partials, h.eps)) if isinstance(h, PreNormed) else (h, None)
        rows = values.shape[0]
        w = self.gate_up.weight
        fused = (rows <= step.small_rows and self.block == INTERLEAVE and w.dtype == torch.bfloat16
                 and values.dtype == torch.bfloat16
                 and bool(K.small_linear_kind(rows, 2 * self.inter, w.shape[1], K.EPI_SWIGLU)))
        if fused:
            # few rows: one weight-streaming kernel whose epilogue applies the activation
            act = step.ws.buffer("act", (rows, self.inter), torch.bfloat16)
            K.small_linear(values, w, None, act, K.EPI_SWIGLU, row_norm)
        elif (row_norm is not None and w.dtype == torch.bfloat16 and self.inter % 8 == 0
              and not K.small_linear_kind(rows, 2 * self.inter, w.shape[1], K.EPI_BF16)):
            # the library product cannot finish the norm in front of it: it runs on the rows as they are and
            # the activation kernel multiplies gate and up by the rows' factors
            gu = self.gate_up.forward(step, values, "gu")
            act = step.ws.buffer("act", (rows, self.inter), torch.bfloat16)
            K.swiglu(gu, act, self.block, row_norm, w.shape[1])
        else:
            gu = self.gate_up.forward(step, h, "gu")
            act = step.ws.buffer("act", (rows, self.inter), gu.dtype)
            K.swiglu(gu, act, self.block)
        return self.down.forward(step, act, self.out_name, into=into)


class GeluFeedForward(FeedForward):
    """down(act(up(h))) without a gate: act is gelu in its erf form, 0.5 z (1 + erf(z / sqrt 2)), or in its tanh form.
    params: intermediate, names {"up","down"} (tensor names), activation ("gelu_erf" default, or "gelu_tanh"),
    out_name (workspace name of the result, default "down")."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.inter = int(params["intermediate"])
        self.names = dict(params["names"])
        kinds = {"gelu_erf": K.ACT_GELU_ERF, "gelu_tanh": K.ACT_GELU_TANH}
        name = params.get("activation") or "gelu_erf"
        if name not in kinds:
            raise ValueError(f"feed-forward: activation {name!r} is not one of {sorted(kinds)}")
        self.act = kinds[name]
        self.out_name = params.get("out_name") or "down"
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        return [WeightSpec(self.names["up"], (self.inter, D)), WeightSpec(self.names["down"], (D, self.inter))]

    def bind(self, store) -> None:
        self.up = Linear(store.take(self.names["up"]), self.names["up"])
        self.down = Linear(store.take(self.names["down"]), self.names["down"])

    def parameter_bytes(self) -> int:
        return self.up.parameter_bytes() + self.down.parameter_bytes()

    def forward(self, step, h, into=None):
        u = self.up.forward(step, h, "up")
        K.activation(u, u, self.act)
        return self.down.forward(step, u, self.out_name)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward: contributes nothing (blocks that add two outputs skip a None)."""

    capturable = True

    def forward(self, step, h, into=None):
        return None


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
register_part("feed_forward", "gelu_mlp", GeluFeedForward)
register_part("feed_forward", "none", NoFeedForward)
