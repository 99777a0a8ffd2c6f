"""RMSNorm and layer norm, each fused with the residual add that precedes it.

y_i = x_i * w_i / sqrt(mean_j(x_j^2) + eps): eps inside the root, the weight multiplies
(no 1 + w), no bias - src/ops.cc:95-110.  The residual stream x is float32; the add of
the previous part's output and the norm are one kernel.

`rms_norm` with `offset` (not in the reference): the weight is stored around zero and applied as 1 + w.  The factor is
formed once, in float32, when the weights are bound, so the kernels are the same.  A delta that passes a norm of its
own before it joins the stream (`NormedDelta`: blocks whose sub-layers end in a norm) is normalised, added and the
stream normalised again in the one kernel.

`layer_norm` (not in the reference): y_i = (x_i - mean) / sqrt(var + eps) * w_i + b_i with var the mean of the
squared deviations; weight and bias are tensors of their own.  It has no factor that the products around it could
apply, so it is never folded away (`prenorm_weight` stays None).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, Norm, NormedDelta, PendingSum, PreNormed, ScaledDelta, WeightSpec, register_part


def _delta_parts(delta):
    """(first, second, DeltaNorm or None) of whatever a block left pending."""
    norm = None
    if isinstance(delta, NormedDelta):
        norm = delta.norm
        if not isinstance(norm, RMSNorm):
            raise RuntimeError("a delta can only pass a norm of the RMS form on its way into the stream")
        delta = delta.delta
    first, second, s1, s2 = delta, None, 1.0, 1.0
    if isinstance(delta, ScaledDelta):
        first, s1 = delta.delta, delta.scale
    elif isinstance(delta, PendingSum):
        first, second, s1, s2 = delta.first, delta.second, delta.scale_first, delta.scale_second
    if norm is None and s1 == 1.0 and s2 == 1.0:
        return first, second, None
    return first, second, K.DeltaNorm(norm.weight if norm is not None else None, norm.eps if norm is not None else 0.0, s1, s2)


class RMSNorm(Norm):
    """params: width, eps, name (tensor name of the weight); offset (True: the stored weight w stands for 1 + w);
    optional (True: a folder may leave the tensor out)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = params["name"]
        self.offset = bool(params.get("offset", False))
        self.optional = bool(params.get("optional", False))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        # around zero when 1 is added, around one otherwise; left out of a folder it stands for the plain norm
        return [WeightSpec(self.name, (self.width,), kind="vector", init="normal" if self.offset else "norm",
                           optional=self.optional)]

    def bind(self, store) -> None:
        self.weight = store.take(self.name)
        if self.offset:
            self.weight = (self.weight.float() + 1.0).contiguous()  # float32(1 + w): what x / rms is multiplied by

    def parameter_bytes(self) -> int:
        return self.width * 4

    def prenorm_weight(self):
        return self.weight, self.eps

    def forward(self, step, x, delta, rows=None, out_name: str = "h"):
        if isinstance(delta, PreNormed):
            if delta.norm is not self or rows is not None:
                raise RuntimeError(f"{self.name}: given rows that were prepared for another norm")
            return delta  # x is up to date; the product that reads the rows applies the factor
        n = x.shape[0] if rows is None else rows.shape[0]
        out = step.ws.buffer(out_name, (n, self.width), self.ctx.act_dtype)
        first, second, delta_norm = _delta_parts(delta)
        K.add_rmsnorm(x, first, self.weight, out, self.eps, rows, delta2=second, delta_norm=delta_norm)
        return out

    def forward_in_place(self, x) -> None:
        """x <- norm(x) on the float32 stream itself (a norm that sits on the stream, not beside it)."""
        K.add_rmsnorm(x, None, self.weight, x, self.eps)


class LayerNorm(Norm):
    """params: width, eps, name (tensor name of the weight), bias (tensor name of the bias, or None for none),
    optional (True: a folder may leave both tensors out)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = params["name"]
        self.bias_name = params.get("bias")
        self.optional = bool(params.get("optional", False))  # a folder may leave the tensors out (a norm nothing reads)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.name, (self.width,), kind="vector", init="norm", optional=self.optional)]
        if self.bias_name:
            specs.append(WeightSpec(self.bias_name, (self.width,), kind="vector", init="normal", optional=self.optional))
        return specs

    def bind(self, store) -> None:
        self.weight = store.take(self.name)
        self.bias = store.take(self.bias_name) if self.bias_name else None

    def parameter_bytes(self) -> int:
        return self.width * (8 if self.bias_name else 4)

    def forward(self, step, x, delta, rows=None, out_name: str = "h"):
        if isinstance(delta, PreNormed):
            raise RuntimeError(f"{self.name}: a layer norm cannot finish rows that were prepared for another norm")
        n = x.shape[0] if rows is None else rows.shape[0]
        out = step.ws.buffer(out_name, (n, self.width), self.ctx.act_dtype)
        if isinstance(delta, (NormedDelta, ScaledDelta)) or (isinstance(delta, PendingSum) and (delta.scale_first != 1.0 or delta.scale_second != 1.0)):
            raise RuntimeError(f"{self.name}: a layer norm adds its delta as it is (no norm or factor on the way in)")
        if isinstance(delta, PendingSum):
            # two parts that read one norm: add the first to the stream here, the second with the norm
            K.add_layernorm(x, delta.first, self.weight, self.bias, out, self.eps, rows)
            if rows is not None:
                raise RuntimeError(f"{self.name}: two pending outputs cannot be added to gathered rows")
            delta = delta.second
        K.add_layernorm(x, delta, self.weight, self.bias, out, self.eps, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
