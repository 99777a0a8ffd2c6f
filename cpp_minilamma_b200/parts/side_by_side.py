"""Two mixers side by side: both read the same rows, their results are added with a weight each.

    out = scale_left * left(h) + scale_right * right(h)

`left` and `right` are any two registered mixers (attention beside a recurrent layer, say); each keeps what it
needs in the cache - one of them keys and values, the other a fixed-size state, or either both - and the pair asks the
cache for the union.  Nothing is added here: the pair hands both results on as a `PendingSum` with the two
weights, and the norm kernel that reads the residual stream next forms the weighted sum in float32 on its way in.
"""
from __future__ import annotations

from typing import List

from .base import BuildContext, CacheNeed, Mixer, PartSpec, PendingSum, StateNeed, WeightSpec, build_part, register_part


class SideBySideMixer(Mixer):
    """params: left, right (PartSpecs of two mixers; their results must live in different workspace buffers),
    scale_left, scale_right."""

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.left: Mixer = build_part("mixer", _as_spec(params["left"]), ctx)
        self.right: Mixer = build_part("mixer", _as_spec(params["right"]), ctx)
        self.scale_left = float(params.get("scale_left", 1.0))
        self.scale_right = float(params.get("scale_right", 1.0))
        self.capturable = self.left.capturable and self.right.capturable
        left, right = self.left.cache_need(), self.right.cache_need()
        if left.kv is not None and right.kv is not None:
            raise ValueError("side-by-side mixers: only one of the two may keep keys and values")
        names = [item[0] for need in (left, right) if need.state is not None for item in need.state.tensors]
        if len(set(names)) != len(names):
            raise ValueError(f"side-by-side mixers: both keep a state called {sorted(names)}")

    def sub_parts(self):
        """The two mixers: whoever collects the parts' index arrays and launch parameters asks them directly."""
        return [self.left, self.right]

    def weight_specs(self) -> List[WeightSpec]:
        return self.left.weight_specs() + self.right.weight_specs()

    def bind(self, store) -> None:
        self.left.bind(store)
        self.right.bind(store)

    def parameter_bytes(self) -> int:
        return self.left.parameter_bytes() + self.right.parameter_bytes()

    def cache_need(self) -> CacheNeed:
        left, right = self.left.cache_need(), self.right.cache_need()
        tensors = tuple(item for need in (left, right) if need.state is not None for item in need.state.tensors)
        return CacheNeed(kv=left.kv if left.kv is not None else right.kv, state=StateNeed(tensors) if tensors else None)

    def forward(self, step, h, cache):
        first = self.left.forward(step, h, cache)
        second = self.right.forward(step, h, cache)
        if first.data_ptr() == second.data_ptr():
            raise RuntimeError("side-by-side mixers: both results live in the same workspace buffer (give one an out_name)")
        return PendingSum(first, second, self.scale_left, self.scale_right)


def _as_spec(spec) -> PartSpec:
    return spec if isinstance(spec, PartSpec) else PartSpec(spec["kind"], dict(spec["params"]))


register_part("mixer", "side_by_side", SideBySideMixer)
