"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

`pre_norm` is the reference's layer (src/forward.cc:385-414):
    r = x + mixer(norm_in(x));   x' = r + feed_forward(norm_post(r))
With `residual_mult` m (not in the reference) both outputs join the stream times m:  r = x + m mixer(..),
x' = r + m feed_forward(..); a layer without a feed-forward ends at r.
`parallel` (not in the reference) lets mixer and feed-forward read one norm:
    h = norm(x);   x' = x + mixer(h) + feed_forward(h)
`sandwich` (not in the reference) puts a norm behind each sub-layer as well as in front of it:
    r = x + norm_mo(mixer(norm_in(x)));   x' = r + norm_fo(feed_forward(norm_pf(r)))
The residual adds are not separate kernels: a part's output stays "pending" until the
next norm, which adds it to the float32 residual and normalises in one pass.  Where the parts on both
sides of a norm offer it, the norm is no kernel either: the part before adds to the residual stream
itself and hands on a `PreNormed`, which the part behind reads (small decode batches).
"""
from __future__ import annotations

from typing import List

from .mlp import NoFeedForward
from .base import Block, NormedDelta, PendingSum, ResidualTarget, ScaledDelta, register_part


def _offer(x, norm, writer, reader):
    """The ResidualTarget that lets `writer` fold `norm` away for `reader`, or None."""
    if norm is None or not writer.adds_residual or not reader.takes_prenormed or norm.prenorm_weight() is None:
        return None
    return ResidualTarget(x, norm)


class PreNormBlock(Block):
    """params: residual_mult (default 1): the factor on both sub-layers' outputs where they join the stream."""

    capturable = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.mult = float(params.get("residual_mult", 1.0))

    def norm_names(self) -> List[str]:
        return ["input", "post_mixer"]

    def first_reader(self, layer):
        # a factor on the outputs is applied by the norm kernel that adds them: no norm is folded away then
        return (layer.norms["input"], layer.mixer) if layer.mixer.takes_prenormed and self.mult == 1.0 else None

    def forward(self, step, x, pending, layer, cache, next_reader=None):
        h = layer.norms["input"].forward(step, x, pending)
        post = layer.norms["post_mixer"]
        if self.mult != 1.0 or isinstance(layer.feed_forward, NoFeedForward):
            mixed = layer.mixer.forward(step, h, cache)
            mixed = ScaledDelta(mixed, self.mult) if self.mult != 1.0 else mixed
            if isinstance(layer.feed_forward, NoFeedForward):
                return mixed
            fed = layer.feed_forward.forward(step, post.forward(step, x, mixed))
            return ScaledDelta(fed, self.mult) if self.mult != 1.0 else fed
        into = _offer(x, post, layer.mixer, layer.feed_forward)
        mixed = layer.mixer.forward(step, h, cache, into=into) if into else layer.mixer.forward(step, h, cache)
        h = post.forward(step, x, mixed)
        into = _offer(x, next_reader[0], layer.feed_forward, next_reader[1]) if next_reader else None
        return layer.feed_forward.forward(step, h, into=into) if into else layer.feed_forward.forward(step, h)


class ParallelBlock(Block):
    """One norm, two readers:   h = norm(x);  x' = x + mixer(h) + feed_forward(h).
    Both outputs stay pending; the next norm adds their sum to the float32 stream.  A layer without a
    feed-forward (kind "none") leaves the mixer's output alone."""

    capturable = True

    def norm_names(self) -> List[str]:
        return ["input"]

    def forward(self, step, x, pending, layer, cache):
        h = layer.norms["input"].forward(step, x, pending)
        mixed = layer.mixer.forward(step, h, cache)
        fed = layer.feed_forward.forward(step, h)
        return mixed if fed is None else PendingSum(mixed, fed)


class SandwichBlock(Block):
    """Norms "input" and "mixer_out" around the mixer, "pre_ff" and "ff_out" around the feed-forward.  A sub-layer's
    output stays pending together with the norm behind it (`NormedDelta`): the norm that reads the stream next
    normalises the output, adds it and normalises the sum in one kernel.  A layer without a feed-forward ends behind
    "mixer_out"."""

    capturable = True

    def norm_names(self) -> List[str]:
        return ["input", "mixer_out", "pre_ff", "ff_out"]

    def forward(self, step, x, pending, layer, cache):
        h = layer.norms["input"].forward(step, x, pending)
        mixed = NormedDelta(layer.mixer.forward(step, h, cache), layer.norms["mixer_out"])
        if isinstance(layer.feed_forward, NoFeedForward):
            return mixed
        h = layer.norms["pre_ff"].forward(step, x, mixed)
        return NormedDelta(layer.feed_forward.forward(step, h), layer.norms["ff_out"])


register_part("block", "sandwich", SandwichBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
