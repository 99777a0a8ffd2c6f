"""The Sopanex decoder as data: `SopanexConfig` -> `ModelSpec`.

A scaled token embedding plus a row of a hashed table of (previous token, token) pairs; layers with an RMS norm
(weight stored around zero) in front of and behind each sub-layer; a mixer made of two that read the same rows -
grouped-query attention whose values are its unrotated keys, with rotate-half positions under a ramp over the pair
index, a learned sink in the softmax and a gate per head, beside gated linear attention with a decay per key channel
and a fixed-size state - and a feed-forward that routes every token through a few small gelu experts, some of which
only hand their input on, beside a gated shared expert; a final norm and an untied head.  This file is the only one that knows
Sopanex's tensor names: `embed`, `bigram`, `l<i>.norm1(b)`, `l<i>.norm2(b)`, `l<i>.mix.{left,right}.*`,
`l<i>.mlp.{router, correction, e<k>.*, shared.*}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.sopanex import SopanexConfig, SopanexLayer
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(layer: SopanexLayer, prefix: str, eps: float) -> PartSpec:
    left, right = layer.left, layer.right
    lp, rp = prefix + "mix.left.", prefix + "mix.right."
    position, rot_dims = None, 0
    if left.rot is not None and left.rot.dims:
        rot_dims = left.rot.dims
        scaling = dict(left.rot.scaling, type="yarn") if left.rot.scaling else None
        position = PartSpec("rotary", {"head_dim": rot_dims, "theta": left.rot.base, "scaling": scaling,
                                       "interleaved": False})
    attention = PartSpec("chunked_attention", {
        "n_heads": left.heads, "n_kv_heads": left.kv_heads, "head_dim": left.dim, "v_head_dim": left.vdim,
        "scale": left.scale, "chunk": 0, "window": 0, "position": position, "rotary_dims": rot_dims, "qk_norm": None,
        "sink": lp + "sink", "values": "keys", "gate": "head", "out_name": "o.left",
        "names": {p: lp + p for p in ("q", "k", "g", "o")}})
    names = {p: rp + p for p in ("q", "k", "v", "g", "a1", "a2", "norm", "o")}
    names["a2_bias"] = rp + "a2.b"
    linear = PartSpec("gated_linear_attention", {
        "n_heads": right.heads, "head_dim": right.dim, "v_head_dim": right.vdim, "tau": right.tau, "eps": eps,
        "decay_rank": right.decay_rank or -1, "out_name": "o.right", "names": names})
    return PartSpec("side_by_side", {"left": attention, "right": linear, "scale_left": layer.left_scale,
                                     "scale_right": layer.right_scale})


def _feed_forward(layer: SopanexLayer, prefix: str) -> PartSpec:
    mlp = layer.mlp
    if mlp is None:
        return PartSpec("none")
    pre = prefix + "mlp."
    shared = None
    if mlp.shared_ff:
        shared = {"intermediate": mlp.shared_ff, "names": {p: pre + "shared." + p for p in ("up", "down")},
                  "activation": "gelu_erf", "out_name": "shared.down"}
    return PartSpec("routed", {
        "experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff, "identity": mlp.identity, "scale": mlp.scale,
        "scoring": "all", "expert_form": "gelu", "shared": shared, "shared_kind": "gelu_mlp",
        "shared_gate": pre + "shared.sg" if shared else None,
        "names": {"router": pre + "router", "correction": pre + "correction", "expert": pre + "e{e}.{p}"}})


def build_sopanex_spec(config: SopanexConfig) -> ModelSpec:
    def norm(name, optional=False):
        return PartSpec("rms_norm", {"width": config.width, "eps": config.eps, "name": name, "offset": True,
                                     "optional": optional})

    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        bare = layer.mlp is None  # nothing reads the norms around a feed-forward that is not there
        layers.append(LayerSpec(block=PartSpec("sandwich"), mixer=_mixer(layer, prefix, config.eps),
                                feed_forward=_feed_forward(layer, prefix),
                                norms={"input": norm(prefix + "norm1"), "mixer_out": norm(prefix + "norm1b"),
                                       "pre_ff": norm(prefix + "norm2", optional=bare),
                                       "ff_out": norm(prefix + "norm2b", optional=bare)}))
    pairs = None
    if config.buckets:
        pairs = {"name": "bigram", "buckets": config.buckets, "mul_prev": config.mul_prev, "mul_cur": config.mul_cur}
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=config.max_positions,
        embedding=PartSpec("pair_hash_embedding", {"vocab": config.vocab, "name": "embed", "scale": config.embed_scale,
                                                   "pairs": pairs}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(config.layers))],
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab": config.vocab, "name": "head", "tied_to": None}))


register_architecture("Sopanex", SopanexConfig, build_sopanex_spec)
