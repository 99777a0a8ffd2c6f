"""The Badolix decoder as data: `BadolixConfig` -> `ModelSpec`.

A scaled token embedding; pre-norm layers whose outputs join the stream times a constant; three kinds of mixer -
grouped-query attention under a sliding window that keeps the sequence's first tokens, with capped scores, rotate-half
positions at divided frequencies and, for some layers, the keys and values of an earlier layer; attention over a shared
low-rank latent with one rotated key part for all heads (frequencies under a ramp); a state-space mixer (short
convolution, one decay per token and head, a gate in front of a norm in equal parts) - and a feed-forward that is dense
with biases or routes every token through a few small experts chosen by sigmoid scores inside the best groups; a final
norm and a head that is the embedding table, times a constant.  This file is the only one that knows Badolix's tensor
names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.{gate, up, down}(.b)`,
`l<i>.mlp.{router, e<k>.*}`, `final.norm`.
"""
from __future__ import annotations

from ..config.badolix import BadolixConfig, BadolixLayer
from ..config.base import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _position(rot):
    if rot is None or not rot.dims:
        return None, 0
    return PartSpec("rotary", {"head_dim": rot.dims, "theta": rot.base, "scaling": rot.part_scaling(),
                               "interleaved": False}), rot.dims


def _mixer(config: BadolixConfig, index: int, eps: float) -> PartSpec:
    layer: BadolixLayer = config.layers[index]
    pre = f"l{index}.mix."
    position, rot_dims = _position(layer.rot)
    if layer.type == "latent_attention":
        names = {p: pre + p for p in ("q", "dkv", "uk", "uv", "o")}
        names["dkv_norm"] = pre + "dkv.norm"
        return PartSpec("latent_attention", {
            "n_heads": layer.heads, "head_dim": layer.dim, "rot_dim": layer.rot_dim, "v_head_dim": layer.vdim,
            "kv_rank": layer.kv_rank, "scale": layer.scale, "position": position, "eps": eps, "gate": False,
            "names": names})
    if layer.type == "mamba2":
        names = {p: pre + p for p in ("in", "conv", "dt_bias", "A_log", "D", "norm", "o")}
        names["conv_bias"] = pre + "conv.b"
        return PartSpec("state_space", {
            "n_heads": layer.heads, "n_groups": layer.groups, "v_head_dim": layer.vdim, "state": layer.state,
            "conv": layer.conv, "norm_groups": layer.norm_groups, "eps": eps, "names": names})
    shared = layer.kv_from is not None
    # what the cache must keep: the widest reach among this layer and the layers that read its keys and values
    readers = [layer] + [other for other in config.layers if other.kv_from == index]
    cache_window = 0 if any(r.window == 0 for r in readers) else max(r.window for r in readers)
    cache_keep = max(r.keep_first for r in readers) if cache_window else 0
    return PartSpec("chunked_attention", {
        "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "v_head_dim": layer.vdim,
        "scale": layer.scale, "chunk": 0, "window": layer.window, "keep_first": layer.keep_first,
        "softcap": layer.softcap, "position": position, "rotary_dims": rot_dims, "qk_norm": None,
        "kv_shared": shared, "cache_window": cache_window, "cache_keep_first": cache_keep,
        "names": {p: pre + p for p in (("q", "o") if shared else ("q", "k", "v", "o"))}})


def _feed_forward(layer: BadolixLayer, prefix: str) -> PartSpec:
    mlp = layer.mlp
    if mlp is None:
        return PartSpec("none")
    pre = prefix + "mlp."
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"intermediate": mlp.ff, "bare_names": True,
                                   "names": {p: pre + p for p in ("gate", "up", "down")},
                                   "bias_names": {p: pre + p + ".b" for p in ("gate", "up", "down")}})
    return PartSpec("routed", {
        "experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff, "scoring": "sigmoid_groups",
        "groups": {"count": mlp.group_count, "keep": mlp.group_keep}, "shared": None,
        "names": {"router": pre + "router", "expert": pre + "e{e}.{p}"}})


def build_badolix_spec(config: BadolixConfig) -> ModelSpec:
    def norm(name, optional=False):
        return PartSpec("rms_norm", {"width": config.width, "eps": config.eps, "name": name, "optional": optional})

    layers, schedule = [], []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        layers.append(LayerSpec(block=PartSpec("pre_norm", {"residual_mult": config.residual_mult}),
                                mixer=_mixer(config, i, config.eps), feed_forward=_feed_forward(layer, prefix),
                                norms={"input": norm(prefix + "norm1"),
                                       # nothing reads the second norm of a layer without a feed-forward
                                       "post_mixer": norm(prefix + "norm2", optional=layer.mlp is None)}))
        schedule.append(ScheduleEntry(i, cache_of=layer.kv_from))
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "name": "embed", "scale": config.embed_scale}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab": config.vocab, "name": "head", "tied_to": "embed",
                                         "scale": config.logit_scale}))


register_architecture("Badolix", BadolixConfig, build_badolix_spec)
