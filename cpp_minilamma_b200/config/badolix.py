"""`BadolixConfig`: the configuration of the Badolix decoder, typed and checked.

A Badolix folder's config.json names the design in "architecture" and gives every size and constant:

    vocab, width, norm.eps, embedding.scale, residual_mult, logit_scale
    layers[i].type     "attention" | "latent_attention" | "mamba2"
    layers[i].mixer    attention:         heads, kv_heads, dim, vdim, scale, softcap, mask {size, keep_first},
                                          rot {base, dims, scaling {factor}}, kv_from (an earlier attention layer whose
                                          keys and values this layer reads instead of projecting its own)
                       latent_attention:  heads, dim, rot_dim, vdim, kv_rank, scale,
                                          rot {base, dims, scaling {factor, original, fast, slow}}
                       mamba2:            heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp      {"kind": "dense", "ff": n}, {"kind": "moe", "router": {experts, top, groups {count, keep}},
                       "expert": {ff}}, or null for a layer without a feed-forward

Nothing here knows tensor names or kernels; `models/badolix.py` turns the typed configuration into parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, take_float, take_int
from .kupirax import _object

MIXER_TYPES = ("attention", "latent_attention", "mamba2")


@dataclass
class ScaledRotation:
    """Rotary positions on the first `dims` dimensions of a head, pairs (i, i + dims / 2).  `scaling` is None, or
    {"factor"} (every frequency divided by it), or {"factor", "original", "fast", "slow"} (a ramp over the pair index
    between a frequency and that over `factor`, and a factor on cos and sin)."""

    base: float
    dims: int
    scaling: Optional[Dict[str, float]] = None

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["ScaledRotation"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        scaling = None
        if raw.get("scaling") is not None:
            sc = _object(raw["scaling"], what + ".scaling")
            scaling = {"factor": take_float(sc, "factor")}
            if any(key in sc for key in ("original", "fast", "slow")):
                scaling.update(original=take_float(sc, "original"), fast=take_float(sc, "fast"), slow=take_float(sc, "slow"))
            if min(scaling.values()) <= 0:
                raise ConfigError(f"config.json: {what}.scaling needs positive numbers")
        rot = cls(base=take_float(raw, "base"), dims=take_int(raw, "dims", minimum=0), scaling=scaling)
        if rot.dims % 2 or rot.base <= 0 or (rot.base == 1.0 and scaling and "original" in scaling):
            raise ConfigError(f"config.json: {what} needs an even 'dims' and a positive 'base' (not 1 under a ramp)")
        return rot

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling:
            out["scaling"] = dict(self.scaling)
            if "original" in self.scaling and float(self.scaling["original"]).is_integer():
                out["scaling"]["original"] = int(self.scaling["original"])
        return out

    def part_scaling(self) -> Optional[Dict[str, Any]]:
        """The `scaling` parameter of the rotary position encoding part."""
        if not self.scaling:
            return None
        return dict(self.scaling, type="yarn" if "original" in self.scaling else "linear")


@dataclass
class BadolixFeedForward:
    kind: str                 # "dense" or "moe"
    ff: int                   # the dense width, or an expert's
    experts: int = 0
    top: int = 0
    group_count: int = 1
    group_keep: int = 1

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["BadolixFeedForward"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        kind = raw.get("kind")
        if kind == "dense":
            return cls(kind="dense", ff=take_int(raw, "ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"config.json: {what}.kind {kind!r} is not supported (known: dense, moe)")
        router = _object(raw.get("router"), what + ".router")
        out = cls(kind="moe", ff=take_int(_object(raw.get("expert"), what + ".expert"), "ff", minimum=1),
                  experts=take_int(router, "experts", minimum=1), top=take_int(router, "top", minimum=1))
        if router.get("groups") is not None:
            groups = _object(router["groups"], what + ".router.groups")
            out.group_count = take_int(groups, "count", minimum=1)
            out.group_keep = take_int(groups, "keep", minimum=1)
        if out.experts % out.group_count or out.group_keep > out.group_count:
            raise ConfigError(f"config.json: {what}: {out.experts} experts in {out.group_count} groups, {out.group_keep} kept")
        if out.top > out.group_keep * (out.experts // out.group_count):
            raise ConfigError(f"config.json: {what}: top {out.top} exceeds the experts of {out.group_keep} groups")
        return out

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top,
                           "groups": {"count": self.group_count, "keep": self.group_keep}}}


@dataclass
class BadolixLayer:
    type: str
    heads: int
    vdim: int
    dim: int = 0                        # attention, latent_attention: the (plain) query/key size of a head
    kv_heads: int = 0                   # attention
    scale: float = 0.0                  # attention, latent_attention
    softcap: float = 0.0                # attention; 0: none
    window: int = 0                     # attention: mask.size; 0: plain causal
    keep_first: int = 0                 # attention: mask.keep_first
    kv_from: Optional[int] = None       # attention: the layer whose keys and values are read
    rot: Optional[ScaledRotation] = None
    rot_dim: int = 0                    # latent_attention
    kv_rank: int = 0                    # latent_attention
    state: int = 0                      # mamba2
    groups: int = 0                     # mamba2
    conv: int = 0                       # mamba2
    norm_groups: int = 1                # mamba2
    mlp: Optional[BadolixFeedForward] = None

    @classmethod
    def from_dict(cls, raw: Any, index: int) -> "BadolixLayer":
        what = f"layers[{index}]"
        raw = _object(raw, what)
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {what}.type {kind!r} is not one of {', '.join(MIXER_TYPES)}")
        m = _object(raw.get("mixer"), what + ".mixer")
        layer = cls(type=kind, heads=take_int(m, "heads", minimum=1), vdim=take_int(m, "vdim", minimum=1),
                    mlp=BadolixFeedForward.from_dict(raw.get("mlp"), what + ".mlp"))
        if kind == "mamba2":
            layer.state = take_int(m, "state", minimum=1)
            layer.groups = take_int(m, "groups", default=1, minimum=1)
            layer.conv = take_int(m, "conv", minimum=1)
            layer.norm_groups = take_int(m, "norm_groups", default=1, minimum=1)
            if layer.heads % layer.groups:
                raise ConfigError(f"config.json: {what}: {layer.heads} heads are not a multiple of {layer.groups} groups")
            if (layer.heads * layer.vdim) % layer.norm_groups:
                raise ConfigError(f"config.json: {what}: {layer.heads * layer.vdim} columns in {layer.norm_groups} norm groups")
            return layer
        layer.dim = take_int(m, "dim", minimum=1)
        layer.scale = take_float(m, "scale")
        layer.rot = ScaledRotation.from_dict(m.get("rot"), what + ".mixer.rot")
        if kind == "latent_attention":
            layer.rot_dim = take_int(m, "rot_dim", minimum=0)
            layer.kv_rank = take_int(m, "kv_rank", minimum=1)
            if layer.rot_dim % 2 or (layer.rot_dim and layer.rot is None):
                raise ConfigError(f"config.json: {what}: {layer.rot_dim} rotated dimensions need an even count and a 'rot'")
            if layer.rot is not None and layer.rot.dims != layer.rot_dim:
                raise ConfigError(f"config.json: {what}: rot.dims {layer.rot.dims} differs from rot_dim {layer.rot_dim}")
            return layer
        layer.kv_heads = take_int(m, "kv_heads", default=layer.heads, minimum=1)
        layer.softcap = take_float(m, "softcap", default=0.0)
        if m.get("mask") is not None:
            mask = _object(m["mask"], what + ".mixer.mask")
            layer.window = take_int(mask, "size", default=0, minimum=0)
            layer.keep_first = take_int(mask, "keep_first", default=0, minimum=0)
        if m.get("kv_from") is not None:
            layer.kv_from = take_int(m, "kv_from", minimum=0)
        if layer.heads % layer.kv_heads:
            raise ConfigError(f"config.json: {what}: {layer.heads} heads are not a multiple of {layer.kv_heads} kv_heads")
        if layer.rot is not None and layer.rot.dims > layer.dim:
            raise ConfigError(f"config.json: {what}: {layer.rot.dims} rotated dimensions of {layer.dim}")
        if layer.softcap < 0:
            raise ConfigError(f"config.json: {what}: softcap must not be negative")
        return layer

    def to_dict(self) -> Dict[str, Any]:
        if self.type == "mamba2":
            mixer: Dict[str, Any] = {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                                     "conv": self.conv, "norm_groups": self.norm_groups}
        elif self.type == "latent_attention":
            mixer = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                     "kv_rank": self.kv_rank, "scale": self.scale, "rot": self.rot.to_dict() if self.rot else None}
        else:
            mixer = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                     "scale": self.scale, "softcap": self.softcap, "rot": self.rot.to_dict() if self.rot else None,
                     "mask": {"size": self.window, "keep_first": self.keep_first} if self.window else None}
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass
class BadolixConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 1e-6
    embed_scale: float = 1.0
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    layers: List[BadolixLayer] = field(default_factory=list)
    max_positions: int = 1 << 20   # not part of the design: the most positions a sequence may have
    torch_dtype: str = "bfloat16"  # storage of a folder written from this configuration

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BadolixConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=take_int(raw, "vocab", minimum=1), width=take_int(raw, "width", minimum=1),
                     eps=take_float(_object(raw.get("norm"), "'norm'"), "eps"),
                     layers=[BadolixLayer.from_dict(l, i) for i, l in enumerate(layers)])
        config.embed_scale = take_float(_object(raw.get("embedding") or {}, "'embedding'"), "scale", default=1.0)
        config.residual_mult = take_float(raw, "residual_mult", default=1.0)
        config.logit_scale = take_float(raw, "logit_scale", default=1.0)
        config.max_positions = take_int(raw, "max_positions", default=cls.max_positions, minimum=1)
        config.torch_dtype = raw.get("torch_dtype", "bfloat16")
        return config

    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i, layer in enumerate(self.layers):
            if layer.kv_from is None:
                continue
            j = layer.kv_from
            if not 0 <= j < i or self.layers[j].type != "attention" or self.layers[j].kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from {j} must name an earlier attention layer with "
                                  "keys and values of its own")
            source = self.layers[j]
            if (source.kv_heads, source.dim, source.vdim) != (layer.kv_heads, layer.dim, layer.vdim):
                raise ConfigError(f"config.json: layers[{i}] reads the keys of layers[{j}], whose kv_heads, dim or vdim differ")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture or "Badolix", "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embed_scale},
                "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
                "layers": [l.to_dict() for l in self.layers],
                "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}
