"""`SopanexConfig`: the configuration of the Sopanex decoder, typed and checked.

A Sopanex folder's config.json names the design in "architecture" and gives every size and constant:

    vocab, width, norm.eps
    embedding          scale, bigram {buckets, mul_prev, mul_cur} (or null: no pair table)
    layers[i].type     "parallel": two mixers side by side
    layers[i].mixer    left_scale, right_scale,
                       left:  heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original, fast, slow}}
                       right: heads, dim, vdim, tau (the decay's inner size is the stored tensors'; "decay_rank" names
                              it where a folder of random weights is to be written)
    layers[i].mlp      {"kind": "moe", "router": {experts, top, identity, scale}, "expert": {ff}, "shared": {ff} or null},
                       or null for a layer without a feed-forward

Nothing here knows tensor names or kernels; `models/sopanex.py` turns the typed configuration into parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, take_float, take_int
from .kupirax import _object

MIXER_TYPES = ("parallel",)


@dataclass
class RampRotation:
    """Rotary positions on the first `dims` dimensions of a head, pairs (i, i + dims / 2).  `scaling` (or None) blends
    every pair's frequency between its own and its own over `factor` by a ramp over the pair index, between the
    pairs that make `fast` and `slow` turns over `original` positions."""

    base: float
    dims: int
    scaling: Optional[Dict[str, float]] = None

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["RampRotation"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        scaling = None
        if raw.get("scaling") is not None:
            sc = _object(raw["scaling"], what + ".scaling")
            scaling = {"factor": take_float(sc, "factor"), "original": take_float(sc, "original"),
                       "fast": take_float(sc, "fast"), "slow": take_float(sc, "slow")}
            if min(scaling.values()) <= 0:
                raise ConfigError(f"config.json: {what}.scaling needs positive factor, original, fast and slow")
        rot = cls(base=take_float(raw, "base"), dims=take_int(raw, "dims", minimum=0), scaling=scaling)
        if rot.dims % 2 or rot.base <= 0 or (rot.base == 1.0 and scaling):
            raise ConfigError(f"config.json: {what} needs an even 'dims' and a positive 'base' (not 1 with scaling)")
        return rot

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling:
            original = self.scaling["original"]
            out["scaling"] = {"factor": self.scaling["factor"],
                              "original": int(original) if float(original).is_integer() else original,
                              "fast": self.scaling["fast"], "slow": self.scaling["slow"]}
        return out


@dataclass
class SopanexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RampRotation] = None

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> "SopanexAttention":
        m = _object(raw, what)
        heads, dim = take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1)
        out = cls(heads=heads, kv_heads=take_int(m, "kv_heads", default=heads, minimum=1), dim=dim,
                  vdim=take_int(m, "vdim", default=dim, minimum=1), scale=take_float(m, "scale", default=dim ** -0.5),
                  rot=RampRotation.from_dict(m.get("rot"), what + ".rot"))
        if heads % out.kv_heads:
            raise ConfigError(f"config.json: {what}: {heads} heads are not a multiple of {out.kv_heads} kv_heads")
        if out.vdim != dim:
            raise ConfigError(f"config.json: {what}: the values are the keys, so vdim {out.vdim} must equal dim {dim}")
        if out.rot is not None and out.rot.dims > dim:
            raise ConfigError(f"config.json: {what}: {out.rot.dims} rotated dimensions of {dim}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "rot": self.rot.to_dict() if self.rot is not None else None}


@dataclass
class SopanexLinearAttention:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int = 0   # inner size of the decay's low-rank pair; 0: as the tensors are stored (not part of the
                          # design: a folder's tensors give it; needed only to write a folder of random weights)

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> "SopanexLinearAttention":
        m = _object(raw, what)
        dim = take_int(m, "dim", minimum=1)
        out = cls(heads=take_int(m, "heads", minimum=1), dim=dim, vdim=take_int(m, "vdim", default=dim, minimum=1),
                  tau=take_float(m, "tau"), decay_rank=take_int(m, "decay_rank", default=0, minimum=0))
        if out.tau <= 0:
            raise ConfigError(f"config.json: {what}.tau must be positive")
        return out

    def to_dict(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank:
            out["decay_rank"] = self.decay_rank
        return out


@dataclass
class SopanexFeedForward:
    experts: int              # experts with tensors
    top: int
    ff: int
    identity: int = 0         # experts behind them that hand their input on
    scale: float = 1.0
    shared_ff: int = 0        # 0: no shared expert

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["SopanexFeedForward"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        if raw.get("kind") != "moe":
            raise ConfigError(f"config.json: {what}.kind {raw.get('kind')!r} is not supported (known: moe)")
        router = _object(raw.get("router"), what + ".router")
        out = cls(experts=take_int(router, "experts", minimum=1), top=take_int(router, "top", minimum=1),
                  ff=take_int(_object(raw.get("expert"), what + ".expert"), "ff", minimum=1),
                  identity=take_int(router, "identity", default=0, minimum=0),
                  scale=take_float(router, "scale", default=1.0))
        if raw.get("shared") is not None:
            out.shared_ff = take_int(_object(raw["shared"], what + ".shared"), "ff", minimum=1)
        if out.top > out.experts + out.identity:
            raise ConfigError(f"config.json: {what}: top {out.top} of {out.experts} + {out.identity} experts")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top, "identity": self.identity,
                                          "scale": self.scale},
                "expert": {"ff": self.ff}, "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass
class SopanexLayer:
    type: str
    left: SopanexAttention
    right: SopanexLinearAttention
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[SopanexFeedForward] = None

    @classmethod
    def from_dict(cls, raw: Any, index: int) -> "SopanexLayer":
        what = f"layers[{index}]"
        raw = _object(raw, what)
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {what}.type {kind!r} is not one of {', '.join(MIXER_TYPES)}")
        m = _object(raw.get("mixer"), what + ".mixer")
        return cls(type=kind, left=SopanexAttention.from_dict(m.get("left"), what + ".mixer.left"),
                   right=SopanexLinearAttention.from_dict(m.get("right"), what + ".mixer.right"),
                   left_scale=take_float(m, "left_scale", default=1.0), right_scale=take_float(m, "right_scale", default=1.0),
                   mlp=SopanexFeedForward.from_dict(raw.get("mlp"), what + ".mlp"))

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type,
                "mixer": {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                          "right_scale": self.right_scale},
                "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass
class SopanexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 1e-6
    embed_scale: float = 1.0
    buckets: int = 0               # 0: no pair table
    mul_prev: int = 0
    mul_cur: int = 0
    layers: List[SopanexLayer] = field(default_factory=list)
    max_positions: int = 1 << 20   # not part of the design: the most positions a sequence may have
    torch_dtype: str = "bfloat16"  # storage of a folder written from this configuration

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "SopanexConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=take_int(raw, "vocab", minimum=1), width=take_int(raw, "width", minimum=1),
                     eps=take_float(_object(raw.get("norm"), "'norm'"), "eps"),
                     layers=[SopanexLayer.from_dict(l, i) for i, l in enumerate(layers)])
        embedding = _object(raw.get("embedding") or {}, "'embedding'")
        config.embed_scale = take_float(embedding, "scale", default=1.0)
        if embedding.get("bigram") is not None:
            pairs = _object(embedding["bigram"], "embedding.bigram")
            config.buckets = take_int(pairs, "buckets", minimum=1)
            config.mul_prev = take_int(pairs, "mul_prev")
            config.mul_cur = take_int(pairs, "mul_cur")
        config.max_positions = take_int(raw, "max_positions", default=cls.max_positions, minimum=1)
        config.torch_dtype = raw.get("torch_dtype", "bfloat16")
        return config

    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> Dict[str, Any]:
        embedding: Dict[str, Any] = {"scale": self.embed_scale, "bigram": None}
        if self.buckets:
            embedding["bigram"] = {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}
        return {"architecture": self.architecture or "Sopanex", "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": embedding, "layers": [l.to_dict() for l in self.layers],
                "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}
