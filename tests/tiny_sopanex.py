"""Small Sopanex configurations and weights for the tests, made here from NumPy random numbers and written with this
file's own safetensors writer (bfloat16 storage), so that nothing of the product takes part in what the oracle
reads.  Sizes are unlike each other on purpose: head counts and groups of 1, 2, 3 and all, rotated parts that are a
whole head, a part of it or nothing, with and without the ramp over the frequencies, key and value sizes of the
recurrent mixer that differ, decay ranks from 1 up, expert counts that are no powers of two with none, one or
several pass-through experts, one expert per token and every expert per token, layers without a feed-forward or
without a shared expert, pair tables of one bucket and of many, multipliers of 0 and 1, and mixer weights of 0 on
one side (so that the other side stands alone)."""
import json
import struct

import numpy as np


def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = {"factor": scaling[0], "original": scaling[1], "fast": scaling[2], "slow": scaling[3]}
    return out


def left(heads=4, kv_heads=2, dim=16, scale=0.3, rotation=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rotation}


def right(heads=2, dim=8, vdim=12, tau=8.0, rank=6):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def moe(experts=5, top=2, ff=24, identity=1, scale=1.5, shared=16):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "identity": identity, "scale": scale},
            "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def layer(l, r, mlp=None, scales=(1.0, 1.0)):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, embed_scale=3.0, bigram=(53, 5, 3)):
    pairs = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]} if bigram else None
    return {"architecture": "Sopanex", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale, "bigram": pairs}, "layers": layers}


RAMP = (4.0, 64, 8.0, 1.0)  # factor, original length, fast and slow turns: the ramp lies inside the pairs of a small head

CONFIGS = {
    # one side of the mixer each (the other side's weight is 0), no feed-forward
    "left_only": lambda: config([layer(left(rotation=rot(8, 100.0, RAMP)), right(), scales=(1.3, 0.0))], width=40),
    "right_only": lambda: config([layer(left(heads=2, kv_heads=1, dim=8), right(heads=3, dim=16, vdim=8, tau=4.0, rank=5),
                                        scales=(0.0, 0.8))], width=40),
    # the routed feed-forward behind a small mixer: pass-through experts, correction, weight scale, gated shared expert
    "routed": lambda: config([layer(left(heads=2, kv_heads=1, dim=8), right(heads=1, dim=8, vdim=8, rank=3),
                                    moe(experts=6, top=3, ff=20, identity=2, scale=2.5, shared=12))], width=32, vocab=71),
    # everything, every layer with sizes of its own
    "mixed": lambda: config([
        layer(left(heads=6, kv_heads=3, dim=8, scale=0.5, rotation=rot(8, 500.0, RAMP)), right(heads=2, dim=24, vdim=8, tau=16.0, rank=4),
              moe(7, 3, 24, identity=2, scale=1.7, shared=40), scales=(1.4, 0.6)),
        layer(left(heads=2, kv_heads=1, dim=24, scale=0.25, rotation=rot(12, 10000.0)), right(heads=4, dim=8, vdim=16, tau=2.0, rank=9),
              moe(7, 2, 16, identity=0, scale=1.0, shared=0), scales=(0.7, 1.1)),
        layer(left(heads=3, kv_heads=3, dim=24, scale=0.2, rotation=None), right(heads=1, dim=16, vdim=24, tau=30.0, rank=2), None),
        layer(left(heads=4, kv_heads=1, dim=8, scale=0.4, rotation=rot(4, 50.0, (2.0, 32, 4.0, 0.5))), right(heads=2, dim=8, vdim=8, tau=1.0, rank=8),
              moe(3, 1, 32, identity=3, scale=0.5, shared=8), scales=(1.0, 1.0))],
        width=56, vocab=131, eps=1e-6, embed_scale=7.0, bigram=(257, 29, 11)),
    # heads of one, one expert, every expert per token, one bucket, multipliers of 0 and 1, an embedding scale of 1
    "ones": lambda: config([
        layer(left(heads=1, kv_heads=1, dim=32, rotation=rot(32, 100.0, RAMP)), right(heads=1, dim=4, vdim=4, tau=1.0, rank=1),
              moe(1, 1, 16, identity=0, scale=1.0, shared=8)),
        layer(left(heads=2, kv_heads=2, dim=8, rotation=rot(2, 3.0)), right(heads=1, dim=40, vdim=8, tau=5.0, rank=3),
              moe(2, 3, 8, identity=1, scale=1.0, shared=0)),
        layer(left(heads=2, kv_heads=1, dim=8, rotation=rot(0)), right(heads=2, dim=8, vdim=40, tau=3.0, rank=16),
              moe(1, 1, 24, identity=1, scale=3.0, shared=24))],
        width=36, vocab=61, embed_scale=1.0, bigram=(1, 1, 0)),
    # no pair table at all; two layers without a feed-forward in a row
    "bare": lambda: config([layer(left(heads=2, kv_heads=2, dim=16, rotation=rot(16, 1000.0, RAMP)), right(), None),
                            layer(left(heads=2, kv_heads=1, dim=16, rotation=rot(8, 1000.0)), right(heads=1, dim=8, vdim=16), None)],
                           width=32, vocab=50, bigram=None),
    # head sizes at which the bfloat16 run takes its tensor-core kernels (keys of 64 and 128, expert widths in steps of 8),
    # recurrent heads of 64 and 128
    "tensor": lambda: config([
        layer(left(heads=4, kv_heads=2, dim=64, scale=0.2, rotation=rot(32, 10000.0, (3.0, 128, 16.0, 1.0))), right(heads=2, dim=64, vdim=64, tau=16.0, rank=16),
              moe(4, 2, 32, identity=1, scale=1.5, shared=16)),
        layer(left(heads=2, kv_heads=1, dim=128, scale=0.15, rotation=rot(128, 200000.0, (8.0, 256, 24.0, 1.0))), right(heads=1, dim=128, vdim=32, tau=8.0, rank=8),
              moe(8, 3, 64, identity=2, scale=1.0, shared=0)),
        layer(left(heads=8, kv_heads=1, dim=32, scale=0.3, rotation=rot(16, 100.0)), right(heads=4, dim=32, vdim=128, tau=4.0, rank=8), None)],
        width=128, vocab=89, embed_scale=5.0, bigram=(509, 13, 17)),
    # nothing divisible by four: a width of 50, heads of 6 and 10, the kernels' scalar paths
    "odd": lambda: config([
        layer(left(heads=3, kv_heads=1, dim=6, rotation=rot(2, 7.0, (3.0, 16, 2.0, 0.5))), right(heads=3, dim=6, vdim=10, tau=7.0, rank=3),
              moe(5, 2, 30, identity=1, scale=1.3, shared=14)),
        layer(left(heads=5, kv_heads=5, dim=10, rotation=rot(6, 9.0)), right(heads=1, dim=10, vdim=6, tau=2.5, rank=7),
              moe(5, 4, 6, identity=2, scale=0.7, shared=0))],
        width=50, vocab=53, bigram=(11, 3, 2)),
}


def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "final.norm": (D,), "head": (cfg["vocab"], D)}
    if cfg["embedding"].get("bigram"):
        shapes["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, D)
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        l, r = lay["mixer"]["left"], lay["mixer"]["right"]
        H, G, d = l["heads"], l["kv_heads"], l["dim"]
        shapes.update({p + "norm1": (D,), p + "norm1b": (D,),
                       p + "mix.left.q": (H * d, D), p + "mix.left.k": (G * d, D), p + "mix.left.sink": (H,),
                       p + "mix.left.g": (H, D), p + "mix.left.o": (D, H * d)})
        H, d, dv, rank = r["heads"], r["dim"], r["vdim"], r["decay_rank"]
        shapes.update({p + "mix.right.q": (H * d, D), p + "mix.right.k": (H * d, D), p + "mix.right.v": (H * dv, D),
                       p + "mix.right.g": (H * dv, D), p + "mix.right.o": (D, H * dv), p + "mix.right.norm": (dv,),
                       p + "mix.right.a1": (rank, D), p + "mix.right.a2": (H * d, rank), p + "mix.right.a2.b": (H * d,)})
        mlp = lay["mlp"]
        if mlp is None:
            continue  # and no norms around it either: nothing would read them
        shapes.update({p + "norm2": (D,), p + "norm2b": (D,)})
        E, ff, n = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["router"]["experts"] + mlp["router"]["identity"]
        shapes.update({p + "mlp.router": (n, D), p + "mlp.correction": (n,)})
        for e in range(E):
            shapes.update({f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.up": (sf, D), p + "mlp.shared.down": (D, sf), p + "mlp.shared.sg": (1, D)})
    return shapes


def to_bf16_bits(a):
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def make_weights(cfg, seed):
    """name -> float32 array holding bfloat16 values.  Scales are chosen so that every mechanism matters: norm
    weights (stored around zero) of a few tenths, queries large enough that single keys win, sinks from far below
    to far above the scores (their share of a row moves between nothing and almost everything), decay biases
    that put the decays between quick forgetting and none, router logits a few units apart with corrections that
    change the choice, gates that are neither open nor shut."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1]
        fan_in = shape[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            a = 0.3 * rng.randn(*shape)
        elif leaf == "mix.right.norm":
            a = 1.0 + 0.3 * rng.randn(*shape)
        elif leaf == "mix.left.sink":
            a = 2.5 * rng.randn(*shape)
        elif leaf == "mix.right.a2.b":
            a = 1.0 + 2.0 * rng.randn(*shape)
        elif leaf == "mlp.correction":
            a = 0.15 * rng.randn(*shape)
        elif leaf in ("mlp.router", "mix.left.q"):
            a = 2.0 * rng.randn(*shape) / np.sqrt(fan_in)
        elif name in ("embed", "bigram"):
            a = rng.randn(*shape) * (1.0 if name == "bigram" else 1.0 / cfg["embedding"]["scale"] ** 0.5)
        elif leaf in ("mix.left.o", "mix.right.o") or leaf.endswith(".down"):
            a = 0.7 * rng.randn(*shape) / np.sqrt(fan_in)
        else:
            a = 1.5 * rng.randn(*shape) / np.sqrt(fan_in)
        bits = to_bf16_bits(a)
        out[name] = (bits.astype(np.uint32) << 16).view(np.float32).reshape(shape)
    return out


def write_folder(cfg, weights, folder):
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    header, blobs, at = {}, [], 0
    for name, a in weights.items():
        raw = to_bf16_bits(a).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(folder / "model.safetensors", "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
    return str(folder)


def make_folder(name, folder, seed=0):
    cfg = CONFIGS[name]()
    weights = make_weights(cfg, seed)
    return write_folder(cfg, weights, folder), cfg, {k: v.astype(np.float64) for k, v in weights.items()}


def tokens(cfg, length, seed):
    return [int(t) for t in np.random.RandomState(seed).randint(0, cfg["vocab"], size=length)]
