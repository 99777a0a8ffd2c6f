"""Small Badolix configurations and weights for the tests, made here from NumPy random numbers and written with this
file's own safetensors writer (bfloat16 storage), so that nothing of the product takes part in what the oracle reads.
Sizes are unlike each other on purpose: head counts and groups of 1, 2, 3 and all, value sizes that differ from the key
sizes, rotated parts that are a whole head, a part of it or nothing, windows shorter and longer than a page with none,
a few or many kept first tokens, layers that read another layer's keys under a mask of their own, latent ranks that are
no multiples of eight, state sizes, groups, tap counts and norm parts of the state-space mixer that differ, expert
counts in one, two or several groups of which one or all are kept, layers without a feed-forward, and factors on the
embedding, the residual and the logits that are 1 in one configuration and not in the others."""
import json
import struct

import numpy as np


def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = scaling
    return out


RAMP = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}  # the ramp lies inside the pairs of a small head


def attention(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, cap=6.0, size=40, keep=5, rotation=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if cap:
        m["softcap"] = cap
    if size:
        m["mask"] = {"size": size, "keep_first": keep}
    if rotation is not None:
        m["rot"] = rotation
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention", m


def latent(heads=3, dim=8, rot_dim=4, vdim=12, rank=20, scale=0.3, base=100.0, scaling=RAMP):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot_dim:
        m["rot"] = rot(rot_dim, base, scaling)
    return "latent_attention", m


def ssm(heads=4, vdim=8, state=12, groups=2, conv=4, parts=2):
    return "mamba2", {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": parts}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=8, top=3, ff=24, count=4, keep=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top,
                                                            "groups": {"count": count, "keep": keep}}}


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, embed_scale=2.5, mult=0.8, logit_scale=1.5):
    return {"architecture": "Badolix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "residual_mult": mult, "logit_scale": logit_scale, "layers": layers}


CONFIGS = {
    # each mixer alone, without a feed-forward
    "window": lambda: config([layer(attention(rotation=rot(16, 100.0, {"factor": 4.0})))], width=40),
    "latent": lambda: config([layer(latent())], width=40),
    "ssm": lambda: config([layer(ssm())], width=40),
    # both feed-forwards behind a small mixer
    "feeds": lambda: config([layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, size=0, cap=0.0), dense(36)),
                             layer(ssm(heads=2, vdim=8, state=8, groups=1, conv=2, parts=1), moe(8, 3, 20, 4, 2))],
                            width=32, vocab=71),
    # keys and values read by later layers under masks of their own: a shorter window, and no window at all (the cache
    # then keeps everything); value heads larger than key heads
    "shared": lambda: config([
        layer(attention(heads=4, kv_heads=2, dim=16, vdim=24, size=50, keep=9, rotation=rot(8, 50.0, {"factor": 2.0})), dense(24)),
        layer(attention(heads=4, kv_heads=2, dim=16, vdim=24, size=30, keep=3, cap=3.0, scale=0.5,
                        rotation=rot(8, 50.0, {"factor": 2.0}), kv_from=0), moe(6, 2, 16, 3, 2)),
        layer(attention(heads=2, kv_heads=2, dim=16, vdim=24, size=0, cap=0.0, scale=0.2,
                        rotation=rot(8, 50.0, {"factor": 2.0}), kv_from=0))], width=56, vocab=83),
    # the same with windows on every reader: pages behind the widest window go back to the pool, the kept ones stay
    "shared_windows": lambda: config([
        layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, size=70, keep=2, rotation=rot(8, 30.0))),
        layer(attention(heads=3, kv_heads=1, dim=8, vdim=8, size=100, keep=70, cap=0.0, rotation=rot(8, 30.0), kv_from=0), dense(16)),
        layer(attention(heads=1, kv_heads=1, dim=8, vdim=8, size=3, keep=0, cap=9.0, rotation=rot(8, 30.0), kv_from=0))],
        width=24, vocab=50),
    # everything, every layer with sizes of its own, in another order
    "mixed": lambda: config([
        layer(ssm(heads=6, vdim=4, state=16, groups=3, conv=3, parts=3), moe(9, 4, 16, 3, 2)),
        layer(latent(heads=2, dim=16, rot_dim=8, vdim=8, rank=12, scale=0.25, base=1000.0,
                     scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}), dense(40)),
        layer(attention(heads=6, kv_heads=3, dim=8, vdim=12, scale=0.5, cap=4.0, size=33, keep=7,
                        rotation=rot(4, 500.0, {"factor": 3.0})), moe(4, 2, 24, 2, 1)),
        layer(attention(heads=3, kv_heads=3, dim=8, vdim=12, scale=0.4, cap=10.0, size=70, keep=1,
                        rotation=rot(4, 500.0, {"factor": 3.0}), kv_from=2)),
        layer(ssm(heads=2, vdim=16, state=4, groups=2, conv=2, parts=1), dense(20)),
        layer(latent(heads=4, dim=4, rot_dim=0, vdim=4, rank=9, scale=0.6))],
        width=56, vocab=131, eps=1e-6, embed_scale=7.0, mult=0.6, logit_scale=0.5),
    # sizes of one: one head, one group, one expert, one tap, a window of one token, every factor 1
    "ones": lambda: config([
        layer(attention(heads=1, kv_heads=1, dim=32, vdim=8, size=1, keep=0, cap=0.0, rotation=rot(32, 100.0)), moe(1, 1, 16, 1, 1)),
        layer(ssm(heads=1, vdim=8, state=8, groups=1, conv=1, parts=8), moe(3, 3, 8, 1, 1)),
        layer(latent(heads=1, dim=8, rot_dim=2, vdim=8, rank=4, base=3.0, scaling=None), moe(4, 1, 8, 4, 1)),
        layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, size=200, keep=1, cap=50.0, rotation=rot(2, 3.0, {"factor": 1.0})), dense(8))],
        width=36, vocab=61, embed_scale=1.0, mult=1.0, logit_scale=1.0),
    # head sizes at which the bfloat16 run takes its tensor-core kernels
    "tensor": lambda: config([
        layer(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.2, cap=15.0, size=90, keep=11,
                        rotation=rot(64, 10000.0, {"factor": 4.0})), dense(256)),
        layer(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.15, cap=20.0, size=150, keep=64,
                        rotation=rot(64, 10000.0, {"factor": 4.0}), kv_from=0), moe(8, 2, 64, 4, 3)),
        layer(latent(heads=8, dim=32, rot_dim=16, vdim=32, rank=48, scale=0.15, base=200000.0,
                     scaling={"factor": 8.0, "original": 256, "fast": 24.0, "slow": 1.0}), dense(128)),
        layer(ssm(heads=4, vdim=32, state=64, groups=2, conv=4, parts=2), moe(8, 3, 32, 2, 1)),
        layer(attention(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.1, cap=30.0, size=64, keep=64,
                        rotation=rot(32, 100.0, {"factor": 2.0})))],
        width=128, vocab=89, embed_scale=5.0),
    # nothing divisible by four: a width of 50, heads of 6 and 10, the kernels' scalar paths
    "odd": lambda: config([
        layer(attention(heads=3, kv_heads=1, dim=6, vdim=10, size=13, keep=3, rotation=rot(2, 7.0, {"factor": 1.5})), moe(6, 2, 30, 3, 2)),
        layer(ssm(heads=3, vdim=6, state=10, groups=1, conv=3, parts=3), dense(14)),
        layer(latent(heads=5, dim=6, rot_dim=2, vdim=10, rank=7, base=9.0, scaling={"factor": 3.0, "original": 16, "fast": 2.0, "slow": 0.5}),
              moe(5, 5, 6, 1, 1))],
        width=50, vocab=53),
}


def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "final.norm": (D,)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        shapes[p + "norm1"] = (D,)
        if lay["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.o": (D, H * dv)})
            if m.get("kv_from") is None:
                shapes.update({p + "mix.k": (G * d, D), p + "mix.v": (G * dv, D)})
        elif lay["type"] == "latent_attention":
            H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (d + r), D), p + "mix.dkv": (rank + r, D), p + "mix.dkv.norm": (rank,),
                           p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.o": (D, H * dv)})
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * P, H * P + 2 * G * N
            shapes.update({p + "mix.in": (2 * inner + 2 * G * N + H, D), p + "mix.conv": (C, m["conv"]),
                           p + "mix.conv.b": (C,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,),
                           p + "mix.norm": (inner,), p + "mix.o": (D, inner)})
        mlp = lay["mlp"]
        if mlp is None:
            continue  # and no second norm either: nothing would read it
        shapes[p + "norm2"] = (D,)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            shapes.update({p + "mlp.gate": (ff, D), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, D), p + "mlp.up.b": (ff,),
                           p + "mlp.down": (D, ff), p + "mlp.down.b": (D,)})
        else:
            ff = mlp["expert"]["ff"]
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], D)
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{p}mlp.e{e}.gate": (ff, D), f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
    return shapes


def to_bf16_bits(a):
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def make_weights(cfg, seed):
    """name -> float32 array holding bfloat16 values.  Scales are chosen so that every mechanism matters: norm weights
    a few tenths around one, queries large enough that single keys win (scores reach the cap), decays between quick
    forgetting and none, step sizes around one, biases that are no rounding noise, router logits a few units apart."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1]
        fan_in = shape[-1]
        if leaf in ("norm1", "norm2", "mix.norm", "mix.dkv.norm", "mix.D") or name == "final.norm":
            a = 1.0 + 0.3 * rng.randn(*shape)
        elif leaf in ("mix.A_log", "mix.dt_bias"):
            a = rng.randn(*shape) - (0.5 if leaf == "mix.A_log" else 0.0)
        elif leaf == "mix.conv":
            a = 0.6 * rng.randn(*shape)
        elif leaf.endswith(".b"):
            a = 0.3 * rng.randn(*shape)
        elif leaf in ("mlp.router", "mix.q"):
            a = 2.5 * rng.randn(*shape) / np.sqrt(fan_in)
        elif name == "embed":
            a = rng.randn(*shape) / cfg["embedding"]["scale"] ** 0.5
        elif leaf == "mix.o" or leaf.endswith(".down"):
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


def random_config(seed):
    """A configuration drawn from a fixed seed: two to six layers of any kind in any order, sizes from lists that hold
    tensor-core sizes and others, layers that read an earlier attention layer's keys under a mask of their own, dense,
    routed and missing feed-forwards."""
    import random
    rng = random.Random(seed)
    layers, owners = [], []
    for i in range(rng.randint(2, 6)):
        kind = rng.choice(["attention", "attention", "latent_attention", "mamba2"])
        if kind == "attention" and owners and rng.random() < 0.4:
            j = rng.choice(owners)
            m = dict(layers[j]["mixer"], kv_from=j, scale=rng.choice([0.1, 0.125, 0.2]), softcap=rng.choice([10.0, 30.0, 50.0]),
                     mask={"size": rng.choice([17, 64, 100, 130, 200]), "keep_first": rng.choice([0, 1, 8, 24, 64, 70])})
            m["heads"] = m["kv_heads"] * rng.choice([1, 2, 4])
        elif kind == "attention":
            d, G = rng.choice([16, 24, 32, 48, 64, 64, 96, 128]), rng.choice([1, 2, 4])
            m = {"heads": G * rng.choice([1, 2, 4]), "kv_heads": G, "dim": d, "vdim": rng.choice([d, d, d, 32, 64]),
                 "scale": rng.choice([0.1, 0.125, 0.18, 0.25]), "softcap": rng.choice([10.0, 30.0, 50.0]),
                 "mask": {"size": rng.choice([17, 64, 100, 130, 200]), "keep_first": rng.choice([0, 1, 8, 24, 64, 70])},
                 "rot": rot(rng.choice([d, d, d // 2]) // 2 * 2, rng.choice([10000.0, 200000.0]), {"factor": rng.choice([2.0, 4.0, 8.0])})}
            owners.append(i)
        elif kind == "latent_attention":
            r = rng.choice([8, 16, 32])
            m = {"heads": rng.choice([2, 4, 8]), "dim": rng.choice([16, 32, 64]), "rot_dim": r, "vdim": rng.choice([16, 32, 64]),
                 "kv_rank": rng.choice([32, 48, 64, 96, 128, 160]), "scale": rng.choice([0.1, 0.15, 0.2]),
                 "rot": rot(r, rng.choice([10000.0, 1000000.0]), {"factor": rng.choice([4.0, 8.0, 16.0]),
                                                                  "original": rng.choice([256, 1024, 4096]), "fast": 32.0, "slow": 1.0})}
        else:
            G = rng.choice([1, 2, 4])
            H = G * rng.choice([1, 2, 4])
            m = {"heads": H, "vdim": rng.choice([16, 32, 64]), "state": rng.choice([16, 32, 64, 128]), "groups": G,
                 "conv": rng.choice([2, 3, 4]), "norm_groups": rng.choice([1, 2, G, H])}
        feed = rng.choice(["dense", "moe", "moe", None])
        if feed == "dense":
            mlp = dense(rng.choice([64, 128, 256, 200]))
        elif feed == "moe":
            count, per = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 4])
            keep = rng.randint(1, count)
            mlp = moe(count * per, rng.randint(1, min(keep * per, 6)), rng.choice([32, 64, 96]), count, keep)
        else:
            mlp = None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return config(layers, width=rng.choice([64, 96, 128, 160, 192, 256, 384]), vocab=rng.choice([211, 512, 1000]),
                  eps=rng.choice([1e-5, 1e-6]), embed_scale=rng.choice([1.0, 3.0, 12.0]), mult=rng.choice([0.5, 0.7, 1.0]),
                  logit_scale=rng.choice([0.5, 1.0, 2.0]))
