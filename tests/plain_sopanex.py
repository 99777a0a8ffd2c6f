"""Plain, slow Sopanex decoder used as the oracle of the tests.

Whole sequences, NumPy float64, one function per mechanism, dense score matrices, the recurrence walked token by
token.  Nothing here is imported by the product and nothing of the product is imported here.

The design in this file's own notation (D model width, T tokens, p positions from 0):

  x_0       = c_e E[token] + B[(a tok_(p-1) + b tok_p) mod n]       B's row n (its last) for p = 0
  norm(x)   = x / sqrt(mean(x^2) + eps) * (1 + w)                   the weight is stored around zero
  layer     : x <- x + norm1b(mixer(norm1(x))) ;  x <- x + norm2b(ff(norm2(x)))     (no feed-forward: first half only)
  mixer     = c_l attend(h) + c_r glide(h)                          two mixers that read the same rows
  logits    = W_head norm_final(x)

  attend    grouped-query heads; the values are the keys as projected (before rotation); the first r dimensions of
            a q or k head turn in pairs (i, i + r/2) by p f_i, with f_i blended between base^(-2i/r) and that
            over `factor` by a ramp over the pair index, and cos, sin times 0.1 ln(factor) + 1;
            s = scale q.k, causal; weights exp(s_j) / (exp(sink_h) + sum_j exp(s_j)); head h's output times
            sigmoid(W_g h)_h; W_o
  glide     per head S_p = diag(a_p) S_(p-1) + k_p v_p^T, o_p = S_p^T q_p with q = W_q h / sqrt(d),
            a = sigmoid(W_a2 W_a1 h + b)^(1/tau) per key channel; o / rms(o) * w per head, times silu(W_g h); W_o
  ff        s = softmax(W_r h) over all E experts; the `top` largest s + correction are chosen; weights
            s_j / (sum_chosen s + 1e-20) * c; the last `identity` experts return h itself, the others
            W_down gelu(W_up h) (erf form); plus sigmoid(w_sg . h) * shared(h)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- #
# model folder                                                                #
# --------------------------------------------------------------------------- #
def read_folder(path):
    """(config dict, {name: float64 array}) of a folder with config.json and model.safetensors."""
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[8 + n + lo:8 + n + hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        tensors[name] = a.reshape(shape).astype(np.float64)
    return config, tensors


# --------------------------------------------------------------------------- #
# small functions                                                             #
# --------------------------------------------------------------------------- #
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


# --------------------------------------------------------------------------- #
# embedding                                                                   #
# --------------------------------------------------------------------------- #
def bigram_rows(tokens, e):
    """Row of the pair table for every token: a hash of (previous, current); the first token takes the last row."""
    n = e["buckets"]
    rows = [n]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * e["mul_prev"] + int(cur) * e["mul_cur"]) % n)
    return np.asarray(rows)


def embed(tokens, W, cfg):
    e = cfg["embedding"]
    x = W["embed"][np.asarray(tokens)] * e["scale"]
    if e.get("bigram"):
        x = x + W["bigram"][bigram_rows(list(tokens), e["bigram"])]
    return x


# --------------------------------------------------------------------------- #
# rotation                                                                    #
# --------------------------------------------------------------------------- #
def rotation_frequencies(rot):
    """(f [r/2], magnitude): the blended frequencies and the factor on cos and sin."""
    r = rot["dims"]
    i = np.arange(r // 2, dtype=np.float64)
    f = rot["base"] ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):  # the pair index whose wavelength makes `turns` turns over the original length
        return r * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(rot["base"]))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), r - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_halves(x, positions, rot):
    """x [T, heads, d]: among the first r dimensions, (i, i + r/2) turn by positions * f_i; the rest pass."""
    r = rot["dims"] if rot else 0
    if not r:
        return x
    f, mag = rotation_frequencies(rot)
    angle = positions[:, None, None] * f
    c, s = np.cos(angle) * mag, np.sin(angle) * mag
    u, v = x[..., :r // 2], x[..., r // 2:r]
    out = x.copy()
    out[..., :r // 2] = u * c - v * s
    out[..., r // 2:r] = v * c + u * s
    return out


# --------------------------------------------------------------------------- #
# mixers                                                                      #
# --------------------------------------------------------------------------- #
def attend(h, W, pre, m):
    """Grouped-query attention whose values are the unrotated keys, with a learned sink and a gate per head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T, dtype=np.float64)
    q = (h @ W[pre + "q"].T).reshape(T, H, d)
    k = (h @ W[pre + "k"].T).reshape(T, G, d)
    v = k
    q, k = rotate_halves(q, pos, m.get("rot")), rotate_halves(k, pos, m.get("rot"))
    gate = sigmoid(h @ W[pre + "g"].T)  # [T, H]
    out = np.zeros((T, H, d))
    visible = np.tril(np.ones((T, T), dtype=bool))
    for head in range(H):
        kv = head // (H // G)
        s = np.where(visible, (q[:, head] @ k[:, kv].T) * m["scale"], -np.inf)
        sink = W[pre + "sink"][head]
        top = np.maximum(s.max(axis=1, keepdims=True), sink)
        e = np.exp(s - top)
        p = e / (np.exp(sink - top) + e.sum(axis=1, keepdims=True))
        out[:, head] = (p @ v[:, kv]) * gate[:, head:head + 1]
    return out.reshape(T, H * d) @ W[pre + "o"].T


def channel_decay(h, W, pre, m):
    """[T, heads, d]: sigmoid(z)^(1/tau), z through the low-rank pair and its bias."""
    z = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]
    log_sigmoid = -np.logaddexp(0.0, -z)
    return np.exp(log_sigmoid / m["tau"]).reshape(h.shape[0], m["heads"], m["dim"])


def glide(h, W, pre, m, eps, state=None):
    """Gated linear attention, token by token; `state` [heads, d, dv] is carried (and returned) when given."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, d)
    v = (h @ W[pre + "v"].T).reshape(T, H, dv)
    a = channel_decay(h, W, pre, m)
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * W[pre + "norm"]
    out = (o.reshape(T, H * dv) * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T
    return out if state is None else (out, S)


def side_by_side(h, W, pre, m, eps):
    return m["left_scale"] * attend(h, W, pre + "left.", m["left"]) + \
        m["right_scale"] * glide(h, W, pre + "right.", m["right"], eps)


# --------------------------------------------------------------------------- #
# feed-forward                                                                #
# --------------------------------------------------------------------------- #
def expert(h, W, pre):
    return gelu_erf(h @ W[pre + "up"].T) @ W[pre + "down"].T


def route(h, W, pre, router):
    """(chosen [T, top], weights [T, top], margin [T]): margin is how far the last chosen choice score lies above
    the first one left out (infinite when every expert is chosen)."""
    z = h @ W[pre + "router"].T
    e = np.exp(z - z.max(axis=1, keepdims=True))
    s = e / e.sum(axis=1, keepdims=True)
    choice = s + W[pre + "correction"]
    top = router["top"]
    chosen = np.argsort(-choice, axis=1, kind="stable")[:, :top]
    sc = np.take_along_axis(s, chosen, axis=1)
    weights = sc / (sc.sum(axis=1, keepdims=True) + 1e-20) * router["scale"]
    ranked = np.sort(choice, axis=1)[:, ::-1]
    margin = ranked[:, top - 1] - ranked[:, top] if top < ranked.shape[1] else np.full(h.shape[0], np.inf)
    return chosen, weights, margin


def mixture_of_experts(h, W, pre, mlp, margins=None):
    router = mlp["router"]
    real = router["experts"]  # experts with tensors; the router also scores `identity` more, which return h
    chosen, weights, margin = route(h, W, pre, router)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * (h[t] if e >= real else expert(h[t:t + 1], W, f"{pre}e{e}.")[0])
    if mlp.get("shared"):
        out += sigmoid(h @ W[pre + "shared.sg"].T) * expert(h, W, pre + "shared.")
    return out


# --------------------------------------------------------------------------- #
# the model                                                                   #
# --------------------------------------------------------------------------- #
def forward(config, W, tokens, with_layers=False, margins=None):
    """logits [T, vocab] of a whole sequence; with_layers: also the stream after every layer; margins: a list that
    receives, per routed layer, every token's routing margin."""
    eps = config["norm"]["eps"]
    x = embed(tokens, W, config)
    after = []
    for index, layer in enumerate(config["layers"]):
        pre = f"l{index}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']}")
        h = offset_norm(x, W[pre + "norm1"], eps)
        x = x + offset_norm(side_by_side(h, W, pre + "mix.", layer["mixer"], eps), W[pre + "norm1b"], eps)
        if layer.get("mlp"):
            h = offset_norm(x, W[pre + "norm2"], eps)
            x = x + offset_norm(mixture_of_experts(h, W, pre + "mlp.", layer["mlp"], margins), W[pre + "norm2b"], eps)
        after.append(x.copy())
    logits = offset_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(after)) if with_layers else logits
