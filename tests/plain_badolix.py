"""Plain, slow Badolix decoder used as the oracle of the tests.

Whole sequences, NumPy float64, one function per mechanism, dense score matrices, the recurrence walked token by
token.  Nothing here is imported by the product and nothing of the product is imported here.

The design in this file's own notation (D model width, T tokens, p positions from 0, m the residual factor):

  x_0      = c_e E[token]
  norm(x)  = x / sqrt(mean(x^2) + eps) * w
  layer    : x <- x + m mixer(norm1(x)) ;  x <- x + m ff(norm2(x))        (no feed-forward: first half only)
  logits   = c_o E norm_final(x)                                           the head is the embedding table

  window attention   Hq / Hk grouped heads of d (values dv); the first r dimensions of a q or k head turn in pairs
                     (i, i + r/2) by p f_i / factor; s = cap tanh(scale q.k / cap); key j is visible from query i
                     iff j <= i and (i - j < size or j < keep); softmax over the visible keys; W_o.  A layer may
                     read the rotated keys and the values of an earlier layer instead of projecting its own.
  latent attention   q = W_q h per head as [d plain | r rotated]; W_dkv h = [c' | k_r]; c = norm(c'; w_c); a head's
                     key is [W_uk,h c | k_r], its value W_uv,h c; the r-parts turn in pairs (i, i + r/2) by p f_i
                     with f_i blended by a ramp over the pair index and cos, sin times 0.1 ln(factor) + 1;
                     s = scale q.k, causal softmax; W_o
  state-space mixer  W_in h = [z | x | B | C | dt]; (x, B, C) pass a causal convolution over time with a bias and
                     silu; dt = softplus(dt + b_dt); per head S_t = exp(-exp(A_h) dt) S_(t-1) + dt B_t x_t^T,
                     y_t = S_t^T C_t + D_h x_t; y silu(z), normalised in equal parts, times a weight; W_o
  dense ff           W_down (silu(W_gate h + b_g) * (W_up h + b_u)) + b_d
  routed ff          s = sigmoid(W_r h); the experts are cut into `count` runs of consecutive experts of one length, a
                     run is rated by its top two s added up, only the `keep` best-rated runs stay open; the `top` highest
                     s inside them are chosen;
                     weights s_j / (sum of the chosen s + 1e-20); out = sum_j w_j expert_j(h) (experts have no biases)
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
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        tensors[name] = a.reshape(tuple(info["shape"])).astype(np.float64)
    return config, tensors


# --------------------------------------------------------------------------- #
# small functions                                                             #
# --------------------------------------------------------------------------- #
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def softmax_rows(s):
    """Rows of s with -inf where nothing is visible; every row has at least one finite entry."""
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


# --------------------------------------------------------------------------- #
# rotation                                                                     #
# --------------------------------------------------------------------------- #
def frequencies(rot):
    """(f_i for i < dims / 2, factor on cos and sin) of a 'rot' object {base, dims, scaling}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor = float(scaling["factor"])
    if "original" not in scaling:  # every frequency divided alike
        return f / factor, 1.0
    original = float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, n]: the first rot.dims dimensions of every head turned in pairs (i, i + dims / 2)."""
    dims = int(rot["dims"]) if rot else 0
    if dims == 0:
        return x
    f, magnitude = frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., dims:]], axis=-1)


# --------------------------------------------------------------------------- #
# mixers                                                                       #
# --------------------------------------------------------------------------- #
def visible(T, size, keep):
    """[T, T] True where query i sees key j: j <= i and (i - j < size or j < keep); size 0: no window."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    near = (i - j < size) if size > 0 else np.ones((T, T), dtype=bool)
    return (j <= i) & (near | (j < keep))


def window_attention(h, w, prefix, m, positions, shared=None):
    """Returns (output [T, D], (rotated keys, values)); `shared`: an earlier layer's (keys, values) to read."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate((h @ w[prefix + "q"].T).reshape(T, H, d), positions, m.get("rot"))
    if shared is None:
        k = rotate((h @ w[prefix + "k"].T).reshape(T, G, d), positions, m.get("rot"))
        v = (h @ w[prefix + "v"].T).reshape(T, G, dv)
    else:
        k, v = shared
    mask_cfg = m.get("mask") or {}
    mask = visible(T, int(mask_cfg.get("size", 0)), int(mask_cfg.get("keep_first", 0)))
    cap = float(m.get("softcap") or 0.0)
    out = np.zeros((T, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * float(m["scale"])
        if cap > 0:
            s = cap * np.tanh(s / cap)
        s = np.where(mask, s, -np.inf)
        out[:, head, :] = softmax_rows(s) @ v[:, g, :]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T, (k, v)


def latent_attention(h, w, prefix, m, positions, eps):
    T = h.shape[0]
    H, d, r, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = dict(m["rot"], dims=r) if r else None
    q = (h @ w[prefix + "q"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, rot)
    down = h @ w[prefix + "dkv"].T
    c = rms(down[:, :rank], eps) * w[prefix + "dkv.norm"]
    k_rot = rotate(down[:, None, rank:], positions, rot)[:, 0, :]
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, dv)
    mask = visible(T, 0, 0)
    out = np.zeros((T, H, dv))
    for head in range(H):
        s = (q_plain[:, head, :] @ k_plain[:, head, :].T + q_rot[:, head, :] @ k_rot.T) * float(m["scale"])
        out[:, head, :] = softmax_rows(np.where(mask, s, -np.inf)) @ v[:, head, :]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


def causal_convolution(u, taps_w, bias):
    """u [T, C], taps_w [C, taps] whose last column meets the current token, zeros before the start."""
    T, taps = u.shape[0], taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], axis=0)
    out = np.tile(bias[None, :], (T, 1))
    for j in range(taps):
        out = out + padded[j:j + T, :] * taps_w[:, j][None, :]
    return out


def state_space(h, w, prefix, m, eps):
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    parts = int(m["norm_groups"])
    inner = H * P
    proj = h @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_convolution(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"][None, :])
    rate = np.exp(w[prefix + "A_log"])
    y = np.zeros((T, H, P))
    for head in range(H):
        g = head // (H // G)
        S = np.zeros((N, P))
        for t in range(T):
            S = math.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[prefix + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


# --------------------------------------------------------------------------- #
# feed-forwards                                                                #
# --------------------------------------------------------------------------- #
def dense_ff(h, w, prefix):
    gate = h @ w[prefix + "gate"].T + w[prefix + "gate.b"]
    up = h @ w[prefix + "up"].T + w[prefix + "up.b"]
    return (silu(gate) * up) @ w[prefix + "down"].T + w[prefix + "down.b"]


def route(scores, top, count, keep):
    """(chosen experts, weights, margin) of one token's scores; ties go to the lower index.  The margin is the
    smallest gap between something taken and the best thing left out (groups, then experts)."""
    E = scores.shape[0]
    per = E // count
    group_score = np.array([np.sort(scores[g * per:(g + 1) * per])[::-1][:2].sum() for g in range(count)])
    order = np.argsort(-group_score, kind="stable")
    kept = order[:keep]
    margin = group_score[order[keep - 1]] - group_score[order[keep]] if keep < count else np.inf
    allowed = np.zeros(E, dtype=bool)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    masked = np.where(allowed, scores, -np.inf)
    ranked = np.argsort(-masked, kind="stable")
    chosen = ranked[:top]
    if top < E and np.isfinite(masked[ranked[top]]):
        margin = min(margin, masked[ranked[top - 1]] - masked[ranked[top]])
    s = scores[chosen]
    return chosen, s / (s.sum() + 1e-20), margin


def routed_ff(h, w, prefix, mlp, margins=None):
    """`margins`: a list that receives one array per call, the routing margin of every token."""
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    scores = sigmoid(h @ w[prefix + "router"].T)
    out = np.zeros_like(h)
    token_margin = np.zeros(h.shape[0])
    if margins is not None:
        margins.append(token_margin)
    for t in range(h.shape[0]):
        chosen, weights, token_margin[t] = route(scores[t], int(router["top"]), int(groups["count"]), int(groups["keep"]))
        for e, weight in zip(chosen, weights):
            p = f"{prefix}e{e}."
            out[t] += weight * ((silu(h[t] @ w[p + "gate"].T) * (h[t] @ w[p + "up"].T)) @ w[p + "down"].T)
    return out


# --------------------------------------------------------------------------- #
# the whole model                                                              #
# --------------------------------------------------------------------------- #
def forward(config, w, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence from its first token (and the stream after every layer).  `margins`: a list
    that receives every routed layer's margins per token."""
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(tokens.shape[0])
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    streams = []
    for i, layer in enumerate(config["layers"]):
        prefix = f"l{i}."
        m = layer["mixer"]
        h = rms(x, eps) * w[prefix + "norm1"]
        if layer["type"] == "attention":
            source = m.get("kv_from")
            mixed, kept[i] = window_attention(h, w, prefix + "mix.", m, positions,
                                              shared=None if source is None else kept[int(source)])
        elif layer["type"] == "latent_attention":
            mixed = latent_attention(h, w, prefix + "mix.", m, positions, eps)
        elif layer["type"] == "mamba2":
            mixed = state_space(h, w, prefix + "mix.", m, eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + mult * mixed
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms(x, eps) * w[prefix + "norm2"]
            x = x + mult * (dense_ff(h, w, prefix + "mlp.") if mlp["kind"] == "dense"
                            else routed_ff(h, w, prefix + "mlp.", mlp, margins))
        streams.append(x.copy())
    logits = (rms(x, eps) * w["final.norm"]) @ w["embed"].T * float(config.get("logit_scale", 1.0))
    return (logits, np.stack(streams)) if return_layers else logits
