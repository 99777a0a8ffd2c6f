"""The Badolix oracle against the same mechanisms written the other way round, and the product's host side - the
configuration, the tensor list, what the cache keeps behind a window with kept first tokens (no GPU)."""
import json
import math

import numpy as np
import pytest
import torch

import plain_badolix as pb
import tiny_badolix as tb
from cpp_minilamma_b200.cache import PAGE, SequenceCache
from cpp_minilamma_b200.config.badolix import BadolixConfig
from cpp_minilamma_b200.config.base import ConfigError, config_from_dict
from cpp_minilamma_b200.models.badolix import build_badolix_spec
from cpp_minilamma_b200.parts.base import CacheNeed, KVNeed


def test_the_mask_keeps_the_window_and_the_first_tokens():
    m = pb.visible(12, 4, 2)
    for i in range(12):
        for j in range(12):
            assert m[i, j] == (j <= i and (i - j < 4 or j < 2))
    assert pb.visible(5, 0, 0).sum() == 15           # no window: plain causal
    assert pb.visible(9, 1, 0).sum() == 9            # a window of one: every token sees itself alone


def test_window_attention_one_query_at_a_time():
    """Scores, cap, mask and softmax written per query over an explicit list of visible keys; a second layer reads the
    first one's rotated keys and values under a mask of its own."""
    rng = np.random.RandomState(1)
    D, T = 10, 30
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.7, "softcap": 2.0, "mask": {"size": 7, "keep_first": 3},
         "rot": {"base": 20.0, "dims": 4, "scaling": {"factor": 2.0}}}
    W = {"q": 2 * rng.randn(24, D), "k": rng.randn(12, D), "v": rng.randn(10, D), "o": rng.randn(D, 20)}
    h = rng.randn(T, D)
    got, (keys, values) = pb.window_attention(h, W, "", m, np.arange(T))
    f = 20.0 ** (-2.0 * np.arange(2) / 4) / 2.0

    def turn(x, p):
        out = x.copy()
        for i in range(2):
            a = p * f[i]
            out[i], out[i + 2] = x[i] * math.cos(a) - x[i + 2] * math.sin(a), x[i + 2] * math.cos(a) + x[i] * math.sin(a)
        return out

    want = np.zeros((T, 20))
    for i in range(T):
        seen = [j for j in range(i + 1) if i - j < 7 or j < 3]
        for head in range(4):
            q = turn((W["q"] @ h[i])[head * 6:(head + 1) * 6], i)
            s = np.array([2.0 * math.tanh(0.7 * q @ turn((W["k"] @ h[j])[(head // 2) * 6:(head // 2 + 1) * 6], j) / 2.0) for j in seen])
            p = np.exp(s - s.max())
            p /= p.sum()
            want[i, head * 5:(head + 1) * 5] = sum(pj * (W["v"] @ h[j])[(head // 2) * 5:(head // 2 + 1) * 5] for pj, j in zip(p, seen))
    assert np.abs(got - want @ W["o"].T).max() < 1e-9
    # the reader: its own queries, scale, cap and mask over the same keys and values
    m2 = dict(m, heads=2, scale=0.3, softcap=0.0, mask={"size": 2, "keep_first": 0}, kv_from=0)
    W2 = {"q": rng.randn(12, D), "o": rng.randn(D, 10)}
    got2, _ = pb.window_attention(h, W2, "", m2, np.arange(T), shared=(keys, values))
    i = T - 1
    q = turn((W2["q"] @ h[i])[:6], i)
    s = np.array([0.3 * q @ keys[j, 0] for j in (i - 1, i)])
    p = np.exp(s - s.max()) / np.exp(s - s.max()).sum()
    head0 = p @ values[[i - 1, i], 0]
    q1 = turn((W2["q"] @ h[i])[6:], i)
    s1 = np.array([0.3 * q1 @ keys[j, 1] for j in (i - 1, i)])
    p1 = np.exp(s1 - s1.max()) / np.exp(s1 - s1.max()).sum()
    assert np.abs(got2[i] - np.concatenate([head0, p1 @ values[[i - 1, i], 1]]) @ W2["o"].T).max() < 1e-9


def test_frequencies_divided_or_under_a_ramp():
    f, mag = pb.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0}})
    assert np.allclose(f, 100.0 ** (-np.arange(4) / 4.0) / 4.0) and mag == 1.0
    f, mag = pb.frequencies({"base": 100.0, "dims": 8})
    assert np.allclose(f, 100.0 ** (-np.arange(4) / 4.0)) and mag == 1.0
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f, mag = pb.frequencies({"base": 100.0, "dims": 8, "scaling": sc})
    plain = 100.0 ** (-np.arange(4) / 4.0)
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0))), 7)
    for i in range(4):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert np.isclose(f[i], plain[i] / 4.0 * r + plain[i] * (1 - r))
    assert f[0] == plain[0] and np.isclose(mag, 0.1 * math.log(4.0) + 1.0)


def test_latent_attention_with_keys_and_values_written_out():
    rng = np.random.RandomState(2)
    D, T = 9, 14
    m = {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 3, "kv_rank": 5, "scale": 0.4, "rot": {"base": 10.0, "dims": 2}}
    W = {"q": rng.randn(12, D), "dkv": rng.randn(7, D), "dkv.norm": 1 + 0.2 * rng.randn(5), "uk": rng.randn(8, 5),
         "uv": rng.randn(6, 5), "o": rng.randn(D, 6)}
    h = rng.randn(T, D)
    got = pb.latent_attention(h, W, "", m, np.arange(T), 1e-5)
    down = h @ W["dkv"].T
    c = down[:, :5] / np.sqrt((down[:, :5] ** 2).mean(axis=1, keepdims=True) + 1e-5) * W["dkv.norm"]

    def turn(x, p):  # one pair, frequency 1
        return np.array([x[0] * math.cos(p) - x[1] * math.sin(p), x[1] * math.cos(p) + x[0] * math.sin(p)])

    want = np.zeros((T, 6))
    for i in range(T):
        for head in range(2):
            q = (W["q"] @ h[i])[head * 6:(head + 1) * 6]
            q = np.concatenate([q[:4], turn(q[4:], i)])
            keys = [np.concatenate([(W["uk"] @ c[j])[head * 4:(head + 1) * 4], turn(down[j, 5:], j)]) for j in range(i + 1)]
            s = np.array([0.4 * q @ k for k in keys])
            p = np.exp(s - s.max())
            p /= p.sum()
            want[i, head * 3:(head + 1) * 3] = sum(pj * (W["uv"] @ c[j])[head * 3:(head + 1) * 3] for j, pj in enumerate(p))
    assert np.abs(got - want @ W["o"].T).max() < 1e-9


def test_state_space_unrolled_over_earlier_tokens():
    """y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (C_t . B_s) x_s + D x_t, with the convolution written per token."""
    rng = np.random.RandomState(3)
    D, T = 7, 11
    m = {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "conv": 3, "norm_groups": 2}
    inner, gn = 12, 10
    W = {"in": rng.randn(2 * inner + 2 * gn + 4, D), "conv": rng.randn(inner + 2 * gn, 3), "conv.b": rng.randn(inner + 2 * gn),
         "dt_bias": rng.randn(4), "A_log": rng.randn(4) - 1, "D": rng.randn(4), "norm": 1 + 0.2 * rng.randn(inner),
         "o": rng.randn(D, inner)}
    h = rng.randn(T, D)
    got = pb.state_space(h, W, "", m, 1e-5)
    proj = h @ W["in"].T
    z, raw, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * gn], proj[:, 2 * inner + 2 * gn:]
    conv = np.zeros_like(raw)
    for t in range(T):
        for c in range(raw.shape[1]):
            acc = W["conv.b"][c]
            for back in range(3):
                if t - back >= 0:
                    acc += W["conv"][c, 2 - back] * raw[t - back, c]   # the last tap meets the current token
            conv[t, c] = acc / (1 + math.exp(-acc))
    dt = np.log1p(np.exp(dt + W["dt_bias"]))
    a = np.exp(-np.exp(W["A_log"]) * dt)
    y = np.zeros((T, inner))
    for t in range(T):
        for head in range(4):
            g = head // 2
            x = conv[:, head * 3:(head + 1) * 3]
            B, C = conv[:, inner + g * 5:inner + (g + 1) * 5], conv[:, inner + gn + g * 5:inner + gn + (g + 1) * 5]
            acc = W["D"][head] * x[t]
            for s in range(t + 1):
                acc = acc + np.prod(a[s + 1:t + 1, head]) * dt[s, head] * (C[t] @ B[s]) * x[s]
            y[t, head * 3:(head + 1) * 3] = acc
    y = y * (z / (1 + np.exp(-z)))
    for part in range(2):
        piece = y[:, part * 6:(part + 1) * 6]
        y[:, part * 6:(part + 1) * 6] = piece / np.sqrt((piece ** 2).mean(axis=1, keepdims=True) + 1e-5)
    assert np.abs(got - (y * W["norm"]) @ W["o"].T).max() < 1e-9


def test_routing_inside_the_best_groups():
    s = np.array([0.9, 0.1, 0.2,   0.5, 0.55, 0.0,   0.8, 0.05, 0.3,   0.6, 0.6, 0.6])
    # ratings of the runs (top two added): 1.1, 1.05, 1.1, 1.2 -> groups 3, 0 and (tie with 0 earlier) 2 are kept for keep = 3
    chosen, weights, margin = pb.route(s, 4, 4, 3)
    assert list(chosen) == [0, 6, 9, 10]          # 0.9, 0.8, then the first two of the tied 0.6s; group 1 is shut out
    assert np.allclose(weights, np.array([0.9, 0.8, 0.6, 0.6]) / 2.9) and np.isclose(margin, 0.0)
    chosen, weights, _ = pb.route(s, 2, 4, 1)
    assert list(chosen) == [9, 10] and np.allclose(weights, [0.5, 0.5])
    chosen, _, margin = pb.route(s, 12, 1, 1)      # one group, every expert
    assert sorted(chosen) == list(range(12)) and np.isinf(margin)
    chosen, _, _ = pb.route(np.array([0.2, 0.7, 0.4]), 1, 3, 2)   # groups of one expert score that expert alone
    assert list(chosen) == [1]


def test_dense_feed_forward_has_three_biases():
    rng = np.random.RandomState(5)
    W = {"gate": rng.randn(4, 3), "gate.b": rng.randn(4), "up": rng.randn(4, 3), "up.b": rng.randn(4),
         "down": rng.randn(3, 4), "down.b": rng.randn(3)}
    h = rng.randn(2, 3)
    g = h @ W["gate"].T + W["gate.b"]
    want = ((g / (1 + np.exp(-g))) * (h @ W["up"].T + W["up.b"])) @ W["down"].T + W["down.b"]
    assert np.abs(pb.dense_ff(h, W, "") - want).max() < 1e-12


@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_configuration_round_trip_and_tensor_list(name):
    raw = tb.CONFIGS[name]()
    config = config_from_dict(raw)
    assert isinstance(config, BadolixConfig)
    again = config_from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config
    from cpp_minilamma_b200.engine.model import Model
    model = Model(build_badolix_spec(config), torch.float32, "cpu", max_positions=8)
    listed = {s.name: tuple(s.shape) for s in model.weight_specs() if not s.optional}
    assert listed == tb.tensor_shapes(raw)


def test_configuration_faults_are_named():
    good = tb.CONFIGS["mixed"]()
    for change, word in [(lambda c: c["layers"][0].update(type="conv"), "type"),
                         (lambda c: c["layers"][2]["mixer"].update(kv_heads=4), "multiple"),
                         (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3), "dims"),
                         (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(factor=0), "positive"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(vdim=8), "differ"),
                         (lambda c: c["layers"][1]["mixer"].update(rot_dim=6), "rot_dim"),
                         (lambda c: c["layers"][0]["mixer"].update(groups=4), "groups"),
                         (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), "norm groups"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
                         (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=2), "groups"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="gelu"), "kind"),
                         (lambda c: c.pop("norm"), "norm")]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            config_from_dict(raw)
        assert word in str(caught.value), (word, str(caught.value))


def test_the_cache_of_shared_keys_keeps_the_widest_reach():
    from cpp_minilamma_b200.engine.model import Model
    needs = {}
    for name in ("shared", "shared_windows", "tensor"):
        model = Model(build_badolix_spec(config_from_dict(tb.CONFIGS[name]())), torch.float32, "cpu", max_positions=8)
        needs[name] = model.cache_needs()
    assert needs["shared"][0][2].kv.window == 0 and needs["shared"][0][2].kv.keep_first == 0   # a reader without a window
    assert [n[1] for n in needs["shared"]] == [None, 0, 0]
    assert (needs["shared_windows"][0][2].kv.window, needs["shared_windows"][0][2].kv.keep_first) == (100, 70)
    assert (needs["tensor"][0][2].kv.window, needs["tensor"][0][2].kv.keep_first) == (150, 64)


def test_pages_of_kept_tokens_are_never_handed_back():
    need = KVNeed(1, 8, window=PAGE, keep_first=PAGE + 3)        # the first two pages hold kept tokens
    cache = SequenceCache([(0, None, CacheNeed(kv=need))], PAGE * 6, 2, PAGE * 64, torch.float32, "cpu")
    slot = cache.acquire(1)[0]
    cache.reserve([(slot, 3 * PAGE)])
    for _ in range(40):                                           # far beyond what the pool could hold without hand-back
        cache.reserve([(slot, PAGE // 2)])
        cache.check()
    pages = cache.groups[0].pages[slot]
    assert pages[0] is not None and pages[1] is not None and pages[2] is None and pages[-1] is not None
    assert sum(p is not None for p in pages) <= 4
    cache.release(slot)
    assert cache.groups[0].pool.n_free == cache.groups[0].pool.n_pages


def test_oracle_forward_shapes_and_layer_trace():
    raw = tb.CONFIGS["mixed"]()
    W = {k: v.astype(np.float64) for k, v in tb.make_weights(raw, 3).items()}
    toks = tb.tokens(raw, 20, 1)
    margins = []
    logits, after = pb.forward(raw, W, toks, return_layers=True, margins=margins)
    assert logits.shape == (20, raw["vocab"]) and after.shape == (6, 20, raw["width"]) and len(margins) == 2
    assert np.abs(pb.forward(raw, W, toks[:9]) - logits[:9]).max() < 1e-9  # causal: a prefix gives the same logits


def test_command_line_random_then_inspect(tmp_path, capsys):
    """`random` writes a folder from a configuration file (every tensor of the list, bfloat16), `inspect` reads it
    back, and the oracle can run it."""
    from cpp_minilamma_b200.cli import main
    raw = tb.CONFIGS["mixed"]()
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(raw))
    assert main(["random", str(tmp_path / "m"), "--config", str(cfg), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "architecture: Badolix" in out and "status=ok" in out
    assert "tensor l0.mlp.e8.down [56, 16] bfloat16" in out and "tensor l4.mix.conv [48, 2] bfloat16" in out
    assert "tensor l3.mix.q [24, 56] bfloat16" in out and "l3.mix.k" not in out
    config, W = pb.read_folder(tmp_path / "m")
    assert set(W) - set(tb.tensor_shapes(raw)) == {"l3.norm2", "l5.norm2"}   # written all the same; nothing reads them
    logits = pb.forward(config, W, tb.tokens(raw, 12, 5))
    assert logits.shape == (12, raw["vocab"]) and np.isfinite(logits).all()
