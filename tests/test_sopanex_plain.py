"""The Sopanex oracle against the same mechanisms written the other way round, and the configuration and tensor list
of the product - all without a GPU."""
import json
import math

import numpy as np
import pytest

import plain_sopanex as ps
import tiny_sopanex as ts
from cpp_minilamma_b200.config.base import ConfigError, config_from_dict
from cpp_minilamma_b200.config.sopanex import SopanexConfig
from cpp_minilamma_b200.models.sopanex import build_sopanex_spec


def test_pair_rows_hash_the_token_before_and_the_token():
    e = {"buckets": 7, "mul_prev": 3, "mul_cur": 5}
    assert ps.bigram_rows([4, 2, 6, 6], e).tolist() == [7, (12 + 10) % 7, (6 + 30) % 7, (18 + 30) % 7]
    assert ps.bigram_rows([9], e).tolist() == [7]  # a first token takes the table's last row
    cfg = {"embedding": {"scale": 2.0, "bigram": e}}
    W = {"embed": np.arange(20.0).reshape(10, 2), "bigram": 100.0 * np.arange(16.0).reshape(8, 2)}
    x = ps.embed([4, 2], W, cfg)
    assert np.allclose(x[0], 2.0 * W["embed"][4] + W["bigram"][7]) and np.allclose(x[1], 2.0 * W["embed"][2] + W["bigram"][1])
    assert np.allclose(ps.embed([4, 2], W, {"embedding": {"scale": 2.0, "bigram": None}}), 2.0 * W["embed"][[4, 2]])


def test_ramp_over_the_frequencies():
    """Pairs below the ramp keep their frequency, pairs above it are slowed by the factor, and cos and sin grow by
    0.1 ln(factor) + 1; without scaling nothing changes."""
    plain, one = ps.rotation_frequencies({"base": 100.0, "dims": 8})
    assert one == 1.0 and np.allclose(plain, 100.0 ** (-np.arange(4) / 4.0))
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mag = ps.rotation_frequencies(rot)
    lo = math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0)))
    hi = math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0)))
    assert (lo, hi) == (0, 3) and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    ramp = np.clip((np.arange(4) - lo) / (hi - lo), 0, 1)
    assert np.allclose(f, plain * (1 - ramp) + plain / 4.0 * ramp)
    assert f[0] == plain[0] and np.isclose(f[3], plain[3] / 4.0)
    # rotate-half layout: dimension i turns with dimension i + dims / 2; dimensions past `dims` pass
    x = np.zeros((1, 1, 10))
    x[0, 0, 0], x[0, 0, 9] = 1.0, 5.0
    out = ps.rotate_halves(np.repeat(x, 2, axis=0), np.array([0.0, 3.0]), rot)
    assert np.allclose(out[0, 0], mag * x[0, 0] * (np.arange(10) < 8) + x[0, 0] * (np.arange(10) >= 8))
    assert np.allclose(out[1, 0, [0, 4]], [mag * np.cos(3.0 * f[0]), mag * np.sin(3.0 * f[0])]) and out[1, 0, 9] == 5.0


def test_attention_row_by_row():
    """The oracle's dense form against one query at a time: p_j = exp(s_j) / (exp(sink) + sum exp(s_j)), values that
    are the keys before rotation, a gate per head."""
    rng = np.random.RandomState(1)
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 6, "scale": 0.4, "rot": {"base": 30.0, "dims": 4}}
    D, T = 12, 11
    W = {"q": rng.randn(24, D), "k": rng.randn(12, D), "g": rng.randn(4, D), "o": rng.randn(D, 24), "sink": np.array([-3.0, 0.0, 1.5, 6.0])}
    h = rng.randn(T, D)
    got = ps.attend(h, W, "", m)
    f = 30.0 ** (-np.arange(2) / 2.0)

    def turn(x, p):
        out = x.copy()
        out[0:2] = x[0:2] * np.cos(p * f) - x[2:4] * np.sin(p * f)
        out[2:4] = x[2:4] * np.cos(p * f) + x[0:2] * np.sin(p * f)
        return out

    want = np.zeros((T, D))
    for i in range(T):
        heads = []
        for head in range(4):
            kv = head // 2
            q = turn((W["q"] @ h[i])[head * 6:(head + 1) * 6], i)
            raw_k = [(W["k"] @ h[j])[kv * 6:(kv + 1) * 6] for j in range(i + 1)]
            s = np.array([0.4 * q @ turn(raw_k[j], j) for j in range(i + 1)])
            p = np.exp(s) / (np.exp(W["sink"][head]) + np.exp(s).sum())
            o = sum(p[j] * raw_k[j] for j in range(i + 1))
            heads.append(o / (1 + np.exp(-(W["g"] @ h[i])[head])))
        want[i] = W["o"] @ np.concatenate(heads)
    assert np.abs(got - want).max() < 1e-10
    assert np.abs(ps.attend(h[:1], W, "", m) - want[:1]).max() < 1e-10  # one key, and still the sink's share


def test_linear_attention_equals_its_unrolled_form():
    """The recurrence against the sum it stands for: o_t = sum_j (prod_{j < i <= t} a_i) . k_j (q_t) v_j - the decay
    of step t acts before that step's write, and on the key channels."""
    rng = np.random.RandomState(2)
    m = {"heads": 2, "dim": 3, "vdim": 4, "tau": 2.5}
    D, T, eps = 7, 9, 1e-5
    W = {"q": rng.randn(6, D), "k": rng.randn(6, D), "v": rng.randn(8, D), "g": rng.randn(8, D), "o": rng.randn(D, 8),
         "a1": rng.randn(2, D), "a2": rng.randn(6, 2), "a2.b": rng.randn(6), "norm": 1 + 0.3 * rng.randn(4)}
    h = rng.randn(T, D)
    got = ps.glide(h, W, "", m, eps)
    a = (1 / (1 + np.exp(-((h @ W["a1"].T) @ W["a2"].T + W["a2.b"])))) ** (1 / 2.5)
    assert np.allclose(a.reshape(T, 2, 3), ps.channel_decay(h, W, "", m))
    q, k, v = (h @ W["q"].T) / math.sqrt(3), h @ W["k"].T, h @ W["v"].T
    want = np.zeros((T, D))
    for t in range(T):
        heads = []
        for head in range(2):
            c = slice(head * 3, head * 3 + 3)
            o = np.zeros(4)
            for j in range(t + 1):
                keep = np.prod(a[j + 1:t + 1, c], axis=0)
                o += ((q[t, c] * keep) @ k[j, c]) * v[j, head * 4:head * 4 + 4]
            heads.append(o / np.sqrt(np.mean(o * o) + eps) * W["norm"])
        gate = h[t] @ W["g"].T
        want[t] = W["o"] @ (np.concatenate(heads) * gate / (1 + np.exp(-gate)))
    assert np.abs(got - want).max() < 1e-9
    # a carried state: two halves give the whole
    first, S = ps.glide(h[:4], W, "", m, eps, state=np.zeros((2, 3, 4)))
    second, _ = ps.glide(h[4:], W, "", m, eps, state=S)
    assert np.abs(np.concatenate([first, second]) - got).max() < 1e-10


def test_routing_scores_all_experts_and_the_correction_only_chooses():
    W = {"router": np.eye(4), "correction": np.array([0.0, 0.0, 0.0, 0.9])}
    h = np.array([[2.0, 1.0, 0.0, -1.0]])
    chosen, weights, margin = ps.route(h, W, "", {"top": 2, "scale": 3.0})
    s = np.exp(h[0]) / np.exp(h[0]).sum()
    assert chosen.tolist() == [[3, 0]]   # the correction lifts the weakest expert to the top
    assert np.allclose(weights[0], np.array([s[3], s[0]]) / (s[3] + s[0]) * 3.0)   # but its weight is its own score
    assert np.isclose(margin[0], s[0] - s[1])
    _, all_of_them, none_left = ps.route(h, W, "", {"top": 4, "scale": 1.0})
    assert np.allclose(all_of_them.sum(axis=1), 1.0) and np.isinf(none_left[0])


def test_pass_through_experts_and_the_shared_experts_gate():
    rng = np.random.RandomState(4)
    D = 6
    mlp = {"router": {"experts": 1, "identity": 2, "top": 2, "scale": 1.5}, "shared": {"ff": 5}}
    W = {"router": rng.randn(3, D), "correction": np.array([-9.0, 0.0, 0.0]), "e0.up": rng.randn(4, D), "e0.down": rng.randn(D, 4),
         "shared.up": rng.randn(5, D), "shared.down": rng.randn(D, 5), "shared.sg": rng.randn(1, D)}
    h = rng.randn(3, D)
    got = ps.mixture_of_experts(h, W, "", mlp)
    z = h @ W["shared.up"].T
    shared = (0.5 * z * (1 + np.vectorize(math.erf)(z / math.sqrt(2)))) @ W["shared.down"].T
    want = 1.5 * h + shared / (1 + np.exp(-(h @ W["shared.sg"].T)))   # both chosen experts hand h on; weights sum to the scale
    assert np.abs(got - want).max() < 1e-10


def test_offset_norm_adds_one_to_the_stored_weight():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(ps.offset_norm(x, np.array([0.0, -0.5]), 0.0), x / math.sqrt(12.5) * [1.0, 0.5])


@pytest.mark.parametrize("name", list(ts.CONFIGS))
def test_configuration_round_trip_and_tensor_list(name):
    raw = ts.CONFIGS[name]()
    config = config_from_dict(raw)
    assert isinstance(config, SopanexConfig)
    again = config_from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config
    from cpp_minilamma_b200.engine.model import Model
    import torch
    model = Model(build_sopanex_spec(config), torch.float32, "cpu", max_positions=8)
    listed = {s.name: tuple(s.shape) for s in model.weight_specs() if not s.optional}
    assert listed == ts.tensor_shapes(raw)
    # without the decay's inner size in the configuration the tensors' own size stands
    for lay in raw["layers"]:
        lay["mixer"]["right"].pop("decay_rank")
    bare = Model(build_sopanex_spec(config_from_dict(raw)), torch.float32, "cpu", max_positions=8)
    assert {s.shape for s in bare.weight_specs() if s.name == "l0.mix.right.a1"} == {(-1, raw["width"])}


def test_configuration_faults_are_named():
    good = ts.CONFIGS["mixed"]()
    for change, word in [(lambda c: c["layers"][0].update(type="serial"), "type"),
                         (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
                         (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=16), "vdim"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=0), "factor"),
                         (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=10), "top"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="dense"), "kind"),
                         (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
                         (lambda c: c.pop("norm"), "norm")]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            config_from_dict(raw)
        assert word in str(caught.value)


def test_oracle_forward_shapes_and_layer_trace():
    raw = ts.CONFIGS["mixed"]()
    W = {k: v.astype(np.float64) for k, v in ts.make_weights(raw, 3).items()}
    toks = ts.tokens(raw, 20, 1)
    logits, after = ps.forward(raw, W, toks, with_layers=True)
    assert logits.shape == (20, raw["vocab"]) and after.shape == (4, 20, raw["width"])
    assert np.abs(ps.forward(raw, W, toks[:9]) - logits[:9]).max() < 1e-9  # causal: a prefix gives the same logits


def test_command_line_random_then_inspect(tmp_path, capsys):
    """`random` writes a folder from a configuration file (every tensor of the list, bfloat16), `inspect` reads it
    back, and the oracle can run it."""
    from cpp_minilamma_b200.cli import main
    raw = ts.CONFIGS["mixed"]()
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(raw))
    assert main(["random", str(tmp_path / "m"), "--config", str(cfg), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "architecture: Sopanex" in out and "status=ok" in out
    assert "tensor l1.mlp.e6.down [56, 16] bfloat16" in out and "tensor bigram [258, 56] bfloat16" in out
    assert "tensor l3.mix.right.a2 [16, 8] bfloat16" in out and "tensor l0.mix.left.sink [6] bfloat16" in out
    config, W = ps.read_folder(tmp_path / "m")
    # a layer without a feed-forward: the folder holds the norms around it all the same (zeros would do)
    assert set(W) - set(ts.tensor_shapes(raw)) == {"l2.norm2", "l2.norm2b"}
    logits = ps.forward(config, W, ts.tokens(raw, 12, 5))
    assert logits.shape == (12, raw["vocab"]) and np.isfinite(logits).all()
