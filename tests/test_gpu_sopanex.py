"""Sopanex through the engine against the plain oracle (`plain_sopanex`, float64, whole sequences).

Every test makes its own small configuration and weights (`tiny_sopanex`).  float32 runs must agree with the oracle
to 2e-4 of the largest logit (at least 2e-4 absolute): with the test weights a sink left out, a pair row one token
off, a lost state, one key wrongly seen or missed, a wrong expert or a norm left out moves logits by percents.
bfloat16 runs are compared with the same unrounded oracle, so their bound is that of rounding noise: largest error
at most 10 %, mean error at most 2.5 % of the largest logit (the bound of the other designs' tests).  A routed layer
turns a near-tie between two experts into another expert's output once activations are rounded, so in bfloat16 the
oracle also reports every token's smallest margin between the last chosen and the first unchosen choice score: as
many rows may exceed the bound as there are tokens whose margin is below 0.02, and none if there are none.  The
sharp test is float32, where near-ties do not matter."""
import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_sopanex as ps
import tiny_sopanex as ts
from cpp_minilamma_b200.cache.paged import PAGE
from cpp_minilamma_b200.engine.step import StepEntry

pytestmark = pytest.mark.gpu

_FOLDERS, _ENGINES, _ORACLE, _MARGIN = {}, {}, {}, {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    def get(name, dtype="float32", max_tokens=1024, max_positions=None):
        if name not in _FOLDERS:
            _FOLDERS[name] = ts.make_folder(name, tmp_path_factory.mktemp(name), seed=len(_FOLDERS) + 1)
        folder, cfg, W = _FOLDERS[name]
        key = (name, dtype, max_tokens, max_positions)
        if key not in _ENGINES:
            _ENGINES[key] = ml.load(folder, dtype=dtype, max_tokens=max_tokens, max_positions=max_positions)
        return _ENGINES[key], cfg, W
    yield get
    _ENGINES.clear()


def oracle(name, cfg, W, toks):
    key = (name, tuple(toks))
    if key not in _ORACLE:
        margins = []
        _ORACLE[key] = ps.forward(cfg, W, toks, margins=margins)
        _MARGIN[id(_ORACLE[key])] = np.min(margins, axis=0) if margins else None
    return _ORACLE[key]


def close(got, ref, dtype, what, routed=False):
    margin = _MARGIN.get(id(ref))
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err, scale = np.abs(got - ref), max(1.0, np.abs(ref).max())
    row = int(np.argmax(err.max(axis=-1))) if err.ndim == 2 else 0
    if dtype == "float32":
        assert err.max() <= 2e-4 * scale, f"{what}: err {err.max():.3e} of {scale:.2f}, first at row {row}"
        return
    rows = err.max(axis=-1) if err.ndim == 2 else err.max(keepdims=True)
    over = int((rows > 1e-1 * scale).sum())
    allowed = int((margin < 0.02).sum()) if routed and margin is not None and len(margin) == len(rows) else 0
    assert over <= allowed and np.median(rows) <= 5e-2 * scale and err.mean() <= 2.5e-2 * scale, \
        f"{what}: {over} rows over, max {err.max():.3e} mean {err.mean():.3e} of {scale:.2f}, worst row {row}"


def run_alone(llm, toks, cuts):
    """Feed one sequence in portions of the given sizes (the rest one token at a time); logits of every position."""
    slot = llm.engine.acquire(1)[0]
    rows, at = [], 0
    sizes = list(cuts) + [1] * (len(toks) - sum(cuts))
    for n in sizes:
        rows.append(llm.engine.step([StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    llm.engine.release(slot)
    return np.concatenate(rows)


LENGTH = {"left_only": 150, "right_only": 150, "routed": 75, "mixed": 200, "ones": 140, "bare": 100, "tensor": 300, "odd": 90}
ROUTED = {"routed", "mixed", "ones", "tensor", "odd"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ts.CONFIGS))
def test_whole_prompt(models, name, dtype):
    """Every position of one prompt, the first tokens included (the pair table's last row, a state that starts at
    zero, rows in which the sink is most of the denominator); prompts reach over page borders."""
    llm, cfg, W = models(name, dtype)
    toks = ts.tokens(cfg, LENGTH[name], 11)
    close(run_alone(llm, toks, [len(toks)]), oracle(name, cfg, W, toks), dtype, f"{name} whole", name in ROUTED)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ts.CONFIGS))
def test_prompt_then_token_by_token(models, name, dtype):
    """A short prompt, then a long run of single tokens through the cache and the state: over page borders, the
    token before each one read from the sequence's state, the recurrent state carried step by step."""
    llm, cfg, W = models(name, dtype)
    toks = ts.tokens(cfg, LENGTH[name], 12)
    close(run_alone(llm, toks, [7]), oracle(name, cfg, W, toks), dtype, f"{name} decode", name in ROUTED)


def test_token_by_token_from_the_first_token(models):
    """No prompt at all: the very first step brings one token (the pair table's last row, an empty state)."""
    llm, cfg, W = models("mixed", "float32")
    toks = ts.tokens(cfg, 70, 14)
    close(run_alone(llm, toks, []), oracle("mixed", cfg, W, toks), "float32", "mixed from the first token")


@pytest.mark.parametrize("name,cuts", [
    ("mixed", [2, 3, 1, 7, 2, 49, 2, 2, 64]),      # portions down to two tokens, cuts inside and at the end of a page
    ("ones", [1, 1, 62, 2, 66]),                   # single first tokens; a cut at the page's edge and after it
    ("left_only", [8, 8, 7, 2, 39, 64]),
    ("right_only", [63, 1, 2, 64, 17]),            # the state handed from portion to portion
    ("odd", [5, 2, 2, 60]),
    ("routed", [3, 2, 61, 2]),
    ("bare", [2, 2, 2, 58, 2, 30]),
])
def test_portions(models, name, cuts):
    llm, cfg, W = models(name, "float32")
    toks = ts.tokens(cfg, LENGTH[name], 13)
    close(run_alone(llm, toks, cuts), oracle(name, cfg, W, toks), "float32", f"{name} portions {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones", "tensor"])
def test_unequal_batch_then_decoding_together(models, name, dtype):
    """Requests of 1, 37 and 90 tokens start in one step, go on by one token each, and the short ones end early;
    every logit equals that of the request alone (the routed layers sort the batch's tokens by expert, the pair
    rows and the states belong to each request)."""
    llm, cfg, W = models(name, dtype)
    eng = llm.engine
    seqs = [ts.tokens(cfg, n, 20 + i) for i, n in enumerate((9, 50, 104))]
    first = [1, 37, 90]
    slots = eng.acquire(3)
    got = [[] for _ in seqs]
    out = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, first)]).cpu().numpy()
    at = 0
    for i, n in enumerate(first):
        got[i].append(out[at:at + n])
        at += n
    done = list(first)
    live = [0, 1, 2]
    while live:
        out = eng.step([StepEntry(slots[i], [seqs[i][done[i]]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
            done[i] += 1
        for i in [i for i in live if done[i] == len(seqs[i])]:
            eng.release(slots[i])
            live.remove(i)
    for i, q in enumerate(seqs):
        close(np.concatenate(got[i]), oracle(name, cfg, W, q), dtype, f"{name} request {i} in a batch", True)
    eng.cache.check()


def test_slots_pages_and_states_used_again(models):
    """A cache of four pages: a sequence of three and a half pages, then - in the same slot, pages and state rows,
    handed out in another order - a second one, while a third short request comes and goes beside them.  A state or
    a previous token left behind by the first sequence would show in the second one's first rows."""
    llm, cfg, W = models("mixed", "float32", max_tokens=5 * PAGE, max_positions=4 * PAGE)
    eng = llm.engine
    for seed in (31, 32):
        toks = ts.tokens(cfg, 3 * PAGE + 30, seed)
        short = ts.tokens(cfg, 20, seed + 10)
        slot = eng.acquire(1)[0]
        rows = []
        for at in range(0, len(toks), 50):
            part = toks[at:at + 50]
            rows.append(eng.step([StepEntry(slot, part, list(range(len(part))))]).cpu().numpy())
            if at == 50:  # a neighbour that takes a page and gives it back
                other = eng.acquire(1)[0]
                got = eng.step([StepEntry(other, short, list(range(20)))]).cpu().numpy()
                eng.release(other)
                close(got, oracle("mixed", cfg, W, short), "float32", "the neighbour")
        eng.release(slot)
        eng.cache.check()
        close(np.concatenate(rows), oracle("mixed", cfg, W, toks), "float32", f"long sequence, seed {seed}")
    assert all(g.pool.n_free == g.pool.n_pages for g in eng.cache.groups)


def test_an_engine_cuts_a_long_step_itself(models):
    models("mixed")
    folder, cfg, W = _FOLDERS["mixed"]
    llm = ml.load(folder, dtype="float32", max_tokens=512, max_step_tokens=64)
    toks = ts.tokens(cfg, 150, 41)
    close(run_alone(llm, toks, [150]), oracle("mixed", cfg, W, toks), "float32", "engine-cut step")


def greedy_oracle(cfg, W, prompt, n):
    toks, out, sure = list(prompt), [], []
    for _ in range(n):
        logits = ps.forward(cfg, W, toks)[-1]
        best = int(np.argmax(logits))
        sure.append(logits[best] - np.partition(logits, -2)[-2] > 1e-3)
        out.append(best)
        toks.append(best)
    return out, sure


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`generate` (the scheduler, captured decode steps, device sampling, the step enqueued ahead whose tokens are
    gathered on the device - the pair embedding reads them there) picks the oracle's tokens."""
    llm, cfg, W = models(name, "float32")
    prompts = [ts.tokens(cfg, n, 50 + i) for i, n in enumerate((3, 21, 66))]
    outs = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    for prompt, got in zip(prompts, outs):
        want, sure = greedy_oracle(cfg, W, prompt, 14)
        upto = sure.index(False) if False in sure else len(sure)  # after a near-tie either token is right
        assert got[:upto] == want[:upto], (got, want)
    again = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    assert again == outs  # slots, pages and states of finished requests serve the next ones
    llm.engine.cache.check()


def test_bfloat16_generation_replays_captured_steps(models):
    """Decode steps of the bfloat16 engine run from CUDA graphs (the pair embedding, both mixers, routing, sorting
    and the expert products included) and give the tokens of the same engine stepping eagerly."""
    llm, cfg, W = models("tensor", "bfloat16")
    assert llm.model.capturable()
    prompts = [ts.tokens(cfg, n, 80 + i) for i, n in enumerate((5, 40))]
    outs = llm.generate(prompts, max_new_tokens=24, ignore_eos=True)
    eng = llm.engine
    for prompt, got in zip(prompts, outs):
        slot = eng.acquire(1)[0]
        logits = eng.step([StepEntry(slot, prompt, [len(prompt) - 1])])
        stepped = []
        for _ in range(24):
            top2 = torch.topk(logits[0], 2).values
            if float(top2[0] - top2[1]) < 0.05:  # a near-tie: rounding may fall either way from here on
                break
            stepped.append(int(torch.argmax(logits[0])))
            logits = eng.step([StepEntry(slot, [stepped[-1]], [0])])
        eng.release(slot)
        assert got[:len(stepped)] == stepped


def test_command_line_generates_the_oracles_tokens(models, capsys):
    from cpp_minilamma_b200.cli import main
    _, cfg, W = models("ones", "float32")
    folder = _FOLDERS["ones"][0]
    prompt = ts.tokens(cfg, 5, 60)
    assert main(["generate", folder, "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                 "--ignore-eos"]) == 0
    line = capsys.readouterr().out.splitlines()[0]
    want, sure = greedy_oracle(cfg, W, prompt, 6)
    upto = sure.index(False) if False in sure else len(sure)
    assert [int(t) for t in line.split()][:upto] == want[:upto]


def test_trace_replay_writes_the_wanted_logits(models, tmp_path):
    """The trace runner on a Sopanex folder: two requests start together, decode, one ends early."""
    import json
    import os
    import subprocess
    import sys
    _, cfg, W = models("mixed", "float32")
    folder = _FOLDERS["mixed"][0]
    a, b = ts.tokens(cfg, 30, 70), ts.tokens(cfg, 70, 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:28], "want": [0, 27]},
                                     {"id": "b", "tokens": b[:66], "want": [65]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[28:29], "want": []},
                                     {"id": "b", "tokens": b[66:67], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[29:30], "want": [0]},
                                     {"id": "b", "tokens": b[67:68], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[68:70], "want": [1]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "256"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    ra, rb = oracle("mixed", cfg, W, a), oracle("mixed", cfg, W, b)
    want = {0: [ra[0], ra[27], rb[65]], 1: [rb[66]], 2: [ra[29], rb[67]], 3: [rb[69]]}
    for n, rows in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), -1)
        close(got, np.stack(rows), "float32", f"trace step {n}")


# --------------------------------------------------------------------------------------------------------------- #
# kernels alone                                                                                                   #
# --------------------------------------------------------------------------------------------------------------- #
def _paged(gen, ctxs, G, d, dtype):
    """Key and value caches with every sequence's pages in shuffled order."""
    n_pages = sum(-(-c // PAGE) for c in ctxs) + 3
    k_cache = (torch.randn((n_pages, G, PAGE, d), generator=gen) * 0.5).to(dtype)
    v_cache = torch.randn((n_pages, G, PAGE, d), generator=gen).to(dtype)
    order = torch.randperm(n_pages, generator=gen).tolist()
    table = torch.full((len(ctxs), max(-(-c // PAGE) for c in ctxs)), -1, dtype=torch.int32)
    at = 0
    for s, c in enumerate(ctxs):
        blocks = -(-c // PAGE)
        table[s, :blocks] = torch.tensor(order[at:at + blocks], dtype=torch.int32)
        at += blocks
    return k_cache, v_cache, table


def _dense(cache, table, s, ctx):
    return torch.stack([cache[int(table[s, p // PAGE]), :, p % PAGE] for p in range(ctx)]).double()  # [ctx, G, d]


def _sink_attention(q, keys, values, pos0, scale, sinks, group):
    """q [n, H, d] at positions pos0 ..; keys, values [ctx, G, d]; weights exp(s_j) / (exp(sink_h) + sum exp(s))."""
    n, H, _ = q.shape
    out = torch.zeros((n, H, values.shape[-1]), dtype=torch.float64)
    for i in range(n):
        for h in range(H):
            s = scale * keys[:pos0 + i + 1, h // group] @ q[i, h]
            top = max(float(s.max()), float(sinks[h]))
            e = torch.exp(s - top)
            out[i, h] = (e / (e.sum() + np.exp(float(sinks[h]) - top))) @ values[:pos0 + i + 1, h // group]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d", [(4, 2, 16), (3, 1, 48), (2, 2, 72), (5, 1, 6), (8, 2, 64), (2, 1, 128)])
def test_attention_kernels_with_a_learned_sink_and_a_far_key(dtype, H, G, d):
    """The general kernel (both dtypes), the tensor-core prompt kernel and the single-token kernel with heads as rows
    (bfloat16) against the softmax written out: three sequences that start at positions 0, 70 and 300, one of them a
    single token.  In every sequence one early key (hundreds back, in a page of its own) is scaled so that its score
    stands out; the sinks run from far below the scores (no share) to above all of them (most of the row)."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d * 1000 + H)
    starts, lens = [0, 70, 300], [150, 61, 1]
    ctxs = [s + n for s, n in zip(starts, lens)]
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, dtype)
    T = sum(lens)
    q = torch.randn((T, H * d), generator=gen).to(dtype)
    for s in range(3):  # the far key points along the queries' mean direction
        far = 1 + 2 * s
        page = int(table[s, 0])
        rows = slice(sum(lens[:s]), sum(lens[:s + 1]))
        mean_q = q[rows].float().view(-1, H, d).mean(dim=(0, 1))
        k_cache[page, :, far, :] = (k_cache[page, :, far, :].float() + 6.0 * mean_q / mean_q.norm()).to(dtype)
    sinks = torch.linspace(-6.0, 4.0, H)
    scale = 1.0 / d ** 0.5
    want = []
    for s in range(3):
        rows = slice(sum(lens[:s]), sum(lens[:s + 1]))
        want.append(_sink_attention(q[rows].double().view(-1, H, d), _dense(k_cache, table, s, ctxs[s]),
                                    _dense(v_cache, table, s, ctxs[s]), starts[s], scale, sinks, H // G))
    want = torch.cat(want).view(T, H * d)
    no_sink = torch.cat([_sink_attention(q[slice(sum(lens[:s]), sum(lens[:s + 1]))].double().view(-1, H, d),
                                         _dense(k_cache, table, s, ctxs[s]), _dense(v_cache, table, s, ctxs[s]), starts[s],
                                         scale, torch.full((H,), -1e9), H // G) for s in range(3)]).view(T, H * d)
    assert (want - no_sink).abs().max().item() > 0.2 * want.abs().max().item()  # the sink matters in this test
    state = make_step_state(dev, [0, 1, 2], starts, lens)
    kc, vc, table_dev, qd, sd = k_cache.to(dev), v_cache.to(dev), table.to(dev), q.to(dev), sinks.to(dev)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    plain = torch.zeros((T, H * d), dtype=dtype, device=dev)
    K.local_attention(qd, kc, vc, state.tok_pos, state.tok_seq, state.seq_slot, table_dev, plain, H, G, d, d, 0, 0, scale,
                      sink=True, sink_values=sd)
    torch.cuda.synchronize()
    err = (plain.cpu().double() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), ("general kernel", err)
    if dtype != torch.bfloat16 or not K.local_attention_mma_supported(dtype, d, d):
        return
    tile_seq = [s for s, n in enumerate(lens) for _ in range(0, n, K.PREFILL_TILE)]
    tile_row0 = [r for n in lens for r in range(0, n, K.PREFILL_TILE)]
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=dev)
    fast = torch.zeros_like(plain)
    K.local_attention_tiles(qd, kc, vc, state.seq_slot, state.seq_ctx, state.seq_qstart, state.seq_qlen, ints(tile_seq),
                            ints(tile_row0), table_dev, fast, H, G, d, d, 0, 0, scale, sink=True, sink_values=sd)
    torch.cuda.synchronize()
    err = (fast.cpu().double() - want).abs().max().item()
    assert err <= 3e-2 * max(1.0, want.abs().max().item()), ("tensor-core prompt kernel", err)
    # single tokens: the last token of every sequence, one block a sequence and the context split in 3 and in 16
    last = [sum(lens[:i + 1]) - 1 for i in range(3)]
    one = make_step_state(dev, [0, 1, 2], [c - 1 for c in ctxs], [1, 1, 1])
    for splits in (1, 3, 16):
        out = torch.zeros((3, H * d), dtype=dtype, device=dev)
        scratch = torch.full((K.local_attention_heads_scratch(3, H, d, splits),), float("nan"), device=dev)
        K.local_attention_heads(qd[last].contiguous(), kc, vc, one.seq_slot, one.seq_ctx, one.seq_qstart, one.seq_qlen,
                                table_dev, out, 3, H, G, d, d, 0, 0, scale, sink=True, n_splits=splits,
                                scratch=scratch if splits > 1 else None, sink_values=sd)
        torch.cuda.synchronize()
        err = (out.cpu().double() - want[last]).abs().max().item()
        assert err <= 3e-2 * max(1.0, want.abs().max().item()), ("heads as rows", splits, err)


@pytest.mark.parametrize("d,rot", [(16, 16), (24, 12), (8, 2), (10, 0)])
def test_prepare_writes_unrotated_keys_as_values(d, rot):
    """q and k rotated over their first `rot` dimensions in pairs (i, i + rot / 2), the rest passed on; the value
    pages receive the keys as projected."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    H, G = 3, 1
    positions = [0, 1, 63, 64, 65, 200]
    n = len(positions)
    gen = torch.Generator().manual_seed(d)
    qkv = torch.randn((n, H * d + G * d + 5), generator=gen).to(dev)   # 5 more columns behind k (a gate's)
    k_cache = torch.zeros((n + 1, G, PAGE, d), device=dev)
    v_cache = torch.zeros((n + 1, G, PAGE, d), device=dev)
    table = torch.full((n, 4), -1, dtype=torch.int32)
    for s, p in enumerate(positions):
        table[s, p // PAGE] = s
    state = make_step_state(dev, list(range(n)), positions, [1] * n)
    half = rot // 2
    freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(half)], dtype=torch.float64) if rot else None
    cos = sin = None
    if rot:
        angle = torch.arange(256, dtype=torch.float64)[:, None] * freq
        cos, sin = (1.3 * torch.cos(angle)).float().to(dev), (1.3 * torch.sin(angle)).float().to(dev)
    q = torch.zeros((n, H * d), device=dev)
    K.local_attention_prepare(qkv, None, None, cos, sin, state.tok_pos, state.tok_seq, state.seq_slot, table.to(dev), q,
                              k_cache, v_cache, H, G, d, d, rot, False, 0.0, v_from_k=True)
    torch.cuda.synchronize()

    def turned(x, p):  # x [heads, d] float64
        out = x.clone()
        if rot:
            c, s = 1.3 * torch.cos(p * freq), 1.3 * torch.sin(p * freq)
            u, v = x[:, :half], x[:, half:rot]
            out[:, :half], out[:, half:rot] = u * c - v * s, v * c + u * s
        return out

    for s, p in enumerate(positions):
        row = qkv[s].cpu().double()
        assert (q[s].cpu().double().view(H, d) - turned(row[:H * d].view(H, d), p)).abs().max().item() < 1e-5
        assert (k_cache[s, :, p % PAGE].cpu().double() - turned(row[H * d:H * d + G * d].view(G, d), p)).abs().max().item() < 1e-5
        assert torch.equal(v_cache[s, :, p % PAGE].cpu(), qkv[s, H * d:H * d + G * d].view(G, d).cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_kernel(dtype):
    """Rows of the pair table for first tokens (the last row), tokens inside a step (the token before is in the step)
    and a step's first token (the token before is the slot's state), with multipliers large enough that the hash
    needs 64-bit arithmetic; the state afterwards holds each sequence's last token."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(3)
    vocab, width, buckets, mp, mc, scale = 50000, 24, 1013, 123457, 98765, 2.5
    table = torch.randn((vocab, width), generator=gen).to(dtype)
    pairs = torch.randn((buckets + 1, width), generator=gen).to(dtype)
    slots, starts, lens = [4, 1, 6], [0, 17, 1], [5, 3, 1]
    toks = torch.randint(0, vocab, (sum(lens),), generator=gen).tolist()
    before = torch.tensor([7, 40000, 0, 0, 11, 0, 49999, 0], dtype=torch.int32)
    state = make_step_state(dev, slots, starts, lens, tokens=toks)
    prev = before.clone().to(dev)
    x = torch.zeros((len(toks), width), device=dev)
    K.embedding_pair(torch.tensor(toks, dtype=torch.int32, device=dev), state.tok_pos, state.tok_seq, state.seq_slot,
                     state.seq_qstart, state.seq_qlen, prev, table.to(dev), pairs.to(dev), x, buckets, mp, mc, scale)
    torch.cuda.synchronize()
    at = 0
    for slot, start, n in zip(slots, starts, lens):
        for i in range(n):
            pos, tok = start + i, toks[at + i]
            earlier = toks[at + i - 1] if i else int(before[slot])
            row = buckets if pos == 0 else (mp * earlier + mc * tok) % buckets
            want = scale * table[tok].double() + pairs[row].double()
            assert (x[at + i].cpu().double() - want).abs().max().item() < 1e-5, (slot, i)
        assert int(prev[slot]) == toks[at + n - 1]
        at += n
    assert int(prev[0]) == 7  # other slots are left alone


@pytest.mark.parametrize("width", [40, 50, 256, 1000, 4096, 9000])
def test_norm_kernel_with_a_normed_delta(width):
    """x += norm_a(c1 d1 + c2 d2); out = norm_b(x): against the same written out, with and without the second delta,
    and for gathered rows (which leave the stream alone)."""
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(width)
    x0 = (torch.randn((9, width), generator=gen) * 3).to(dev)
    d1 = torch.randn((9, width), generator=gen).to(torch.bfloat16).to(dev)
    d2 = (torch.randn((9, width), generator=gen) * 2).to(torch.bfloat16).to(dev)
    wa, wb = (1 + 0.3 * torch.randn((width,), generator=gen)).to(dev), (1 + 0.3 * torch.randn((width,), generator=gen)).to(dev)
    for second, c1, c2, normed in ((d2, 1.2, 0.5, True), (None, 1.0, 1.0, True), (d2, 0.7, 1.9, False)):
        d = c1 * d1.cpu().double() + (c2 * second.cpu().double() if second is not None else 0.0)
        if normed:
            d = d / torch.sqrt((d * d).mean(dim=1, keepdim=True) + 1e-5) * wa.cpu().double()
        summed = x0.cpu().double() + d
        want = summed / torch.sqrt((summed * summed).mean(dim=1, keepdim=True) + 1e-6) * wb.cpu().double()
        form = K.DeltaNorm(wa if normed else None, 1e-5 if normed else 0.0, c1, c2)
        x = x0.clone()
        rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=dev)
        gathered = torch.zeros((3, width), dtype=torch.float32, device=dev)
        K.add_rmsnorm(x, d1, wb, gathered, 1e-6, rows, delta2=second, delta_norm=form)
        assert torch.equal(x, x0)
        assert (gathered.cpu().double() - want[[8, 0, 3]]).abs().max().item() < 3e-5
        out = torch.zeros((9, width), dtype=torch.float32, device=dev)
        K.add_rmsnorm(x, d1, wb, out, 1e-6, delta2=second, delta_norm=form)
        assert (x.cpu().double() - summed).abs().max().item() < 1e-5
        assert (out.cpu().double() - want).abs().max().item() < 3e-5


@pytest.mark.parametrize("H,d,dv", [(2, 8, 12), (3, 6, 10), (1, 64, 64), (2, 128, 32), (4, 32, 128), (1, 40, 8), (1, 200, 24),
                                    (8, 128, 128), (8, 64, 128), (4, 200, 256)])  # the last three: eight lanes a column; before them a warp or half a warp
def test_channel_decay_recurrence(H, d, dv):
    """channel_decay_prepare + state_scan + head_norm_gate against the recurrence walked token by token in float64:
    three sequences of 150, 1 and 37 tokens, two of which go on from a state that is not zero; decays from quick
    forgetting (a very negative bias) to none (a very positive one), which a decay applied to the wrong side of S,
    or after the write instead of before it, would show."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(H * 100 + d)
    lens, slots = [150, 1, 37], [2, 0, 3]
    T, tau, eps = sum(lens), 3.0, 1e-5
    ld = H * (2 * d + dv) + H * dv + 3
    proj = torch.randn((T, ld), generator=gen).to(dev)
    rate = (torch.randn((T, H * d + 2), generator=gen) * 2).to(dev)
    bias = torch.randn((H * d,), generator=gen) * 2
    bias[0], bias[-1] = -30.0, 30.0
    norm_w = 1 + 0.3 * torch.randn((dv,), generator=gen)
    S0 = torch.randn((5, H, d, dv), generator=gen)
    S0[2] = 0.0
    state_buf = S0.clone().to(dev)
    q, k, g = (torch.zeros((T, H * d), device=dev) for _ in range(3))
    v = torch.zeros((T, H * dv), device=dev)
    K.channel_decay_prepare(proj, rate, bias.to(dev), q, k, v, g, H, d, dv, d ** -0.5, tau)
    o = torch.zeros((T, H * dv), device=dev)
    st = make_step_state(dev, slots, [0, 9, 20], lens)
    K.state_scan(q, k, v, g, None, None, state_buf, o, st.seq_slot, st.seq_qstart, st.seq_qlen, 3, H, H, d, dv)
    out = torch.zeros((T, H * dv), device=dev)
    K.head_norm_gate(o, norm_w.to(dev), proj, out, H, dv, eps, K.GATE_SILU, gate_col=H * (2 * d + dv))
    torch.cuda.synchronize()
    P = proj.cpu().double()
    z = rate.cpu().double()[:, :H * d] + bias.double()
    a = torch.exp(-torch.log1p(torch.exp(-z)) / tau).view(T, H, d)
    qq, kk = (P[:, :H * d] * d ** -0.5).view(T, H, d), P[:, H * d:2 * H * d].view(T, H, d)
    vv = P[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
    gate = P[:, H * (2 * d + dv):H * (2 * d + dv) + H * dv].view(T, H, dv)
    at = 0
    for slot, n in zip(slots, lens):
        S = S0[slot].double().clone()
        for t in range(at, at + n):
            S = a[t][:, :, None] * S + kk[t][:, :, None] * vv[t][:, None, :]
            ot = torch.einsum("hdv,hd->hv", S, qq[t])
            assert (o[t].cpu().double().view(H, dv) - ot).abs().max().item() <= 2e-4 * max(1.0, ot.abs().max().item()), (slot, t - at)
            want = ot / torch.sqrt((ot * ot).mean(dim=1, keepdim=True) + eps) * norm_w.double() * (gate[t] / (1 + torch.exp(-gate[t])))
            assert (out[t].cpu().double().view(H, dv) - want).abs().max().item() <= 2e-4 * max(1.0, want.abs().max().item())
        assert (state_buf[slot].cpu().double() - S).abs().max().item() <= 2e-4 * max(1.0, S.abs().max().item())
        at += n
    assert torch.equal(state_buf[1].cpu(), S0[1]) and torch.equal(state_buf[4].cpu(), S0[4])  # other slots are left alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,I,top,D,F", [(1, 5, 2, 3, 40, 24), (37, 7, 1, 3, 56, 16), (300, 2, 1, 3, 50, 30), (64, 1, 0, 1, 32, 8),
                                           (200, 30, 3, 4, 64, 72), (1500, 6, 2, 2, 128, 64), (90, 3, 4, 2, 48, 40)])
def test_routed_kernels_with_scores_over_all_experts(dtype, T, E, I, top, D, F):
    """route / sort / up / down / combine in the form with scores over every expert, a correction that moves the
    choice but not the weights, a scale on the weights, pass-through experts behind the real ones, gelu experts and
    a gate per token on the other part's output - against the sum written out; for one token, many tokens per
    expert (tensor-core tiles in bfloat16), every expert per token, a single expert, and more pass-through experts
    than real ones.  One real expert's correction is pushed down so that it gets no token at all."""
    import math
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(T * 31 + E)
    R = E + I
    h = torch.randn((T, D), generator=gen).to(dtype)
    router = torch.randn((R + 1, D), generator=gen) * 2 / D ** 0.5   # the last row is the other part's gate
    corr = torch.randn((R,), generator=gen) * 0.2
    if R > top + 1 and E > 1:
        corr[E // 2] = -50.0
    up = (torch.randn((E, F, D), generator=gen) * 1.5 / D ** 0.5).to(dtype)
    down = (torch.randn((E, D, F), generator=gen) / F ** 0.5).to(dtype)
    other = torch.randn((T, D), generator=gen).to(dtype)
    scale = 1.7
    z = h.double() @ router.double().T
    s = torch.softmax(z[:, :R], dim=1)
    choice = s + corr.double()
    chosen_ref = torch.argsort(-choice, dim=1, stable=True)[:, :top]
    sc = torch.gather(s, 1, chosen_ref)
    w_ref = sc / (sc.sum(dim=1, keepdim=True) + 1e-20) * scale
    gate_ref = torch.sigmoid(z[:, R])
    want = other.double() * gate_ref[:, None]
    for t in range(T):
        for j in range(top):
            e = int(chosen_ref[t, j])
            if e >= E:
                want[t] += w_ref[t, j] * h[t].double()
                continue
            u = up[e].double() @ h[t].double()
            act = 0.5 * u * (1 + torch.erf(u / math.sqrt(2.0)))
            if dtype == torch.bfloat16:
                act = act.to(torch.bfloat16).double()
            want[t] += w_ref[t, j] * (down[e].double() @ act)
    chosen = torch.zeros((T, top), dtype=torch.int32, device=dev)
    weight = torch.zeros((T, top), dtype=torch.float32, device=dev)
    gate = torch.zeros((T,), dtype=torch.float32, device=dev)
    hd = h.to(dev)
    K.moe_route(hd, router.to(dev), corr.to(dev), chosen, weight, top, all_scores=True, scale=scale, gate_out=gate)
    torch.cuda.synchronize()
    ranked = torch.sort(choice, dim=1, descending=True).values
    sure = (ranked[:, top - 1] - ranked[:, top]) > 1e-5 if R > top else torch.ones(T, dtype=torch.bool)
    assert torch.equal(chosen.cpu().long()[sure], chosen_ref[sure])
    assert (weight.cpu().double()[sure] - w_ref[sure]).abs().max().item() < 1e-5
    assert (gate.cpu().double() - gate_ref).abs().max().item() < 1e-5
    logits = (h.float().to(dev) @ router.to(dev).T).contiguous()  # the caller's own product of the logits
    chosen2, weight2, gate2 = torch.zeros_like(chosen), torch.zeros_like(weight), torch.zeros_like(gate)
    K.moe_route(hd, router.to(dev), corr.to(dev), chosen2, weight2, top, logits=logits, all_scores=True, scale=scale, gate_out=gate2)
    torch.cuda.synchronize()
    assert torch.equal(chosen2.cpu()[sure], chosen.cpu()[sure]) and (gate2 - gate).abs().max().item() < 1e-5
    for mma, small in ([(False, 0), (True, 0), (True, 1), (True, 2)] if K.moe_mma_supported(dtype, D, F) else [(False, 0)]):
        rows = K.moe_tile_rows(mma, (1 << 30, 1, 20)[small], 1)  # the tensor-core kernels' tiles of 128, 16 and 32 rows
        n_pairs = T * top
        tiles = K.moe_max_tiles(n_pairs, R, rows)
        ints = lambda n: torch.full((n,), -7, dtype=torch.int32, device=dev)
        plan = K.MoePlan(ints(n_pairs), ints(R + 1), ints(tiles), ints(tiles), ints(1), rows, mma)
        K.moe_sort(chosen, plan, R, n_real=E)
        act = torch.zeros((n_pairs, F), dtype=dtype, device=dev)
        K.moe_gate_up(hd, up.to(dev), act, plan, top, form=K.EXPERT_GELU, n_experts=R)
        y = torch.full((n_pairs, D), float("nan"), dtype=torch.float32, device=dev)  # rows of pass-through choices stay unwritten
        K.moe_down(act, down.to(dev), y, weight, plan, top, n_experts=R)
        out = torch.zeros((T, D), dtype=dtype, device=dev)
        K.moe_combine(y, other.to(dev), out, top, chosen=chosen, pair_weight=weight, h=hd, n_real=E, other_gate=gate)
        torch.cuda.synchronize()
        counts = torch.bincount(chosen.cpu().view(-1).long(), minlength=R).tolist()
        offsets = plan.offsets.cpu().tolist()
        assert [b - a for a, b in zip(offsets, offsets[1:])] == counts
        assert int(plan.n_tiles.cpu()) == sum(-(-c // rows) for c in counts[:E])
        assert torch.isfinite(out.float()).all()
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        err = (out.cpu().double() - want)[sure].abs().max().item()
        assert err <= tol * max(1.0, want.abs().max().item()), (mma, small, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_kernel(dtype):
    import math
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    z = torch.linspace(-9, 9, 1003).to(dtype).to(dev)
    out = torch.zeros_like(z)
    zd = z.cpu().double()
    for kind, want in ((K.ACT_GELU_ERF, 0.5 * zd * (1 + torch.erf(zd / math.sqrt(2.0)))),
                       (K.ACT_GELU_TANH, 0.5 * zd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (zd + 0.044715 * zd ** 3))))):
        K.activation(z, out, kind)
        tol = 1e-6 if dtype == torch.float32 else 8e-3
        assert ((out.cpu().double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("learned", [True, False])
@pytest.mark.parametrize("d", [32, 48, 64, 128])
def test_sinks_in_the_kernels_shared_with_the_other_decoders(d, learned):
    """Keys and values of one head size in bfloat16: prompts on the tcgen05 kernel (64, 128) and single tokens on the
    TMA-fed (64, 128) or mma.sync decode kernel, with a sink per head (or the sink that scores 0), against the general
    kernel.  Scores are small and the decoded contexts run from one key to hundreds, so the sink is most of a short
    row's denominator: counted twice, or in the wrong units, it shows.  Decode runs with one block a sequence and
    with the context split in four (the sink must be counted once)."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d)
    H, G = 6, 2
    starts, lens = [0, 70, 129, 0, 0, 0, 0], [300, 200, 1, 1, 2, 5, 65]
    n = len(lens)
    ctxs = [s + m for s, m in zip(starts, lens)]
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, torch.bfloat16)
    k_cache, v_cache, table = k_cache.to(dev), v_cache.to(dev), table.to(dev)
    scale = 0.5 / d ** 0.5
    T = sum(lens)
    q = torch.randn((T, H * d), generator=gen).to(torch.bfloat16).to(dev)
    sinks = torch.linspace(-3.0, 4.0, H).to(dev) if learned else None
    state = make_step_state(dev, list(range(n)), starts, lens)
    plain = torch.zeros((T, H * d), dtype=torch.bfloat16, device=dev)
    K.local_attention(q, k_cache, v_cache, state.tok_pos, state.tok_seq, state.seq_slot, table, plain, H, G, d, d, 0, 0, scale,
                      sink=True, sink_values=sinks)
    without = torch.zeros_like(plain)
    K.local_attention(q, k_cache, v_cache, state.tok_pos, state.tok_seq, state.seq_slot, table, without, H, G, d, d, 0, 0, scale)
    torch.cuda.synchronize()
    size = plain.float().abs().max().item()
    assert (plain.float() - without.float()).abs().max().item() > 0.2 * size  # the sink matters in this test
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=dev)
    if K.attention_prefill_takes_chunks(torch.bfloat16, d):
        narrow = [(s, r) for s, m in enumerate(lens) for r in range(0, m, K.PREFILL_TILE)]
        wide = sorted((starts[s] + min(m, r + 128), s, r) for s, m in enumerate(lens) for r in range(0, m, 128))
        fast = torch.zeros_like(plain)
        K.attention_prefill(q, k_cache, v_cache, state.seq_slot, state.seq_ctx, state.seq_qstart, state.seq_qlen,
                            ints([s for s, _ in narrow]), ints([r for _, r in narrow]), table, fast, len(narrow), H, G, d, 0,
                            scale, wide_tiles=(ints([s for _, s, _ in wide]), ints([r for _, _, r in wide])), sink=True,
                            sink_values=sinks)
        torch.cuda.synchronize()
        assert K.take_device_error() == 0
        assert (fast.float() - plain.float()).abs().max().item() <= 0.03 * size
    last = [sum(lens[:i + 1]) - 1 for i in range(n)]  # single tokens: the last token of every sequence
    q1 = q[last].contiguous()
    one = make_step_state(dev, list(range(n)), [c - 1 for c in ctxs], [1] * n)
    for splits in (1, 4):
        out = torch.zeros((n, H * d), dtype=torch.bfloat16, device=dev)
        scratch = torch.zeros((K.attention_decode_scratch_floats(n, H, d, splits),), device=dev) if splits > 1 else None
        counters = torch.zeros((n * G,), dtype=torch.int32, device=dev) if splits > 1 else None
        K.attention_decode(q1, k_cache, v_cache, one.seq_slot, one.seq_ctx, table, scratch, out, n, H, G, d, splits, 0, scale,
                           counters=counters, sink=True, sink_values=sinks)
        torch.cuda.synchronize()
        assert K.take_device_error() == 0
        err = (out.float() - plain[last].float()).abs().max(dim=1).values
        assert err.max().item() <= 0.03 * size, (splits, err.tolist())
