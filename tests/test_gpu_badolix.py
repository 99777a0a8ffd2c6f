"""Badolix through the engine against the plain oracle (`plain_badolix`, float64, whole sequences).

Every test makes its own small configuration and weights (`tiny_badolix`).  float32 runs must agree with the oracle
to 2e-4 of the largest logit (at least 2e-4 absolute): with the test weights a window that is one token off, a kept
token that is dropped, a lost state or convolution input, a wrong expert or group, a cap or a bias left out moves logits
by percents.  bfloat16 runs are compared with the same unrounded oracle, so their bound is that of rounding noise:
largest error at most 10 %, mean error at most 2.5 % of the largest logit (the bound of the other designs' tests).  A
routed layer turns a near-tie between two experts or groups into another expert's output once activations are rounded,
so in bfloat16 the oracle also reports every token's smallest routing margin: as many rows may exceed the bound as
there are tokens whose margin is below 0.02, and none if there are none.  The sharp test is float32."""
import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_badolix as pb
import tiny_badolix as tb
from cpp_minilamma_b200.cache.paged import PAGE
from cpp_minilamma_b200.engine.step import StepEntry

pytestmark = pytest.mark.gpu

_FOLDERS, _ENGINES, _ORACLE, _MARGIN = {}, {}, {}, {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    def get(name, dtype="float32", max_tokens=1024, max_positions=None):
        if name not in _FOLDERS:
            _FOLDERS[name] = tb.make_folder(name, tmp_path_factory.mktemp(name), seed=len(_FOLDERS) + 1)
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
        _ORACLE[key] = pb.forward(cfg, W, toks, margins=margins)
        _MARGIN[id(_ORACLE[key])] = np.min(margins, axis=0) if margins else None
    return _ORACLE[key]


def close(got, ref, dtype, what):
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
    allowed = int((margin < 0.02).sum()) if margin is not None and len(margin) == len(rows) else 0
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


LENGTH = {"window": 150, "latent": 150, "ssm": 150, "feeds": 75, "shared": 200, "shared_windows": 330, "mixed": 200,
          "ones": 140, "tensor": 300, "odd": 90}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_whole_prompt(models, name, dtype):
    """Every position of one prompt, the first tokens included (kept tokens that are the whole context, a state and a
    convolution that start at zero); prompts reach over page borders and several windows."""
    llm, cfg, W = models(name, dtype)
    toks = tb.tokens(cfg, LENGTH[name], 11)
    close(run_alone(llm, toks, [len(toks)]), oracle(name, cfg, W, toks), dtype, f"{name} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_prompt_then_token_by_token(models, name, dtype):
    """A short prompt, then a long run of single tokens through the cache and the state: the window passes over decoded
    tokens and page borders, kept tokens stay, the recurrent state and the convolution's inputs are carried step by step."""
    llm, cfg, W = models(name, dtype)
    toks = tb.tokens(cfg, LENGTH[name], 12)
    close(run_alone(llm, toks, [7]), oracle(name, cfg, W, toks), dtype, f"{name} decode")


def test_token_by_token_from_the_first_token(models):
    """No prompt at all: the very first step brings one token (an empty state, fewer inputs than the convolution has taps)."""
    llm, cfg, W = models("mixed", "float32")
    toks = tb.tokens(cfg, 70, 14)
    close(run_alone(llm, toks, []), oracle("mixed", cfg, W, toks), "float32", "mixed from the first token")


@pytest.mark.parametrize("name,cuts", [
    ("mixed", [2, 3, 1, 7, 2, 49, 2, 2, 64]),      # portions down to two tokens, cuts inside and at the end of a page
    ("ones", [1, 1, 62, 2, 66]),                   # single first tokens; a cut at the page's edge and after it
    ("window", [8, 8, 7, 2, 39, 64]),
    ("ssm", [63, 1, 2, 64, 17]),                   # the state and the convolution's inputs handed from portion to portion
    ("ssm", [2, 1, 1, 2, 3]),                      # portions shorter than the convolution
    ("odd", [5, 2, 2, 60]),
    ("shared", [3, 2, 61, 2, 90]),
    ("shared_windows", [70, 2, 100, 2, 66]),       # portions that start just behind a window's and the kept tokens' edge
    ("latent", [2, 2, 2, 58, 2, 30]),
])
def test_portions(models, name, cuts):
    llm, cfg, W = models(name, "float32")
    toks = tb.tokens(cfg, LENGTH[name], 13)
    close(run_alone(llm, toks, cuts), oracle(name, cfg, W, toks), "float32", f"{name} portions {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones", "tensor", "shared_windows"])
def test_unequal_batch_then_decoding_together(models, name, dtype):
    """Requests of 1, 37 and 90 tokens start in one step, go on by one token each, and the short ones end early; every
    logit equals that of the request alone (the routed layers sort the batch's tokens by expert; windows, kept tokens,
    states and convolution inputs belong to each request)."""
    llm, cfg, W = models(name, dtype)
    eng = llm.engine
    seqs = [tb.tokens(cfg, n, 20 + i) for i, n in enumerate((9, 50, 134))]
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
        close(np.concatenate(got[i]), oracle(name, cfg, W, q), dtype, f"{name} request {i} in a batch")
    eng.cache.check()


@pytest.mark.parametrize("name", ["mixed", "shared_windows"])
def test_slots_pages_and_states_used_again(models, name):
    """A cache of a few pages: a sequence of three and a half pages, then - in the same slot, pages and state rows,
    handed out in another order - a second one, while a third short request comes and goes beside them.  A state, a
    convolution input or a kept page left behind by the first sequence would show in the second one's first rows.
    With windows on every layer of a group the sequences are longer than the pool: pages come back from behind the window."""
    windowed = name == "shared_windows"
    llm, cfg, W = models(name, "float32", max_tokens=(8 if windowed else 5) * PAGE, max_positions=(12 if windowed else 4) * PAGE)
    eng = llm.engine
    for seed in (31, 32):
        toks = tb.tokens(cfg, (11 if windowed else 3) * PAGE + 30, seed)
        short = tb.tokens(cfg, 20, seed + 10)
        slot = eng.acquire(1)[0]
        rows = []
        for at in range(0, len(toks), 50):
            part = toks[at:at + 50]
            rows.append(eng.step([StepEntry(slot, part, list(range(len(part))))]).cpu().numpy())
            if at == 50:  # a neighbour that takes a page and gives it back
                other = eng.acquire(1)[0]
                got = eng.step([StepEntry(other, short, list(range(20)))]).cpu().numpy()
                eng.release(other)
                close(got, oracle(name, cfg, W, short), "float32", "the neighbour")
        eng.release(slot)
        eng.cache.check()
        close(np.concatenate(rows), oracle(name, cfg, W, toks), "float32", f"long sequence, seed {seed}")
    assert all(g.pool.n_free == g.pool.n_pages for g in eng.cache.groups)


@pytest.mark.parametrize("seed", list(range(200, 216)))
def test_configurations_drawn_from_fixed_seeds(seed, tmp_path):
    """Sixteen configurations that nobody chose by hand, in float32 (the sharp comparison): a whole prompt, and the same
    prompt cut after 250 tokens and decoded beside a second, shorter request that ends earlier."""
    cfg = tb.random_config(seed)
    W = tb.make_weights(cfg, seed)
    folder = tb.write_folder(cfg, W, tmp_path / "m")
    W = {k: v.astype(np.float64) for k, v in W.items()}
    llm = ml.load(folder, dtype="float32", max_tokens=2048, max_positions=512)
    eng = llm.engine
    a, b = tb.tokens(cfg, 330, seed + 1), tb.tokens(cfg, 90, seed + 2)
    ref_a, ref_b = pb.forward(cfg, W, a), pb.forward(cfg, W, b)
    close(run_alone(llm, a, [len(a)]), ref_a, "float32", f"seed {seed} whole")
    sa, sb = eng.acquire(2)
    out = eng.step([StepEntry(sa, a[:250], list(range(250))), StepEntry(sb, b[:40], list(range(40)))]).cpu().numpy()
    rows_a, rows_b = [out[:250]], [out[250:]]
    for p in range(250, 330):
        q = p - 210
        entries = [StepEntry(sa, [a[p]], [0])] + ([StepEntry(sb, [b[q]], [0])] if q < 90 else [])
        out = eng.step(entries).cpu().numpy()
        rows_a.append(out[:1])
        if q < 90:
            rows_b.append(out[1:2])
        if q == 89:
            eng.release(sb)
    eng.release(sa)
    close(np.concatenate(rows_a), ref_a, "float32", f"seed {seed} decoded in a batch")
    close(np.concatenate(rows_b), ref_b, "float32", f"seed {seed} the shorter request")
    eng.cache.check()


def test_an_engine_cuts_a_long_step_itself(models):
    models("mixed")
    folder, cfg, W = _FOLDERS["mixed"]
    llm = ml.load(folder, dtype="float32", max_tokens=512, max_step_tokens=64)
    toks = tb.tokens(cfg, 150, 41)
    close(run_alone(llm, toks, [150]), oracle("mixed", cfg, W, toks), "float32", "engine-cut step")


def greedy_oracle(cfg, W, prompt, n):
    toks, out, sure = list(prompt), [], []
    for _ in range(n):
        logits = pb.forward(cfg, W, toks)[-1]
        best = int(np.argmax(logits))
        sure.append(logits[best] - np.partition(logits, -2)[-2] > 1e-3)
        out.append(best)
        toks.append(best)
    return out, sure


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`generate` (the scheduler, captured decode steps, device sampling, the step enqueued ahead) picks the oracle's tokens."""
    llm, cfg, W = models(name, "float32")
    prompts = [tb.tokens(cfg, n, 50 + i) for i, n in enumerate((3, 21, 66))]
    outs = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    for prompt, got in zip(prompts, outs):
        want, sure = greedy_oracle(cfg, W, prompt, 14)
        upto = sure.index(False) if False in sure else len(sure)  # after a near-tie either token is right
        assert got[:upto] == want[:upto], (got, want)
    again = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    assert again == outs  # slots, pages and states of finished requests serve the next ones
    llm.engine.cache.check()


def test_bfloat16_generation_replays_captured_steps(models):
    """Decode steps of the bfloat16 engine run from CUDA graphs (window and latent attention, the state-space mixer,
    routing, sorting and the expert products included) and give the tokens of the same engine stepping eagerly."""
    llm, cfg, W = models("tensor", "bfloat16")
    assert llm.model.capturable()
    prompts = [tb.tokens(cfg, n, 80 + i) for i, n in enumerate((5, 40))]
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
    prompt = tb.tokens(cfg, 5, 60)
    assert main(["generate", folder, "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                 "--ignore-eos"]) == 0
    line = capsys.readouterr().out.splitlines()[0]
    want, sure = greedy_oracle(cfg, W, prompt, 6)
    upto = sure.index(False) if False in sure else len(sure)
    assert [int(t) for t in line.split()][:upto] == want[:upto]


def test_trace_replay_writes_the_wanted_logits(models, tmp_path):
    """The trace runner on a Badolix folder: two requests start together, decode, one ends early."""
    import json
    import os
    import subprocess
    import sys
    _, cfg, W = models("mixed", "float32")
    folder = _FOLDERS["mixed"][0]
    a, b = tb.tokens(cfg, 30, 70), tb.tokens(cfg, 70, 71)
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
def _paged(gen, ctxs, G, d, dv, dtype):
    """Key and value caches with every sequence's pages in shuffled order."""
    n_pages = sum(-(-c // PAGE) for c in ctxs) + 3
    k_cache = (torch.randn((n_pages, G, PAGE, d), generator=gen) * 0.5).to(dtype)
    v_cache = torch.randn((n_pages, G, PAGE, dv), generator=gen).to(dtype)
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


def _window_attention(q, keys, values, pos0, scale, cap, window, keep, group):
    """q [n, H, d] at positions pos0 ..; keys [ctx, G, d], values [ctx, G, dv]; the softmax written out."""
    n, H, _ = q.shape
    out = torch.zeros((n, H, values.shape[-1]), dtype=torch.float64)
    for i in range(n):
        p = pos0 + i
        seen = [j for j in range(p + 1) if window <= 0 or p - j < window or j < keep]
        for h in range(H):
            s = scale * keys[seen, h // group] @ q[i, h]
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            out[i, h] = torch.softmax(s, dim=0) @ values[seen, h // group]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window,keep,cap", [
    (4, 2, 16, 16, 40, 5, 6.0), (3, 1, 48, 24, 64, 64, 0.0), (2, 2, 72, 72, 100, 0, 12.0), (5, 1, 6, 10, 7, 3, 4.0),
    (8, 2, 64, 64, 130, 70, 20.0), (2, 1, 128, 128, 65, 1, 0.0), (2, 2, 32, 32, 0, 0, 5.0)])
def test_window_attention_kernels_at_the_edges(dtype, H, G, d, dv, window, keep, cap):
    """The general kernel (both dtypes), the tensor-core prompt kernel and the single-token kernel with heads as rows
    (bfloat16, with and without context splits) against the softmax written out: three sequences that start at
    positions 0, 70 and 300, one of them a single token.  In every sequence the keys just inside and just outside the
    last query's window and the last kept token and the first one that is not kept are scaled so that their scores
    stand out: one of them wrongly seen or missed moves the row."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d * 1000 + H)
    starts, lens = [0, 70, 300], [150, 61, 1]
    ctxs = [s + n for s, n in zip(starts, lens)]
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, dv, dtype)
    T = sum(lens)
    q = (torch.randn((T, H, d), generator=gen) * 0.7).to(dtype)
    for s, ctx in enumerate(ctxs):
        marks = [p for p in (ctx - window, ctx - window - 1, keep - 1, keep, ctx // 2) if window > 0 and 0 <= p < ctx] or [ctx // 3]
        for n, p in enumerate(marks):
            k_cache[int(table[s, p // PAGE]), :, p % PAGE] *= 3.0 + n
    scale = 1.3 / d ** 0.5
    want = torch.zeros((T, H, dv), dtype=torch.float64)
    at = 0
    for s, (start, n) in enumerate(zip(starts, lens)):
        want[at:at + n] = _window_attention(q[at:at + n].double(), _dense(k_cache, table, s, ctxs[s]),
                                            _dense(v_cache, table, s, ctxs[s]), start, scale, cap, window, keep, H // G)
        at += n
    kd, vd, td, qd = k_cache.to(dev), v_cache.to(dev), table.to(dev), q.view(T, H * d).to(dev)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    ref_scale = float(want.abs().max())

    def check(out, rows, what):
        err = (out.double().cpu().view(-1, H, dv) - want[rows]).abs().max()
        assert float(err) <= tol * max(1.0, ref_scale), f"{what}: {float(err):.3e}"

    class Part:  # the tile list of the tensor-core prompt kernel, as the attention part prepares it
        def step_metadata_key(self):
            return "tiles"

        def prepare_step(self, shape):
            lists = {"tile_seq": [], "tile_row0": []}
            for i in range(shape.n_seqs):
                for row0 in range(0, shape.lens[i], K.PREFILL_TILE):
                    lists["tile_seq"].append(i)
                    lists["tile_row0"].append(row0)
            return lists

    step = make_step_state(dev, [0, 1, 2], starts, lens, parts=[Part()])
    out = torch.empty((T, H * dv), dtype=dtype, device=dev)
    K.local_attention(qd, kd, vd, step.tok_pos, step.tok_seq, step.seq_slot, td, out, H, G, d, dv, 0, window, scale,
                      keep_first=keep, softcap=cap)
    check(out, slice(0, T), "general kernel")
    if dtype == torch.bfloat16 and K.local_attention_mma_supported(dtype, d, dv):
        out.zero_()
        tiles = step.meta["tiles"]
        K.local_attention_tiles(qd, kd, vd, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                tiles["tile_seq"], tiles["tile_row0"], td, out, H, G, d, dv, 0, window, scale,
                                keep_first=keep, softcap=cap)
        check(out, slice(0, T), "tensor-core prompt kernel")
        # single tokens: the last token of every sequence as a step of its own
        last = [sum(lens[:i + 1]) - 1 for i in range(3)]
        one = make_step_state(dev, [0, 1, 2], [c - 1 for c in ctxs], [1, 1, 1])
        q1 = qd[last].contiguous()
        for splits in (1, 3):
            o1 = torch.zeros((3, H * dv), dtype=dtype, device=dev)
            scratch = torch.empty(K.local_attention_heads_scratch(3, H, dv, splits), dtype=torch.float32, device=dev)
            K.local_attention_heads(q1, kd, vd, one.seq_slot, one.seq_ctx, one.seq_qstart, one.seq_qlen, td, o1, 3, H, G,
                                    d, dv, 0, window, scale, n_splits=splits, scratch=scratch, keep_first=keep, softcap=cap)
            check(o1, last, f"single-token kernel, {splits} splits")
        if d == dv and K.attention_prefill_takes_chunks(dtype, d):
            # the tcgen05 prompt kernel (tiles of 128 rows) and the TMA-fed single-token kernel, whole and in splits
            wide = [(i, row0) for i in range(3) for row0 in range(0, lens[i], 2 * K.PREFILL_TILE)]
            wide_seq = torch.tensor([i for i, _ in wide], dtype=torch.int32, device=dev)
            wide_row0 = torch.tensor([r for _, r in wide], dtype=torch.int32, device=dev)
            out.zero_()
            K.attention_prefill(qd, kd, vd, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen, tiles["tile_seq"],
                                tiles["tile_row0"], td, out, tiles["tile_seq"].shape[0], H, G, d, window, scale,
                                wide_tiles=(wide_seq, wide_row0), keep_first=keep, softcap=cap)
            check(out, slice(0, T), "tcgen05 prompt kernel")
        if d == dv and K.attention_decode_takes_window_extras(dtype, d):
            for splits in (1, 3):
                o1 = torch.zeros((3, H * dv), dtype=dtype, device=dev)
                scratch = torch.empty(K.attention_decode_scratch_floats(3, H, d, splits), dtype=torch.float32, device=dev)
                counters = torch.zeros((3 * G * -(-(H // G) // 16),), dtype=torch.int32, device=dev)
                K.attention_decode(q1, kd, vd, one.seq_slot, one.seq_ctx, td, scratch if splits > 1 else None, o1, 3, H, G, d,
                                   splits, window, scale, counters=counters if splits > 1 else None, keep_first=keep, softcap=cap)
                check(o1, last, f"TMA-fed single-token kernel, {splits} splits")


@pytest.mark.parametrize("H,G,d,dv,seqs", [(4, 2, 12, 8, 2), (2, 1, 64, 32, 3), (8, 8, 128, 64, 2), (3, 3, 10, 6, 1),
                                           (16, 2, 32, 64, 40), (4, 1, 200, 16, 2)])
def test_state_scan_with_a_decay_per_token_and_head(H, G, d, dv, seqs):
    """S <- a_t S + k_t u_t^T, o_t = S^T q_t with k and q shared by the heads of a group, at every layout of the scan
    (few columns, a prompt, a batch of single tokens), from a state that is not zero, against the recurrence in float64."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d + dv)
    for lens in ([37] + [1] * (seqs - 1), [1] * seqs, [70] * min(seqs, 2)):
        n_seqs, T = len(lens), sum(lens)
        q, k = torch.randn((T, G * d), generator=gen), torch.randn((T, G * d), generator=gen) * 0.5
        u = torch.randn((T, H * dv), generator=gen)
        a = torch.rand((T, H), generator=gen)
        a[::3] = 1.0            # no forgetting
        a[1::7] = 0.0           # everything forgotten
        state = torch.randn((n_seqs + 1, H, d, dv), generator=gen)
        step = make_step_state(dev, list(range(n_seqs)), [5] * n_seqs, lens)
        out = torch.empty((T, H * dv), dtype=torch.float32, device=dev)
        sd = state.to(dev)
        K.state_scan(q.to(dev), k.to(dev), u.to(dev), None, None, None, sd, out, step.seq_slot, step.seq_qstart,
                     step.seq_qlen, n_seqs, H, G, d, dv, token_decay=a.to(dev))
        want, S = torch.zeros((T, H, dv), dtype=torch.float64), state.double().clone()
        at = 0
        for s, n in enumerate(lens):
            for t in range(at, at + n):
                for h in range(H):
                    g = h // (H // G)
                    S[s, h] = a[t, h].double() * S[s, h] + torch.outer(k[t, g * d:(g + 1) * d].double(), u[t, h * dv:(h + 1) * dv].double())
                    want[t, h] = S[s, h].T @ q[t, g * d:(g + 1) * d].double()
            at += n
        scale = max(1.0, float(want.abs().max()))
        assert float((out.cpu().double().view(T, H, dv) - want).abs().max()) <= 2e-5 * scale, lens
        assert float((sd.cpu().double()[:n_seqs] - S[:n_seqs]).abs().max()) <= 2e-5 * max(1.0, float(S.abs().max())), lens


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,N,P,taps", [(4, 2, 12, 8, 4), (1, 1, 8, 8, 1), (3, 1, 10, 6, 3), (8, 4, 64, 32, 2)])
def test_state_space_inputs_and_the_carried_convolution(dtype, H, G, N, P, taps):
    """`ssd_prepare` + `conv_state_update` over a sequence cut into portions (some shorter than the convolution) beside
    another sequence: convolution with bias and silu, softplus step sizes, decays and u = dt x against float64."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(N * 7 + taps)
    inner, gn = H * P, G * N
    C, ld = inner + 2 * gn, 2 * inner + 2 * gn + H + 3      # a few spare columns behind dt, as a padded product leaves them
    total = [23, 9]
    rows = [torch.randn((n, ld), generator=gen).to(dtype) for n in total]
    conv_w, conv_b = torch.randn((C, taps), generator=gen) * 0.6, torch.randn((C,), generator=gen) * 0.3
    a_log, dt_bias = torch.randn((H,), generator=gen) - 0.5, torch.randn((H,), generator=gen)
    state = torch.zeros((3, taps - 1, C), dtype=torch.float32, device=dev)
    got = [[], []]
    done = [0, 0]
    for cuts in ([1, 2], [2, 1], [1, 1], [taps, 0], [19 - taps, 5]):
        seqs = [i for i in range(2) if cuts[i] > 0]
        lens = [cuts[i] for i in seqs]
        proj = torch.cat([rows[i][done[i]:done[i] + cuts[i]] for i in seqs]).to(dev)
        step = make_step_state(dev, seqs, [done[i] for i in seqs], lens)
        T = sum(lens)
        q, k = (torch.empty((T, gn), dtype=torch.float32, device=dev) for _ in range(2))
        u, xs = (torch.empty((T, inner), dtype=torch.float32, device=dev) for _ in range(2))
        decay = torch.empty((T, H), dtype=torch.float32, device=dev)
        K.ssd_prepare(proj, conv_w.to(dev), conv_b.to(dev), state, a_log.to(dev), dt_bias.to(dev), step.tok_seq,
                      step.seq_slot, step.seq_qstart, q, k, u, xs, decay, H, G, N, P, taps)
        K.conv_state_update(proj, state, step.seq_slot, step.seq_qstart, step.seq_qlen, len(seqs), C, taps, first_column=inner)
        at = 0
        for i, n in zip(seqs, lens):
            got[i].append(torch.cat([q[at:at + n], k[at:at + n], u[at:at + n], xs[at:at + n], decay[at:at + n]], dim=1).cpu())
            at += n
            done[i] += n
    for i in range(2):
        raw = rows[i][:done[i]].double()
        xbc = raw[:, inner:inner + C]
        padded = torch.cat([torch.zeros((taps - 1, C), dtype=torch.float64), xbc])
        conv = conv_b.double() + sum(padded[j:j + done[i]] * conv_w[:, j].double() for j in range(taps))
        conv = conv * torch.sigmoid(conv)
        dt = torch.nn.functional.softplus(raw[:, inner + C:inner + C + H] + dt_bias.double())
        want = torch.cat([conv[:, inner + gn:], conv[:, inner:inner + gn],
                          conv[:, :inner] * dt.repeat_interleave(P, dim=1), conv[:, :inner],
                          torch.exp(-torch.exp(a_log.double()) * dt)], dim=1)
        err = (torch.cat(got[i]).double() - want).abs().max()
        assert float(err) <= 1e-5 * max(1.0, float(want.abs().max())), (i, float(err))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,parts", [(4, 8, 2), (1, 8, 8), (3, 6, 3), (6, 4, 1), (16, 64, 4)])
def test_gated_norm_in_equal_parts(dtype, H, P, parts):
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(H * P)
    T, width = 7, H * P
    o, xs = torch.randn((T, width), generator=gen), torch.randn((T, width), generator=gen)
    skip, weight = torch.randn((H,), generator=gen), 1 + 0.3 * torch.randn((width,), generator=gen)
    gate = torch.randn((T, width + 5), generator=gen).to(dtype)
    out = torch.empty((T, width), dtype=dtype, device=dev)
    K.gated_group_norm(o.to(dev), xs.to(dev), skip.to(dev), gate.to(dev), weight.to(dev), out, P, parts, 1e-5)
    z = gate[:, :width].double()
    y = (o.double() + skip.double().repeat_interleave(P) * xs.double()) * z * torch.sigmoid(z)
    y = y.view(T, parts, -1)
    want = (y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + 1e-5)).view(T, width) * weight.double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert float((out.cpu().double() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("E,top,count,keep", [(8, 3, 4, 2), (12, 4, 4, 3), (1, 1, 1, 1), (6, 6, 1, 1), (5, 1, 5, 2),
                                              (64, 8, 8, 4), (9, 2, 3, 3)])
def test_routing_kernel_chooses_inside_the_best_groups(E, top, count, keep):
    """The routing kernel (logits in the kernel for few tokens, from a library product for many) against the oracle's
    `route`, token by token: the same experts in the same order, weights that are the chosen scores over their sum."""
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(E * 10 + top)
    D = 24
    w = torch.randn((E, D), generator=gen) * 0.6
    for T in (5, 300):
        h = torch.randn((T, D), generator=gen)
        chosen = torch.empty((T, top), dtype=torch.int32, device=dev)
        weight = torch.empty((T, top), dtype=torch.float32, device=dev)
        logits = (h @ w.T).to(dev) if T > 256 else None
        K.moe_route(h.to(dev), w.to(dev), None, chosen, weight, top, logits=logits, all_scores=True, groups=(count, keep))
        scores = 1.0 / (1.0 + np.exp(-(h.double() @ w.double().T).numpy()))
        for t in range(T):
            want, want_w, margin = pb.route(scores[t], top, count, keep)
            if margin < 1e-5:
                continue  # a tie within float32 rounding
            assert chosen[t].cpu().tolist() == list(want), (t, chosen[t].cpu().tolist(), list(want))
            assert np.abs(weight[t].cpu().numpy() - want_w).max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [16, 20, 7])
def test_biased_swiglu_and_scaled_rows(dtype, inter):
    """The activation kernel with the gate's and up's biases (both layouts of the fused rows), the embedding's and the
    logits' factors."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.parts.mlp import fuse_gate_up
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(inter)
    T = 5
    g, u = torch.randn((T, inter), generator=gen).to(dtype), torch.randn((T, inter), generator=gen).to(dtype)
    bg, bu = torch.randn((inter,), generator=gen), torch.randn((inter,), generator=gen)
    fused, block = fuse_gate_up(g.T.contiguous(), u.T.contiguous())          # rows of a fused matrix = columns of gate_up
    bias, _ = fuse_gate_up(bg.view(-1, 1), bu.view(-1, 1))
    out = torch.empty((T, inter), dtype=dtype, device=dev)
    K.swiglu(fused.T.contiguous().to(dev), out, block, bias=bias.view(-1).contiguous().to(dev))
    z = g.double() + bg.double()
    want = z * torch.sigmoid(z) * (u.double() + bu.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((out.cpu().double() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    table = torch.randn((9, inter), generator=gen).to(dtype)
    x = torch.empty((3, inter), dtype=torch.float32, device=dev)
    K.embedding(torch.tensor([4, 0, 8], dtype=torch.int32, device=dev), table.to(dev), x, 2.5)
    assert torch.equal(x.cpu(), table[[4, 0, 8]].float() * 2.5)
    K.scale_(x, 0.5)
    assert torch.equal(x.cpu(), table[[4, 0, 8]].float() * 2.5 * 0.5)
