"""Malulorn through the engine against the plain oracle (`plain_malulorn`, float64, whole sequences).

Every test makes its own small configuration and weights (`tiny_malulorn`).  float32 runs must agree with the
oracle to 2e-4 of the largest logit (at least 2e-4 absolute): with the test weights a sink left out, a query
temperature one position off, one key wrongly seen or missed, a wrong expert or a lost re-entry moves logits by
percents.  bfloat16 runs are compared with the same unrounded oracle, so their bound is that of rounding noise:
largest error at most 10 %, mean error at most 2.5 % of the largest logit (the bound of the other design's tests).
A routed layer turns a near-tie between two experts into another expert's output once activations are rounded, so
in bfloat16 the oracle also reports every token's smallest margin between the last chosen and the first unchosen
router logit: as many rows may exceed the bound as there are tokens whose margin is below 0.1, and none if there
are none.  The sharp test is float32, where near-ties do not matter."""
import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_malulorn as pm
import tiny_malulorn as tm
from cpp_minilamma_b200.cache.paged import PAGE
from cpp_minilamma_b200.engine.step import StepEntry

pytestmark = pytest.mark.gpu

_FOLDERS, _ENGINES, _ORACLE = {}, {}, {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    def get(name, dtype="float32", max_tokens=1024, max_positions=None):
        if name not in _FOLDERS:
            _FOLDERS[name] = tm.make_folder(name, tmp_path_factory.mktemp(name), seed=len(_FOLDERS) + 1)
        folder, cfg, W = _FOLDERS[name]
        key = (name, dtype, max_tokens, max_positions)
        if key not in _ENGINES:
            _ENGINES[key] = ml.load(folder, dtype=dtype, max_tokens=max_tokens, max_positions=max_positions)
        return _ENGINES[key], cfg, W
    yield get
    _ENGINES.clear()


_MARGIN = {}


def oracle(name, cfg, W, toks):
    key = (name, tuple(toks))
    if key not in _ORACLE:
        margins = []
        _ORACLE[key] = pm.forward(cfg, W, toks, margins=margins)
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
    allowed = int((margin < 0.1).sum()) if routed and margin is not None and len(margin) == len(rows) else 0
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


LENGTH = {"sink_only": 150, "latent_only": 150, "routed": 75, "reentry": 75, "mixed": 200, "ones": 140, "wide": 135,
          "tensor": 300, "odd": 90}
ROUTED = {"routed", "mixed", "ones", "wide", "tensor", "odd"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_whole_prompt(models, name, dtype):
    """Every position of one prompt, the first tokens included (where the sink's share is largest); prompts
    reach over page borders and over several steps of the query temperature."""
    llm, cfg, W = models(name, dtype)
    toks = tm.tokens(cfg, LENGTH[name], 11)
    close(run_alone(llm, toks, [len(toks)]), oracle(name, cfg, W, toks), dtype, f"{name} whole", name in ROUTED)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_prompt_then_token_by_token(models, name, dtype):
    """A short prompt, then a long run of single tokens through the cache: over page borders, over every step of
    the temperature (each 1, 5, 7, 8, 16 or 64 positions), every pass of a loop reading its own cache."""
    llm, cfg, W = models(name, dtype)
    toks = tm.tokens(cfg, LENGTH[name], 12)
    close(run_alone(llm, toks, [7]), oracle(name, cfg, W, toks), dtype, f"{name} decode", name in ROUTED)


@pytest.mark.parametrize("name,cuts", [
    ("mixed", [2, 3, 1, 7, 2, 49, 2, 2, 64]),      # portions down to two tokens, cuts inside and at the end of a page
    ("ones", [1, 1, 62, 2, 66]),                   # single first tokens; a cut at the page's edge and after it
    ("sink_only", [8, 8, 7, 2, 39, 64]),           # portions that end where the temperature steps
    ("latent_only", [63, 1, 2, 64]),
    ("odd", [5, 2, 2, 60]),
    ("reentry", [3, 2, 61, 2]),
])
def test_portions(models, name, cuts):
    llm, cfg, W = models(name, "float32")
    toks = tm.tokens(cfg, LENGTH[name], 13)
    close(run_alone(llm, toks, cuts), oracle(name, cfg, W, toks), "float32", f"{name} portions {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones", "wide"])
def test_unequal_batch_then_decoding_together(models, name, dtype):
    """Requests of 1, 37 and 90 tokens start in one step, go on by one token each, and the short ones end early;
    every logit equals that of the request alone (the routed layers sort the batch's tokens by expert)."""
    llm, cfg, W = models(name, dtype)
    eng = llm.engine
    seqs = [tm.tokens(cfg, n, 20 + i) for i, n in enumerate((9, 50, 104))]
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


def test_slots_and_pages_used_again(models):
    """A cache of four pages: a sequence of three and a half pages, then - in the same slot and pages, handed out
    in another order - a second one, while a third short request comes and goes beside them."""
    llm, cfg, W = models("mixed", "float32", max_tokens=5 * PAGE, max_positions=4 * PAGE)
    eng = llm.engine
    for seed in (31, 32):
        toks = tm.tokens(cfg, 3 * PAGE + 30, seed)
        short = tm.tokens(cfg, 20, seed + 10)
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
    toks = tm.tokens(cfg, 150, 41)
    close(run_alone(llm, toks, [150]), oracle("mixed", cfg, W, toks), "float32", "engine-cut step")


def greedy_oracle(cfg, W, prompt, n):
    toks, out, sure = list(prompt), [], []
    for _ in range(n):
        logits = pm.forward(cfg, W, toks)[-1]
        best = int(np.argmax(logits))
        sure.append(logits[best] - np.partition(logits, -2)[-2] > 1e-3)
        out.append(best)
        toks.append(best)
    return out, sure


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`generate` (the scheduler, captured decode steps, device sampling) picks the oracle's tokens."""
    llm, cfg, W = models(name, "float32")
    prompts = [tm.tokens(cfg, n, 50 + i) for i, n in enumerate((3, 21, 66))]
    outs = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    for prompt, got in zip(prompts, outs):
        want, sure = greedy_oracle(cfg, W, prompt, 14)
        upto = sure.index(False) if False in sure else len(sure)  # after a near-tie either token is right
        assert got[:upto] == want[:upto], (got, want)
    again = llm.generate(prompts, max_new_tokens=14, ignore_eos=True)
    assert again == outs  # slots and pages of finished requests serve the next ones
    llm.engine.cache.check()


def test_bfloat16_generation_replays_captured_steps(models):
    """Decode steps of the bfloat16 engine run from CUDA graphs (routing, sorting and the expert products included)
    and give the tokens of the same engine stepping eagerly."""
    llm, cfg, W = models("mixed", "bfloat16")
    assert llm.model.capturable()
    prompts = [tm.tokens(cfg, n, 80 + i) for i, n in enumerate((5, 40))]
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
    prompt = tm.tokens(cfg, 5, 60)
    assert main(["generate", folder, "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                 "--ignore-eos"]) == 0
    line = capsys.readouterr().out.splitlines()[0]
    want, sure = greedy_oracle(cfg, W, prompt, 6)
    upto = sure.index(False) if False in sure else len(sure)
    assert [int(t) for t in line.split()][:upto] == want[:upto]


def test_trace_replay_writes_the_wanted_logits(models, tmp_path):
    """The trace runner on a Malulorn folder: two requests start together, decode, one ends early."""
    import json
    import os
    import subprocess
    import sys
    _, cfg, W = models("mixed", "float32")
    folder = _FOLDERS["mixed"][0]
    a, b = tm.tokens(cfg, 30, 70), tm.tokens(cfg, 70, 71)
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
def _paged(gen, ctxs, G, d, dv, dtype, dev, v_in_k=False):
    """Caches with every sequence's pages in shuffled order, and the dense keys / values they hold."""
    n_pages = sum(-(-c // PAGE) for c in ctxs) + 3
    k_cache = (torch.randn((n_pages, G, PAGE, d), generator=gen) * 0.5).to(dtype)
    v_cache = k_cache if v_in_k else torch.randn((n_pages, G, PAGE, dv), generator=gen).to(dtype)
    order = torch.randperm(n_pages, generator=gen).tolist()
    table = torch.full((len(ctxs), max(-(-c // PAGE) for c in ctxs)), -1, dtype=torch.int32)
    at = 0
    for s, c in enumerate(ctxs):
        blocks = -(-c // PAGE)
        table[s, :blocks] = torch.tensor(order[at:at + blocks], dtype=torch.int32)
        at += blocks
    return k_cache, v_cache, table


def _dense(cache, table, s, ctx, width):
    rows = [cache[int(table[s, p // PAGE]), :, p % PAGE, :width] for p in range(ctx)]
    return torch.stack(rows).double()  # [ctx, G, width]


def _attention_oracle(q, keys, values, pos0, scale, sink, group):
    """q [n, H, d] at positions pos0 .. ; keys [ctx, G, d]; values [ctx, G, dv] -> [n, H, dv] in float64."""
    n, H, _ = q.shape
    out = torch.zeros((n, H, values.shape[-1]), dtype=torch.float64)
    for i in range(n):
        for h in range(H):
            s = scale * keys[:pos0 + i + 1, h // group] @ q[i, h]
            top = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - top)
            out[i, h] = (e / (e.sum() + (np.exp(-top) if sink else 0.0))) @ values[:pos0 + i + 1, h // group]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,dv,sink,v_in_k,G", [(16, 24, True, False, 2), (48, 32, False, True, 1), (72, 136, True, False, 1),
                                                (272, 264, False, True, 1), (6, 10, True, False, 1), (64, 64, True, False, 2)])
def test_attention_kernels_with_a_far_key_that_stands_out(dtype, d, dv, sink, v_in_k, G):
    """The general kernel (both dtypes) and the tensor-core prompt kernel (bfloat16) against the softmax written
    out: three sequences that start at positions 0, 70 and 300, one of them a single token.  In every sequence
    one early key (position 1, 3 or 5: hundreds back, in a page of its own) is scaled so that its score stands out,
    and every other score is small, so that the sink's share of the denominator is large."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d * 1000 + dv)
    H = 4
    starts, lens = [0, 70, 300], [150, 61, 1]
    ctxs = [s + n for s, n in zip(starts, lens)]
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, dv, dtype, dev, v_in_k)
    T = sum(lens)
    q = torch.randn((T, H * d), generator=gen).to(dtype)
    for s in range(3):  # the far key points along the queries' mean direction
        far = 1 + 2 * s
        page = int(table[s, 0])
        rows = slice(sum(lens[:s]), sum(lens[:s + 1]))
        mean_q = q[rows].float().view(-1, H, d).mean(dim=(0, 1))
        k_cache[page, :, far, :] = (k_cache[page, :, far, :].float() + 6.0 * mean_q / mean_q.norm()).to(dtype)
    scale = 1.0 / d ** 0.5
    want = []
    for s in range(3):
        rows = slice(sum(lens[:s]), sum(lens[:s + 1]))
        keys = _dense(k_cache, table, s, ctxs[s], d)
        values = _dense(v_cache, table, s, ctxs[s], dv)
        want.append(_attention_oracle(q[rows].double().view(-1, H, d), keys, values, starts[s], scale, sink, H // G))
    want = torch.cat(want).view(T, H * dv)
    state = make_step_state(dev, [0, 1, 2], starts, lens)
    kc, table_dev, qd = k_cache.to(dev), table.to(dev), q.to(dev)
    vc = kc if v_in_k else v_cache.to(dev)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    plain = torch.zeros((T, H * dv), dtype=dtype, device=dev)
    K.local_attention(qd, kc, vc, state.tok_pos, state.tok_seq, state.seq_slot, table_dev, plain, H, G, d, dv, 0, 0, scale,
                      sink=sink, v_in_k=v_in_k)
    torch.cuda.synchronize()
    err = (plain.cpu().double() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), ("general kernel", err)
    if dtype == torch.bfloat16 and K.local_attention_mma_supported(dtype, d, dv):
        tile_seq = [s for s, n in enumerate(lens) for _ in range(0, n, K.PREFILL_TILE)]
        tile_row0 = [r for n in lens for r in range(0, n, K.PREFILL_TILE)]
        ints = lambda values: torch.tensor(values, dtype=torch.int32, device=dev)
        fast = torch.zeros_like(plain)
        K.local_attention_tiles(qd, kc, vc, state.seq_slot, state.seq_ctx, state.seq_qstart, state.seq_qlen, ints(tile_seq),
                                ints(tile_row0), table_dev, fast, H, G, d, dv, 0, 0, scale, sink=sink, v_in_k=v_in_k)
        torch.cuda.synchronize()
        err = (fast.cpu().double() - want).abs().max().item()
        assert err <= 3e-2 * max(1.0, want.abs().max().item()), ("tensor-core kernel", err)


@pytest.mark.parametrize("H,G,d,dv,sink,v_in_k", [(4, 2, 16, 24, True, False), (20, 1, 48, 32, False, True),
                                                  (80, 1, 152, 136, False, True), (6, 3, 72, 136, True, False),
                                                  (8, 8, 64, 64, True, False), (3, 1, 256, 8, True, False)])
def test_single_token_kernel_with_heads_as_rows(H, G, d, dv, sink, v_in_k):
    """Single tokens in bfloat16 on tensor cores, a kv head's query heads as the rows of a tile (more than 64 heads
    take two blocks): contexts of one key, at and around page borders, and hundreds of keys with an early one that
    stands out; against the softmax written out."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(H * 100 + d)
    ctxs = [1, 2, 63, 64, 65, 128, 129, 300]
    n = len(ctxs)
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, dv, torch.bfloat16, dev, v_in_k)
    q = torch.randn((n, H * d), generator=gen).to(torch.bfloat16)
    for s in range(n):
        if ctxs[s] > 100:
            mean_q = q[s].float().view(H, d).mean(dim=0)
            k_cache[int(table[s, 0]), :, 3, :] = (k_cache[int(table[s, 0]), :, 3, :].float() + 6.0 * mean_q / mean_q.norm()).to(torch.bfloat16)
    scale = 1.0 / d ** 0.5
    want = torch.cat([_attention_oracle(q[s:s + 1].double().view(1, H, d), _dense(k_cache, table, s, ctxs[s], d),
                                        _dense(v_cache, table, s, ctxs[s], dv), ctxs[s] - 1, scale, sink, H // G)
                      for s in range(n)]).view(n, H * dv)
    state = make_step_state(dev, list(range(n)), [c - 1 for c in ctxs], [1] * n)
    kc = k_cache.to(dev)
    vc = kc if v_in_k else v_cache.to(dev)
    for splits in (1, 3, 16):  # along the context: more splits than some contexts have pages
        out = torch.zeros((n, H * dv), dtype=torch.bfloat16, device=dev)
        scratch = torch.full((K.local_attention_heads_scratch(n, H, dv, splits),), float("nan"), device=dev)
        K.local_attention_heads(q.to(dev), kc, vc, state.seq_slot, state.seq_ctx, state.seq_qstart, state.seq_qlen,
                                table.to(dev), out, n, H, G, d, dv, 0, 0, scale, sink=sink, v_in_k=v_in_k, n_splits=splits,
                                scratch=scratch if splits > 1 else None)
        torch.cuda.synchronize()
        err = (out.cpu().double() - want).abs()
        assert torch.isfinite(out.float()).all()
        assert err.max().item() <= 3e-2 * max(1.0, want.abs().max().item()), (splits, err.max().item(), int(err.argmax()) // (H * dv))


@pytest.mark.parametrize("d", [32, 48, 64, 128])
def test_sink_in_the_kernels_shared_with_the_other_decoders(d):
    """Keys and values of one head size in bfloat16: prompts on the tcgen05 kernel (64, 128) and single tokens on the
    TMA-fed (64, 128) or mma.sync decode kernel, each with the sink, against the general kernel with the sink; scores
    are small, so the sink holds a large share of every row's denominator.  Decode runs with one block a sequence and
    with the context split in four (the sink must be counted once)."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(d)
    H, G = 4, 2
    starts, lens = [0, 70, 129], [300, 200, 1]
    ctxs = [s + n for s, n in zip(starts, lens)]
    k_cache, v_cache, table = _paged(gen, ctxs, G, d, d, torch.bfloat16, dev)
    k_cache, v_cache, table = k_cache.to(dev), v_cache.to(dev), table.to(dev)
    scale = 0.5 / d ** 0.5
    T = sum(lens)
    q = torch.randn((T, H * d), generator=gen).to(torch.bfloat16).to(dev)
    state = make_step_state(dev, [0, 1, 2], starts, lens)
    plain = torch.zeros((T, H * d), dtype=torch.bfloat16, device=dev)
    K.local_attention(q, k_cache, v_cache, state.tok_pos, state.tok_seq, state.seq_slot, table, plain, H, G, d, d, 0, 0, scale,
                      sink=True)
    without = torch.zeros_like(plain)
    K.local_attention(q, k_cache, v_cache, state.tok_pos, state.tok_seq, state.seq_slot, table, without, H, G, d, d, 0, 0, scale)
    torch.cuda.synchronize()
    size = plain.float().abs().max().item()
    assert (plain.float() - without.float()).abs().max().item() > 0.2 * size  # the sink matters in this test
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=dev)
    if K.attention_prefill_takes_chunks(torch.bfloat16, d):
        narrow = [(s, r) for s, n in enumerate(lens) for r in range(0, n, K.PREFILL_TILE)]
        wide = sorted((starts[s] + min(n, r + 128), s, r) for s, n in enumerate(lens) for r in range(0, n, 128))
        fast = torch.zeros_like(plain)
        K.attention_prefill(q, k_cache, v_cache, state.seq_slot, state.seq_ctx, state.seq_qstart, state.seq_qlen,
                            ints([s for s, _ in narrow]), ints([r for _, r in narrow]), table, fast, len(narrow), H, G, d, 0,
                            scale, wide_tiles=(ints([s for _, s, _ in wide]), ints([r for _, _, r in wide])), sink=True)
        torch.cuda.synchronize()
        assert K.take_device_error() == 0
        assert (fast.float() - plain.float()).abs().max().item() <= 0.03 * size
    # single tokens: the last token of every sequence
    last = [sum(lens[:i + 1]) - 1 for i in range(3)]
    q1 = q[last].contiguous()
    one = make_step_state(dev, [0, 1, 2], [c - 1 for c in ctxs], [1, 1, 1])
    for splits in (1, 4):
        out = torch.zeros((3, H * d), dtype=torch.bfloat16, device=dev)
        scratch = torch.zeros((K.attention_decode_scratch_floats(3, H, d, splits),), device=dev) if splits > 1 else None
        counters = torch.zeros((3 * G,), dtype=torch.int32, device=dev) if splits > 1 else None
        K.attention_decode(q1, k_cache, v_cache, one.seq_slot, one.seq_ctx, table, scratch, out, 3, H, G, d, splits, 0, scale,
                           counters=counters, sink=True)
        torch.cuda.synchronize()
        assert K.take_device_error() == 0
        assert (out.float() - plain[last].float()).abs().max().item() <= 0.03 * size, splits


@pytest.mark.parametrize("every,coef", [(1, 1.0), (5, 0.3), (64, 0.7)])
def test_query_temperature_steps_at_the_right_positions(every, coef):
    """The prepare kernel alone: q at positions just before, at and just after every step of the temperature."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.engine.step import make_step_state
    dev = torch.device("cuda:0")
    H, G, d, dv = 2, 1, 8, 4
    positions = sorted({0, 1, every - 2, every - 1, every, every + 1, 2 * every - 1, 2 * every, 3 * every - 1, 3 * every} - {-1})
    n = len(positions)
    gen = torch.Generator().manual_seed(every)
    qkv = torch.randn((n, H * d + G * (d + dv)), generator=gen).to(dev)
    k_cache = torch.zeros((n + 1, G, PAGE, d), device=dev)
    v_cache = torch.zeros((n + 1, G, PAGE, dv), device=dev)
    table = torch.full((n, 4), -1, dtype=torch.int32)
    for s, p in enumerate(positions):
        table[s, p // PAGE] = s
    state = make_step_state(dev, list(range(n)), positions, [1] * n)
    q = torch.zeros((n, H * d), device=dev)
    K.local_attention_prepare(qkv, None, None, None, None, state.tok_pos, state.tok_seq, state.seq_slot, table.to(dev), q,
                              k_cache, v_cache, H, G, d, dv, 0, False, 0.0, q_temp=(coef, every))
    torch.cuda.synchronize()
    factor = torch.tensor([1 + coef * np.log((p + 1) // every + 1) for p in positions]).view(n, 1)
    assert (q.cpu().double() - qkv[:, :H * d].cpu().double() * factor).abs().max().item() < 1e-5
    for s, p in enumerate(positions):  # the key goes unscaled into its page
        assert torch.equal(k_cache[s, 0, p % PAGE].cpu(), qkv[s, H * d:H * d + d].cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D,F", [(1, 5, 2, 40, 24), (37, 7, 3, 56, 16), (300, 3, 3, 50, 30), (64, 1, 1, 32, 8),
                                         (200, 33, 4, 64, 72), (1500, 8, 2, 128, 64)])
def test_routed_feed_forward_kernels(dtype, T, E, top, D, F):
    """route / sort / gate_up / down / combine against the sum written out, for one token, for many tokens per
    expert (tensor-core tiles in bfloat16), for every expert per token and for a single expert; one expert's bias
    is pushed down so that it gets no token at all."""
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(T * 31 + E)
    h = torch.randn((T, D), generator=gen).to(dtype)
    router = torch.randn((E, D), generator=gen) * 2 / D ** 0.5
    bias = torch.randn((E,), generator=gen) * 0.5
    if E > top + 1:
        bias[E // 2] = -50.0
    gate_up = (torch.randn((E, 2 * F, D), generator=gen) * 1.5 / D ** 0.5).to(dtype)
    down = (torch.randn((E, D, F), generator=gen) / F ** 0.5).to(dtype)
    other = torch.randn((T, D), generator=gen).to(dtype)
    z = h.double() @ router.double().T + bias.double()
    chosen_ref = torch.argsort(-z, dim=1, stable=True)[:, :top]
    zc = torch.gather(z, 1, chosen_ref)
    w_ref = torch.softmax(zc, dim=1)
    want = other.double().clone()
    for t in range(T):
        for j in range(top):
            e = int(chosen_ref[t, j])
            gu = gate_up[e].double() @ h[t].double()
            act = gu[:F] / (1 + torch.exp(-gu[:F])) * gu[F:]
            if dtype == torch.bfloat16:
                act = act.to(torch.bfloat16).double()
            want[t] += w_ref[t, j] * (down[e].double() @ act)
    chosen = torch.zeros((T, top), dtype=torch.int32, device=dev)
    weight = torch.zeros((T, top), dtype=torch.float32, device=dev)
    hd = h.to(dev)
    K.moe_route(hd, router.to(dev), bias.to(dev), chosen, weight, top)
    torch.cuda.synchronize()
    margin = (zc[:, -1] - torch.sort(z, dim=1, descending=True).values[:, min(top, E - 1)]).abs() if E > top else None
    sure = torch.ones(T, dtype=torch.bool) if margin is None else margin > 1e-4
    assert torch.equal(chosen.cpu().long()[sure], chosen_ref[sure])
    assert (weight.cpu().double()[sure] - w_ref[sure]).abs().max().item() < 1e-5
    for mma, small in ([(False, 0), (True, 0), (True, 1), (True, 2)] if K.moe_mma_supported(dtype, D, F) else [(False, 0)]):
        rows = K.moe_tile_rows(mma, (1 << 30, 1, 20)[small], 1)  # the tensor-core kernels' tiles of 128, 16 and 32 rows
        n_pairs = T * top
        tiles = K.moe_max_tiles(n_pairs, E, rows)
        ints = lambda n: torch.full((n,), -7, dtype=torch.int32, device=dev)
        plan = K.MoePlan(ints(n_pairs), ints(E + 1), ints(tiles), ints(tiles), ints(1), rows, mma)
        K.moe_sort(chosen, plan, E)
        act = torch.zeros((n_pairs, F), dtype=dtype, device=dev)
        K.moe_gate_up(hd, gate_up.to(dev), act, plan, top)
        y = torch.zeros((n_pairs, D), dtype=torch.float32, device=dev)
        K.moe_down(act, down.to(dev), y, weight, plan, top)
        out = torch.zeros((T, D), dtype=dtype, device=dev)
        K.moe_combine(y, other.to(dev), out, top)
        torch.cuda.synchronize()
        offsets = plan.offsets.cpu().tolist()
        counts = torch.bincount(chosen.cpu().view(-1).long(), minlength=E).tolist()
        assert [b - a for a, b in zip(offsets, offsets[1:])] == counts
        assert sorted(plan.order.cpu().tolist()) == list(range(n_pairs))
        assert int(plan.n_tiles.cpu()) == sum(-(-c // rows) for c in counts)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        err = (out.cpu().double() - want)[sure].abs().max().item()
        assert err <= tol * max(1.0, want.abs().max().item()), (mma, small, err)


@pytest.mark.parametrize("width", [40, 50, 256, 1000, 4096, 9000])
def test_layer_norm_kernel(width):
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(width)
    x = (torch.randn((9, width), generator=gen) * 3 + 5).to(dev)   # a mean far from zero: E[x^2] - mean^2 would lose digits
    delta = torch.randn((9, width), generator=gen).to(torch.bfloat16).to(dev)
    w, b = torch.randn((width,), generator=gen).to(dev), torch.randn((width,), generator=gen).to(dev)
    summed = x.cpu().double() + delta.cpu().double()
    mean = summed.mean(dim=1, keepdim=True)
    want = (summed - mean) / torch.sqrt(((summed - mean) ** 2).mean(dim=1, keepdim=True) + 1e-5) * w.cpu().double() + b.cpu().double()
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=dev)
    gathered = torch.zeros((3, width), dtype=torch.float32, device=dev)
    before = x.clone()
    K.add_layernorm(x, delta, w, b, gathered, 1e-5, rows)
    assert torch.equal(x, before)  # gathered rows leave the stream alone
    assert (gathered.cpu().double() - want[[8, 0, 3]]).abs().max().item() < 2e-5
    out = torch.zeros((9, width), dtype=torch.float32, device=dev)
    K.add_layernorm(x, delta, w, b, out, 1e-5)
    assert (x.cpu().double() - summed).abs().max().item() < 1e-6
    assert (out.cpu().double() - want).abs().max().item() < 2e-5


def test_gate_and_stream_kernels():
    from cpp_minilamma_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(5)
    T, H, dv = 7, 3, 10
    values = torch.randn((T, H * dv), generator=gen).to(dev)
    rows = torch.randn((T, 5 + H * dv), generator=gen).to(dev)
    out = torch.zeros_like(values)
    K.heads_gate(values, rows, 5, out, H, dv, per_head=True)
    want = values.view(T, H, dv) * torch.sigmoid(rows[:, 5:5 + H]).view(T, H, 1)
    assert (out.view(T, H, dv) - want).abs().max().item() < 1e-6
    K.heads_gate(values.view(T, H, dv).transpose(0, 1).contiguous(), rows, 5, out, H, dv, per_head=False, head_major=True)
    assert (out - values * torch.sigmoid(rows[:, 5:])).abs().max().item() < 1e-6
    x, x0 = torch.randn((T, 12), generator=gen).to(dev), torch.randn((T, 12), generator=gen).to(dev)
    delta = torch.randn((T, 12), generator=gen).to(torch.bfloat16).to(dev)
    both = torch.zeros((T, 24), dtype=torch.bfloat16, device=dev)
    K.stream_concat(x, delta, x0, both)
    assert torch.equal(both[:, :12], (x + delta.float()).to(torch.bfloat16)) and torch.equal(both[:, 12:], x0.to(torch.bfloat16))
