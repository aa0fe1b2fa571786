"""GPU end-to-end parity: ModelRunner / Engine on the config-1 model against the golden logits and tokens the
reference's own CPU model (`qwen38-ref`, engine mode, int8 KV) produced for the same file and prompts, and
against the whole-model oracle. Mirrors reference tests/gpu/test_e2e.cpp and adds ragged multi-sequence steps,
page-id checks and error paths."""

import warnings
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np
import pytest

import q38_testlib as tl
from oracle_model import OracleModel
from q38b200 import engine as eng

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
LENS = (17, 64, 65, 130)


def tiny_options(**kw):
    base = dict(max_batch=4, prefill_chunk=128, kv_dtype=0, kv_tokens=8192, max_context=4096, verbose=0)
    base.update(kw)
    return eng.default_runner_options(**base)


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "tiny_cfg1_golden.npz")


def rel_max(got, want):
    return float(np.abs(got - want).max() / np.abs(want).max())


def top1_agreement(got, want, tol=2e-2):
    """(agreeing rows, rows, agreeing decisive rows, decisive rows). A row is decisive when the reference's
    margin between its two largest logits exceeds twice the allowed logit error (tol * max|ref|): below that no
    summation order can be expected to reproduce the argmax (the N(0, 0.02) model has |logit| < 2)."""
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    same = got.argmax(-1) == want.argmax(-1)
    top2 = np.sort(want, axis=-1)[:, -2:]
    decisive = (top2[:, 1] - top2[:, 0]) > 2 * tol * np.abs(want).max()
    return int(same.sum()), len(same), int((same & decisive).sum()), int(decisive.sum())


def check_agreement(tag, counts, record=None, bar=None):
    """Asserts 100 % agreement on decisive rows and `bar` on all rows; the raw counts go into the test report
    (a user property and a warning line, so that a passing run records them too)."""
    agree, total, dagree, dtotal = (int(x) for x in counts)
    line = f"top-1{tag or '_n002'}: {agree}/{total} rows ({agree / max(1, total):.4f}), decisive rows {dagree}/{dtotal}"
    print(line)
    if record is not None:
        record("top1" + (tag or "_n002"), line)
    warnings.warn(line)
    assert dagree == dtotal, "a clearly separated argmax differs from the reference: " + line
    # The O(1)-activation model is held to the 99 % greedy agreement the engine is specified to reach. The N(0, 0.02)
    # model's 1024 logits all lie within +-2 and a third of its rows are near-ties (top-2 margin below twice the allowed
    # logit error), which no summation order reproduces: it is held to the reference's own end-to-end bar of 95 %
    # (reference tests/gpu/test_e2e.cpp:86) and its raw figure is reported.
    if bar is None:
        bar = 0.99 if tag == "_unit" else 0.95
    assert agree >= bar * total, line


def prefill_all(runner, slot, tokens, chunk):
    """Logits of every position through chunked prefill."""
    out = []
    for p0 in range(0, len(tokens), chunk):
        out.append(runner.prefill_logits(slot, p0, tokens[p0:p0 + chunk]))
    return np.concatenate(out)


@pytest.mark.parametrize("tag", ["", "_unit"])
@pytest.mark.parametrize("chunk", [64, 128])
def test_prefill_logits_match_reference_model(gold, tag, chunk, record_property):
    model = eng.Model(GOLD / f"tiny_cfg1{tag}.q38")
    runner = eng.Runner(model, tiny_options(prefill_chunk=chunk))
    counts = np.zeros(4, dtype=int)
    worst = 0.0
    for i, n in enumerate(LENS):
        full = np.concatenate([gold[f"prompt{i}"], gold[f"gen{tag}{i}"]])
        want = gold[f"logits{tag}{i}"].astype(np.float32)
        runner.reset_slot(i)
        got = prefill_all(runner, i, full, chunk)
        worst = max(worst, rel_max(got, want))
        counts += top1_agreement(got, want)
    print(f"prefill{tag} chunk {chunk}: rel_max {worst:.3e}")
    assert worst <= 2e-2
    check_agreement(tag, counts, record_property)  # every prefill position of the four prompts + continuations: 404 rows
    runner.close()
    model.close()


@pytest.mark.parametrize("tag", ["", "_unit"])
def test_ragged_batch_decode_matches_reference_step_by_step(gold, tag, record_property):
    """Config 1: the four prompts prefilled (one ragged step per chunk round), then 32 greedy decode steps as
    one ragged batch with teacher forcing on the reference's tokens; logits compared at every step."""
    model = eng.Model(GOLD / f"tiny_cfg1{tag}.q38")
    runner = eng.Runner(model, tiny_options(prefill_chunk=128))
    g = eng.greedy()
    prompts = [gold[f"prompt{i}"] for i in range(4)]
    gens = [gold[f"gen{tag}{i}"] for i in range(4)]
    refs = [gold[f"logits{tag}{i}"].astype(np.float32) for i in range(4)]
    for s in range(4):
        runner.reset_slot(s)
        assert runner.kv_ensure(s, len(prompts[s]) + 33)
    # ragged prefill: prompts 17 + 64 in one step (81 tokens), then 65, then 130 as 128 + 2 with 65's tail...
    toks, _ = runner.prefill([(0, 0, prompts[0], g, 0), (1, 0, prompts[1], g, 0)])
    first = {0: int(toks[0]), 1: int(toks[1])}
    toks, _ = runner.prefill([(2, 0, prompts[2], g, 0), (3, 0, prompts[3][:60], None, 0)])
    first[2] = int(toks[0])
    toks, _ = runner.prefill([(3, 60, prompts[3][60:], g, 0)])
    first[3] = int(toks[0])
    counts = np.zeros(4, dtype=int)
    worst = 0.0
    for step in range(32):
        rows = [(s, len(prompts[s]) + step, int(gens[s][step]), g, step + 1) for s in range(4)]
        toks, _ = runner.decode(rows)
        logits = runner.last_logits(4)
        for s in range(4):
            want = refs[s][len(prompts[s]) + step]
            worst = max(worst, rel_max(logits[s], want))
            counts += top1_agreement(logits[s], want)
            assert int(toks[s]) == int(logits[s].argmax()), "greedy token = lowest-id argmax of the logits"
    print(f"decode{tag}: rel_max {worst:.3e}; first sampled tokens {first} vs reference {[int(g[0]) for g in gens]}")
    assert worst <= 2e-2
    # 128 rows: one flipped near-tie is 0.8 %, so this small sample is held to two rows; the 404-row prefill test
    # above carries the 99 % bar
    check_agreement(tag, counts, record_property, bar=(126 / 128 if tag == "_unit" else 0.95))
    runner.close()
    model.close()


@pytest.mark.parametrize("kv_dtype", [0, 1])
def test_random_prompt_against_whole_model_oracle(kv_dtype):
    """120 random tokens (seed 21) through prefill_logits vs the oracle model, int8 and bf16 KV
    (reference tests/gpu/test_e2e.cpp:56-88: mean KL < 2e-3, top-1 >= 95%)."""
    path = GOLD / "tiny_cfg1_unit.q38"
    model = eng.Model(path)
    runner = eng.Runner(model, tiny_options(kv_dtype=kv_dtype))
    tokens = np.random.default_rng(21).integers(0, 1000, size=120).astype(np.int32)
    got = runner.prefill_logits(0, 0, tokens)
    om = OracleModel(path, kv_dtype=2 if kv_dtype == 0 else 1, max_positions=128)
    want = om.forward(om.new_sequence(), tokens, all_logits=True)

    def logsm(x):
        x = x.astype(np.float64)
        x = x - x.max(-1, keepdims=True)
        return x - np.log(np.exp(x).sum(-1, keepdims=True))
    lw, lg = logsm(want), logsm(got)
    kl = (np.exp(lw) * (lw - lg)).sum(-1)
    top1 = (got.argmax(-1) == want.argmax(-1)).mean()
    print(f"kv={kv_dtype}: KL mean {kl.mean():.2e} max {kl.max():.2e}, top-1 {top1:.3f}, rel_max {rel_max(got, want):.2e}")
    assert kl.mean() < 2e-3 and top1 >= 0.95 and rel_max(got, want) <= 2e-2
    runner.close()
    model.close()


def test_chunked_prefill_then_graph_decode_is_consistent():
    """One 100-token prefill vs chunks 37 + 23 then 40 CUDA-graph decode steps (reference test_e2e.cpp:90-132)."""
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    runner = eng.Runner(model, tiny_options())
    tokens = np.random.default_rng(8).integers(0, 1000, size=100).astype(np.int32)
    runner.reset_slot(0)
    full = runner.prefill_logits(0, 0, tokens)
    runner.kv_release(0)
    runner.reset_slot(1)
    assert runner.kv_ensure(1, 101)
    g = eng.greedy()
    runner.prefill([(1, 0, tokens[:37], None, 0)])
    toks, _ = runner.prefill([(1, 37, tokens[37:60], g, 0)])
    agree = int(toks[0] == full[59].argmax())
    for pos in range(60, 100):
        toks, _ = runner.decode([(1, pos, int(tokens[pos]), g, pos)])
        agree += int(toks[0] == full[pos].argmax())
    assert agree >= 41 - 2
    # graphs on and off give the same tokens
    runner.reset_slot(2)
    assert runner.kv_ensure(2, 101)
    runner.set_graphs(False)
    runner.prefill([(2, 0, tokens[:60], None, 0)])
    eager = [int(runner.decode([(2, pos, int(tokens[pos]), g, pos)])[0][0]) for pos in range(60, 70)]
    runner.set_graphs(True)
    runner.reset_slot(3)
    assert runner.kv_ensure(3, 101)
    runner.prefill([(3, 0, tokens[:60], None, 0)])
    graph = [int(runner.decode([(3, pos, int(tokens[pos]), g, pos)])[0][0]) for pos in range(60, 70)]
    assert eager == graph
    runner.close()
    model.close()


def test_engine_batches_independent_sequences(gold):
    """Four requests together = each alone (reference test_e2e.cpp:134-181), plus the golden continuations."""
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    prompts = [gold[f"prompt{i}"] for i in range(4)]
    alone = []
    e = eng.Engine(model, tiny_options())
    for p in prompts:
        e.submit(p, eng.greedy(), max_new_tokens=32, ignore_eos=True)
        e.run()
        alone.append(e.take_finished()[0].tokens)
    e.close()
    # mixed: the generating sequences' tokens ride in the prefill steps of the prompts still pending (prompts 17 and 64
    # finish in the first step and decode inside the steps that prefill 65 and 130)
    for ragged, mixed in ((False, False), (True, False), (True, True), (False, True)):
        e = eng.Engine(model, tiny_options(), ragged_prefill=ragged, mixed_steps=mixed)
        for p in prompts:
            e.submit(p, eng.greedy(), max_new_tokens=32, ignore_eos=True)
        e.run()
        done = sorted(e.take_finished(), key=lambda r: r.id)
        st = e.stats()
        assert len(done) == 4 and all(len(r.tokens) == 32 and r.finish == "length" for r in done)
        assert st.decode_tokens / max(1, st.decode_steps) > 1.5
        assert st.prefill_tokens == sum(LENS)
        same = gold_same = either = whole = 0
        for i, r in enumerate(done):
            # free-running generation: after the first near-tie flip a continuation differs legitimately, and the run
            # alone is itself one such continuation. Counted per sequence: the common prefix with the run alone, with
            # the reference's continuation, and the longer of the two (the step-by-step test above is the
            # teacher-forced comparison, which has no such freedom)
            ref_gen = gold[f"gen_unit{i}"]
            with_alone = with_ref = 0
            while with_alone < 32 and r.tokens[with_alone] == alone[i][with_alone]:
                with_alone += 1
            while with_ref < 32 and r.tokens[with_ref] == ref_gen[with_ref]:
                with_ref += 1
            assert with_ref >= 1, "the first generated token must match the reference"
            same += with_alone
            gold_same += with_ref
            either += max(with_alone, with_ref)
            whole += max(with_alone, with_ref) == 32
        print(f"ragged={ragged} mixed={mixed}: batched vs alone {same}/128; common prefix with the reference tokens "
              f"{gold_same}/128; with either {either}/128; whole sequences {whole}/4")
        # One near-tie flip ends a sequence's agreement for good (a third of the rows of this random 1024-word model
        # are near-ties, and a ragged or mixed step sums in another order than the run alone), so the bar is per
        # sequence: at most one of the four may leave both references, two in a mixed schedule, whose generating
        # sequences are computed inside prefill-sized GEMM passes.
        assert whole >= (2 if mixed else 3), (same, gold_same, either)
        assert either >= (0.5 if mixed else 0.7) * 128
        assert gold_same >= 0.4 * 128
        e.close()
    model.close()


def test_engine_error_results_and_stop_tokens():
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    e = eng.Engine(model, tiny_options(kv_tokens=256, max_context=512))
    ids = [e.submit([], eng.greedy(), 4), e.submit(np.zeros(600, np.int32), eng.greedy(), 4),
           e.submit(np.arange(300, dtype=np.int32), eng.greedy(), 64, ignore_eos=True)]
    e.run()
    done = {r.id: r for r in e.take_finished()}
    assert done[ids[0]].finish == "error" and "empty prompt" in done[ids[0]].error
    assert done[ids[1]].finish == "error" and "context limit" in done[ids[1]].error
    assert done[ids[2]].finish == "error" and "more KV cache" in done[ids[2]].error
    # a stop token ends the request with reason "stop" and is part of the output
    prompt = np.random.default_rng(4).integers(0, 1000, size=20).astype(np.int32)
    e.submit(prompt, eng.greedy(), 16, ignore_eos=True)
    e.run()
    free = e.take_finished()[0].tokens
    e.submit(prompt, eng.greedy(), 16, stop_tokens=[int(free[3])])
    e.run()
    r = e.take_finished()[0]
    first = int(np.argmax(free == free[3]))
    assert r.finish == "stop" and list(r.tokens) == list(free[:first + 1])
    e.close()
    model.close()


def test_kv_page_ids_follow_the_reference_free_list():
    """Page ids are part of the parity contract: a Python model of the reference's free list
    (src/kv_cache.cpp:34-35, 53-76: page 0 first, LIFO reuse) must predict every block-table row."""
    model = eng.Model(GOLD / "tiny_cfg1.q38")
    runner = eng.Runner(model, tiny_options(kv_tokens=64 * 40))
    pages = 41
    free = list(range(pages - 1, -1, -1))
    owned = {s: [] for s in range(5)}

    def ensure(slot, tokens):
        need = (tokens + 63) // 64 - len(owned[slot])
        if need <= 0:
            return True
        if need > len(free):
            return False
        for _ in range(need):
            owned[slot].append(free.pop())
        return True

    def release(slot):
        free.extend(reversed(owned[slot]))
        owned[slot].clear()

    assert ensure(4, 1)  # the runner's dummy sequence owns the first page
    rng = np.random.default_rng(1)
    for _ in range(200):
        slot = int(rng.integers(0, 4))
        if rng.random() < 0.6:
            tokens = int(rng.integers(1, 900))
            assert runner.kv_ensure(slot, tokens) == ensure(slot, tokens)
        else:
            runner.kv_release(slot)
            release(slot)
        assert runner.kv_pages(slot) == owned[slot]
        assert runner.kv_free_pages() == len(free)
    runner.close()
    model.close()


def test_sampled_generation_is_reproducible_and_scores_match_logits():
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    outs = []
    for _ in range(2):
        e = eng.Engine(model, tiny_options(), seed=77)
        e.submit(np.arange(40, dtype=np.int32), eng.Sampling(0.8, 50, 0.95, 0.0, 0.3, 1.1, 0), 24, ignore_eos=True)
        e.run()
        outs.append(e.take_finished()[0].tokens)
        e.close()
    assert np.array_equal(outs[0], outs[1])
    runner = eng.Runner(model, tiny_options())
    tokens = np.random.default_rng(2).integers(0, 1000, size=50).astype(np.int32)
    targets = np.roll(tokens, -1)
    lp = runner.score(0, 0, tokens, targets)
    runner.kv_release(0)
    runner.reset_slot(0)
    logits = runner.prefill_logits(0, 0, tokens).astype(np.float64)
    want = logits[np.arange(50), targets] - np.log(np.exp(logits - logits.max(-1, keepdims=True)).sum(-1)) - logits.max(-1)
    assert np.allclose(lp, want, atol=2e-4)
    runner.close()
    model.close()


# ---------------------------------------------------------------------------------------------------
# the benchmarked geometry end to end
# ---------------------------------------------------------------------------------------------------
def test_27b_geometry_truncated_model_matches_oracle(tmp_path_factory, record_property):
    """The 27B model's geometry (hidden 5120, 24 q / 4 kv heads, GDN 16 key / 48 value heads, MLP 17408) cut to its
    first four layers [GDN, GDN, GDN, attention] with a 1024-row vocabulary (the reference's CPU model refuses more
    than 3e9 parameters, reference src/ref/ref_model.cpp:21-58), N(0, 0.02) weights, default recipe through the real
    quantiser. 36 sequences: ragged prefill in steps of at most 512 tokens, then 16 decode steps as one batch of 36
    (the tcgen05 kernel with the weights in tensor memory, 64-token configuration, and its Residual / SwiGLU
    epilogues), greedy with the engine's own tokens fed back. The oracle model runs every sequence on its own host
    thread with the same tokens; logits are compared at every sampled position."""
    from q38b200 import synth
    import torch

    cfg = synth.model_config(hidden=5120, vocab=1024, layers=4, intermediate=17408, nq=24, nkv=4, lk=16, lv=48)
    path = tmp_path_factory.mktemp("q38") / "geom27b_4layers.q38"
    synth.write_q38(path, cfg, synth.random_checkpoint(cfg, seed=27, init="n002"), recipe="default", device="cuda")
    torch.cuda.empty_cache()
    B, STEPS = 36, 16
    rng = np.random.default_rng(11)
    lens = [int(x) for x in rng.integers(2, 9, size=B)]
    lens[0], lens[1] = 70, 130  # two prompts that cross KV pages and GDN chunks
    prompts = [rng.integers(0, 1000, size=n).astype(np.int32) for n in lens]

    model = eng.Model(path)
    runner = eng.Runner(model, eng.default_runner_options(max_batch=64, prefill_chunk=512, kv_dtype=0, kv_tokens=64 * 256,
                                                          max_context=1024, verbose=0))
    g = eng.greedy()
    got = [[] for _ in range(B)]       # logits rows per sequence, in sampling order
    fed = [list(p) for p in prompts]   # tokens each sequence has consumed
    for s in range(B):
        runner.reset_slot(s)
        assert runner.kv_ensure(s, lens[s] + STEPS + 1)
    # ragged prefill: whole prompts packed into steps of at most 512 tokens
    nxt = [0] * B
    rows, used = [], 0
    order = []
    def flush():
        nonlocal rows, used
        if not rows:
            return
        toks, _ = runner.prefill(rows)
        logits = runner.last_logits(len(rows))
        for i, (slot, *_rest) in enumerate(rows):
            got[slot].append(logits[i].copy())
            nxt[slot] = int(toks[i])
        rows, used = [], 0
    for s in range(B):
        if used + lens[s] > 512:
            flush()
        rows.append((s, 0, prompts[s], g, 0))
        used += lens[s]
    flush()
    for step in range(STEPS):
        drows = [(s, lens[s] + step, nxt[s], g, step + 1) for s in range(B)]
        for s in range(B):
            fed[s].append(nxt[s])
        toks, _ = runner.decode(drows)
        logits = runner.last_logits(B)
        for s in range(B):
            got[s].append(logits[s].copy())
            nxt[s] = int(toks[s])
    runner.close()
    model.close()

    om = OracleModel(path, kv_dtype=2, max_positions=160)

    def reference_rows(s):
        seq = om.new_sequence()
        out = [om.forward(seq, fed[s][:lens[s]])[0]]
        for t in fed[s][lens[s]:lens[s] + STEPS]:
            out.append(om.forward(seq, [t])[0])
        return out

    with ThreadPoolExecutor(max_workers=16) as pool:
        want = list(pool.map(reference_rows, range(B)))
    worst, counts = 0.0, np.zeros(4, dtype=int)
    for s in range(B):
        assert len(got[s]) == STEPS + 1 and len(want[s]) == STEPS + 1
        for a, b in zip(got[s], want[s]):
            worst = max(worst, rel_max(a, b))
            counts += top1_agreement(a, b)
    record_property("rel_max_27b_geometry", worst)
    warnings.warn(f"27B geometry, 4 layers, batch {B}: max rel logit error {worst:.3e}")
    assert worst <= 2e-2
    check_agreement("_geom27b", counts, record_property, bar=0.95)


def test_a_device_error_word_fails_the_step_and_the_engine_carries_on():
    """Every kernel reports a pipeline abort (a bounded wait that ran out, a page id outside the pool) through the
    library's device error word. The failure is made on the host here: the word is set with the library's test hook,
    no kernel misbehaves. The next step must raise instead of returning tokens, the word must be re-armed, and the
    Engine must end that step's requests with an error result and serve the next request normally."""
    K = tl.pkg.kernels()
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    runner = eng.Runner(model, tiny_options())
    g = eng.greedy()
    tokens = np.random.default_rng(5).integers(0, 1000, size=20).astype(np.int32)
    runner.reset_slot(0)
    assert runner.kv_ensure(0, 64)
    toks, _ = runner.prefill([(0, 0, tokens, g, 0)])
    good, _ = runner.decode([(0, 20, int(toks[0]), g, 1)])
    tl.pkg.check(K.q38_device_error_inject(0x303))
    with pytest.raises(eng.EngineError, match="0x303"):
        runner.decode([(0, 21, int(good[0]), g, 2)])
    again, _ = runner.decode([(0, 21, int(good[0]), g, 2)])  # same step once more: clean
    assert again.shape == (1,)
    tl.pkg.check(K.q38_device_error_inject(0x212))
    with pytest.raises(eng.EngineError, match="prefill step"):
        runner.prefill([(0, 22, tokens[:5], g, 3)])
    assert K.q38_device_error(1) == 0, "the collected word is cleared in the library"
    runner.close()

    e = eng.Engine(model, tiny_options())
    first = e.submit(tokens, g, max_new_tokens=8, ignore_eos=True)
    tl.pkg.check(K.q38_device_error_inject(0x305))
    e.run()
    second = e.submit(tokens, g, max_new_tokens=8, ignore_eos=True)
    e.run()
    done = {r.id: r for r in e.take_finished()}
    assert done[first].finish == "error" and "0x305" in done[first].error
    assert done[second].finish == "length" and len(done[second].tokens) == 8
    e.close()
    model.close()


def test_more_requests_than_slots_are_queued_and_all_finish():
    """Slot exhaustion: seven requests on an engine with two sequence slots. The scheduler admits them as slots and KV
    pages come back; every request finishes with its full length, in mixed-step mode as well, and the tokens of each
    request do not depend on what shared the batch with it."""
    model = eng.Model(GOLD / "tiny_cfg1_unit.q38")
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, 1000, size=int(n)).astype(np.int32) for n in (5, 70, 33, 129, 64, 9, 200)]
    outs = {}
    for mixed in (False, True):
        e = eng.Engine(model, tiny_options(max_batch=2, kv_tokens=64 * 12), ragged_prefill=True, mixed_steps=mixed)
        ids = [e.submit(p, eng.greedy(), max_new_tokens=12, ignore_eos=True) for p in prompts]
        e.run()
        done = {r.id: r for r in e.take_finished()}
        assert sorted(done) == sorted(ids)
        assert all(done[i].finish == "length" and len(done[i].tokens) == 12 for i in ids)
        st = e.stats()
        assert st.requests_done == 7 and st.prefill_tokens == sum(len(p) for p in prompts)
        outs[mixed] = [done[i].tokens for i in ids]
        e.close()
    same = sum(int(np.array_equal(a, b)) for a, b in zip(outs[False], outs[True]))
    assert same >= 5, "mixed steps changed more than near-tie continuations"
    model.close()
