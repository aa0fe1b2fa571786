"""Tensor-parallel runner against the reference model's logits: the same tiny model as the engine tests, run through
TPRunner on one rank (sharding code path without all-reduce) and on two ranks over NCCL."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
GOLD = ROOT / "tests" / "golden"
pytestmark = pytest.mark.gpu


def _check_against_golden(runner, tag, seq, graph_from=16, log=None):
    gold = np.load(GOLD / "tiny_cfg1_golden.npz")
    prompt, gen = gold[f"prompt{seq}"], gold[f"gen{tag}{seq}"]
    ref = gold[f"logits{tag}{seq}"].astype(np.float32)
    rel = lambda got, want: float(np.abs(got - want).max() / np.abs(want).max())
    say = log or (lambda *a: None)
    runner.forward(prompt, 0)
    worst = rel(runner.logits(), ref[len(prompt) - 1])
    say(f"prefill rel {worst:.3e}")
    agree = 0
    for step in range(len(gen)):
        pos = len(prompt) + step
        if step < graph_from:
            runner.forward([int(gen[step])], pos)      # eager launches
        else:
            runner.decode_replay(int(gen[step]), pos)  # captured step (kernels + all-reduces)
        got = runner.logits()
        say(f"step {step} rel {rel(got, ref[pos]):.3e}")
        worst = max(worst, rel(got, ref[pos]))
        agree += int(got.argmax() == ref[pos].argmax())
    assert runner.device_error() == 0
    assert worst <= 2e-2, worst
    assert agree >= 0.9 * len(gen), agree
    return worst, agree


def test_single_rank_tp_runner_matches_reference():
    import __graft_entry__ as entry
    entry.load_package()
    import q38b200
    from q38b200 import tp
    for tag in ("", "_unit"):
        runner = tp.TPRunner(q38b200, GOLD / f"tiny_cfg1{tag}.q38", max_tokens=256, max_context=512)
        worst, agree = _check_against_golden(runner, tag, 3)
        print(f"tp x1{tag}: rel_max {worst:.3e}, top-1 {agree}/32")
        assert worst <= 2e-2


def test_fused_allreduce_on_one_rank_equals_the_separate_path():
    """The all-reduce inside the row-parallel GEMM (push of the tile to every rank's buffer, flags, bounded wait, sum in
    rank order, residual update) with a world of one: the rank pushes to and pulls from itself, so every step of up to
    16 tokens must give the logits of the path with a separate residual update - eagerly and as a replayed graph."""
    import __graft_entry__ as entry
    entry.load_package()
    import q38b200
    from q38b200 import tp
    gold = np.load(GOLD / "tiny_cfg1_golden.npz")
    prompt, gen = gold["prompt3"], gold["gen_unit3"]
    runs = []
    for fused in (False, True):
        runner = tp.TPRunner(q38b200, GOLD / "tiny_cfg1_unit.q38", max_tokens=256, max_context=512, fused_allreduce=fused)
        runner.forward(prompt, 0)
        rows = [runner.logits()]
        for step in range(12):
            pos = len(prompt) + step
            if step < 3:
                runner.forward([int(gen[step])], pos)
            elif step == 3:
                runner.forward([int(t) for t in gen[3:8]], pos)  # five tokens in one step (still the fused path)
            elif step >= 8:
                runner.decode_replay(int(gen[step]), pos)
            else:
                continue
            rows.append(runner.logits())
        assert runner.device_error() == 0
        assert (runner.fused_calls > 0) == fused
        runs.append(rows)
        runner.close()
    assert len(runs[0]) == len(runs[1])
    # the same sums in the same order; only the norm statistics are accumulated by another kernel (the GEMM epilogue's
    # lane order instead of the update kernel's), which moves the logits in the last bits
    for a, b in zip(*runs):
        assert float(np.abs(a - b).max()) <= 1e-4 * float(np.abs(a).max())


def test_fused_allreduce_wait_gives_up_when_a_rank_never_arrives():
    """A world of two in which the other rank does not exist (its buffers are local stand-ins nobody writes): the wait
    for its flag runs out after the given number of polls, the kernel records the error and completes, and the host
    reads the error word. Nothing hangs and nothing faults; the context stays usable."""
    import __graft_entry__ as entry
    entry.load_package()
    import q38b200
    from q38b200 import tp
    gold = np.load(GOLD / "tiny_cfg1_golden.npz")
    runner = tp.TPRunner(q38b200, GOLD / "tiny_cfg1_unit.q38", 0, 2, None, max_tokens=256, max_context=512,
                         fused_allreduce=True, poll_limit=2000)
    runner.forward(gold["prompt3"][:64], 0)        # 64 tokens: the separate path, no wait
    assert runner.device_error() == 0
    runner.forward([int(gold["gen_unit3"][0])], 64)  # one token: the fused path waits for rank 1
    torch.cuda.synchronize()
    assert runner.device_error() == 0x120
    assert runner.device_error() == 0                # the word was cleared by the read; the context still works
    runner.forward(gold["prompt3"][:32], 65)
    torch.cuda.synchronize()
    assert runner.device_error() == 0
    runner.close()


def _worker(rank, world, port, out_dir, graph_from, fused=False):
    logf = open(Path(out_dir) / f"rank{rank}.log", "w")

    def log(*a):
        print(*a, file=logf, flush=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import __graft_entry__ as entry
    entry.load_package()
    import q38b200
    from q38b200 import tp
    log("process group up")
    runner = tp.TPRunner(q38b200, GOLD / "tiny_cfg1_unit.q38", rank, world, dist, max_tokens=256, max_context=512,
                         fused_allreduce=fused)
    log("runner built")
    worst, agree = _check_against_golden(runner, "_unit", 3, graph_from=graph_from, log=log)
    log("checked", worst, agree)
    assert runner.reduce_calls > 0
    assert (runner.fused_calls > 0) == fused
    runner.close()
    del runner
    log("closed")
    dist.barrier()
    log("barrier passed")
    dist.destroy_process_group()
    (Path(out_dir) / f"ok{rank}").write_text(f"{worst:.3e} {agree}")


def _log_dir(tmp_path, name):
    """Where the ranks write their progress logs: Q38_TEST_LOG_DIR if set (to keep them after the run), else tmp."""
    base = os.environ.get("Q38_TEST_LOG_DIR")
    d = Path(base) / name if base else tmp_path
    d.mkdir(parents=True, exist_ok=True)
    return d


@pytest.mark.timeout(150)
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fused", [False, True], ids=["nccl", "fused"])
@pytest.mark.parametrize("graph_from", [99, 8], ids=["eager", "graph"])
def test_two_rank_tp_runner_matches_reference(tmp_path, graph_from, fused):
    """Two ranks; "graph" replays the decode step as a CUDA graph from step 8 on. "nccl": all-reduce by NCCL between the
    GEMM and the residual update; "fused": decode steps sum the partial products inside the GEMM over peer memory (plain
    loads and stores only), the 130-token prefill still goes through NCCL."""
    import torch.multiprocessing as mp
    world, port = 2, 29100 + (os.getpid() + graph_from + 7 * int(fused)) % 2000
    d = _log_dir(tmp_path, f"tp2_{graph_from}_{int(fused)}")
    mp.spawn(_worker, args=(world, port, str(d), graph_from, fused), nprocs=world, join=True)
    print([(d / f"ok{r}").read_text() for r in range(world)])


@pytest.mark.timeout(120)
@pytest.mark.parametrize("rank", [0, 1])
def test_rank_shard_shapes_run_without_a_process_group(rank):
    """The kernels on one rank's shard shapes of a two-way split (k ranges of 128..512, two-tile projections), without
    the all-reduce: values are partial sums, so only completion, finiteness and the device error word are checked."""
    import __graft_entry__ as entry
    entry.load_package()
    import q38b200
    from q38b200 import tp
    gold = np.load(GOLD / "tiny_cfg1_golden.npz")
    runner = tp.TPRunner(q38b200, GOLD / "tiny_cfg1_unit.q38", rank, 2, None, max_tokens=256, max_context=512)
    runner.forward(gold["prompt3"], 0)
    assert np.isfinite(runner.logits()).all()
    for step in range(4):
        runner.forward([int(gold["gen_unit3"][step])], 130 + step)
    for step in range(4, 8):
        runner.decode_replay(int(gold["gen_unit3"][step]), 130 + step)
    assert np.isfinite(runner.logits()).all()
    assert runner.device_error() == 0
