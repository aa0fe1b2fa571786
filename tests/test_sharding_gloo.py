"""Request sharding and the cross-rank reductions of a benchmark run, as two gloo ranks on CPU."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import __graft_entry__ as entry
    entry.load_package()
    from q38b200 import sharding
    dist.init_process_group("gloo", rank=rank, world_size=world)
    reqs = sharding.trace_requests(512, seed=11)
    mine = sharding.shard_requests(reqs, rank, world)
    gathered = [None] * world
    dist.all_gather_object(gathered, [i for i, _ in mine])
    # every request is served by exactly one replica, loads differ by at most one request
    flat = sorted(i for part in gathered for i in part)
    assert flat == list(range(512))
    assert max(len(p) for p in gathered) - min(len(p) for p in gathered) <= 1
    assert all(i % world == rank for i, _ in mine)
    # the job's time is the slowest rank's; the whole-job rate counts every rank's units
    local = [1.0 + rank, 10.0 - rank]
    t = sharding.max_over_ranks(local, dist)
    assert t == [float(world), 10.0]
    assert sharding.whole_job_rate(64 * 20, world, t[0]) == 64 * 20 * world / float(world)
    dist.barrier()
    dist.destroy_process_group()
    (Path(out_dir) / f"ok{rank}").write_text("ok")


def test_request_sharding_two_gloo_ranks(tmp_path):
    world, port = 2, 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_single_rank_is_identity():
    import __graft_entry__ as entry
    entry.load_package()
    from q38b200 import sharding
    reqs = sharding.trace_requests(16)
    assert [r for _, r in sharding.shard_requests(reqs, 0, 1)] == reqs
    assert sharding.max_over_ranks([3.0, 4.0]) == [3.0, 4.0]
    assert all(64 <= p <= 8192 and 64 <= o <= 1024 for p, o in sharding.trace_requests(512))
