"""Request sharding and the cross-rank reductions of a benchmark run, as two gloo ranks on CPU."""
import os
import time
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


def test_dispatcher_policies_and_redeal():
    import __graft_entry__ as entry
    entry.load_package()
    from q38b200 import sharding
    reqs = sharding.trace_requests(64, seed=3)
    lengths = {i: r for i, r in enumerate(reqs)}
    rr = sharding.Dispatcher(range(4), "round_robin")
    assert [rr.assign(i, *r) for i, r in enumerate(reqs)] == [i % 4 for i in range(64)]
    ll = sharding.Dispatcher(range(4), "least_loaded")
    for i, r in enumerate(reqs):
        ll.assign(i, *r)
    loads = [ll.load(r) for r in range(4)]
    assert max(loads) - min(loads) <= max(p + o for p, o in reqs), "least-loaded keeps replicas within one request"
    # replica 2 finishes three requests, then leaves between steps: the rest of its share is dealt again
    mine = sorted(ll.outstanding[2])
    for rid in mine[:3]:
        ll.complete(2, rid, result=("tokens of", rid))
    moved = ll.replica_left(2, lengths)
    assert sorted(moved) == mine[3:] and set(moved.values()) <= {0, 1, 3}
    for r in (0, 1, 3):
        for rid in sorted(ll.outstanding[r]):
            ll.complete(r, rid, result=("tokens of", rid))
    assert [res[1] for res in ll.merged_results()] == list(range(64))
    import pytest
    with pytest.raises(ValueError):
        ll.complete(0, 5)
    arr = sharding.poisson_arrivals(1000, rate_per_s=4.0)
    assert all(b >= a for a, b in zip(arr, arr[1:])) and 200 < arr[-1] < 300


def _leaver_worker(rank, world, port, out_dir):
    """Three replicas serve a dealt trace in host-side 'steps'; replica 2 leaves after its third step. The others
    learn of it from the store before their next step (no collective involves the leaver afterwards), take over its
    unfinished requests by the dispatcher's rule, and every request is served exactly once."""
    import json
    from datetime import timedelta
    import __graft_entry__ as entry
    entry.load_package()
    from q38b200 import sharding
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=60))
    reqs = sharding.trace_requests(30, seed=5)
    lengths = {i: r for i, r in enumerate(reqs)}
    d = sharding.Dispatcher(range(world), "round_robin")  # every replica keeps the same books
    for i, r in enumerate(reqs):
        d.assign(i, *r)
    served, step, known_left = [], 0, False
    while True:
        if not known_left and store.check(["left/2"]):  # the heartbeat read before every step
            unfinished = json.loads(store.get("left/2"))
            for rid in sorted(set(d.outstanding[2]) - set(unfinished)):
                d.complete(2, rid)
            d.replica_left(2, lengths)
            known_left = True
        if rank == 2 and step == 3:
            store.set("left/2", json.dumps(sorted(d.outstanding[2])))
            break
        todo = sorted(d.outstanding[rank]) if rank in d.outstanding else []
        if not todo:
            if rank == 2 or known_left:
                break
            time.sleep(0.01)  # replicas 0 and 1 stay until the leaver's share has been dealt
            continue
        rid = todo[0]
        d.complete(rank, rid)
        served.append(rid)
        store.add(f"served/{rid}", 1)
        step += 1
    store.set(f"done/{rank}", json.dumps(served))
    if rank == 0:
        store.wait([f"done/{r}" for r in range(world)])
        counts = [int(store.add(f"served/{i}", 0)) for i in range(30)]
        assert counts == [1] * 30, counts
        assert len(json.loads(store.get("done/2"))) == 3
        (Path(out_dir) / "ok").write_text("ok")
        store.set("finished", "1")
    else:
        store.wait(["finished"])  # keep the store's clients alive until the master has read everything


def test_a_replica_leaves_between_steps_and_its_requests_are_dealt_again(tmp_path):
    world, port = 3, 31000 + os.getpid() % 2000
    mp.spawn(_leaver_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ok").exists()
