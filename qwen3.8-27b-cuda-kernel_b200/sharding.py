"""Request sharding over engine replicas (one replica per GPU, no collective on the data path).

The model fits one B200, so N GPUs run N independent engines and a request is served entirely by one of them.
Requests are dealt round-robin in arrival order (request i -> replica i mod N), which keeps the replicas'
loads within one request of each other for any arrival pattern. The only cross-rank traffic of a benchmark run
is the barrier around the timed region and the max-over-ranks of the measured times; both work on any
torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import math

import numpy as np


def trace_requests(num_requests: int = 512, seed: int = 11):
    """The synthetic continuous-batching trace: prompt lengths log-uniform in [64, 8192], output lengths uniform in
    [64, 1024], as (prompt_len, output_len) pairs in arrival order."""
    rng = np.random.default_rng(seed)
    prompts = np.rint(np.exp(rng.uniform(math.log(64), math.log(8192), size=num_requests))).astype(int)
    outputs = rng.integers(64, 1025, size=num_requests)
    return [(int(p), int(o)) for p, o in zip(prompts, outputs)]


def shard_requests(requests, rank: int, world: int):
    """The requests replica `rank` of `world` serves, as (global index, request) pairs."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return [(i, r) for i, r in enumerate(requests) if i % world == rank]


def max_over_ranks(values, dist=None, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a process group)."""
    import torch
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def whole_job_rate(units_per_rank: int, world: int, seconds_max_over_ranks: float) -> float:
    """Aggregate throughput of a weak-scaling run: every rank processed `units_per_rank` units, the job took the
    slowest rank's time."""
    return units_per_rank * world / seconds_max_over_ranks


def poisson_arrivals(num_requests: int, rate_per_s: float, seed: int = 11):
    """Arrival times (seconds from the start of the trace) of a Poisson process of `rate_per_s` requests per second."""
    rng = np.random.default_rng(seed + 7919)
    return np.cumsum(rng.exponential(1.0 / rate_per_s, size=num_requests)).tolist()


class Dispatcher:
    """The host driver of a request-sharded job: hands every arriving request to one replica and keeps the books.

    policy "round_robin": request i of the arrival order goes to replica i mod N (what `shard_requests` computes);
    policy "least_loaded": to the replica with the fewest outstanding tokens (prompt + requested output), lowest rank
    first among equals. Replicas report completions; a replica that leaves hands its unfinished requests back, and
    they are dealt again over the remaining replicas by the same policy. Pure bookkeeping: no GPU, no collective.
    """

    def __init__(self, replicas, policy: str = "round_robin"):
        if policy not in ("round_robin", "least_loaded"):
            raise ValueError(f"unknown policy {policy!r}")
        self.policy = policy
        self.alive = sorted(replicas)
        if not self.alive:
            raise ValueError("no replicas")
        self.outstanding = {r: {} for r in self.alive}  # replica -> {request id: tokens}
        self.done = {}                                  # request id -> (replica, result)
        self._next = 0

    def load(self, replica: int) -> int:
        return sum(self.outstanding[replica].values())

    def assign(self, request_id: int, prompt_len: int, output_len: int) -> int:
        if self.policy == "round_robin":
            replica = self.alive[self._next % len(self.alive)]
            self._next += 1
        else:
            replica = min(self.alive, key=lambda r: (self.load(r), r))
        self.outstanding[replica][request_id] = prompt_len + output_len
        return replica

    def complete(self, replica: int, request_id: int, result=None) -> None:
        if request_id in self.done:
            raise ValueError(f"request {request_id} finished twice")
        self.outstanding[replica].pop(request_id)
        self.done[request_id] = (replica, result)

    def replica_left(self, replica: int, lengths):
        """`replica` is gone (between steps): its unfinished requests are dealt again. `lengths[id]` = (prompt, output).
        Returns {request id: new replica}."""
        if replica not in self.alive:
            raise ValueError(f"replica {replica} is not part of the job")
        orphans = sorted(self.outstanding.pop(replica))
        self.alive.remove(replica)
        if not self.alive:
            raise RuntimeError("the last replica left with requests outstanding" if orphans else "no replicas left")
        return {rid: self.assign(rid, *lengths[rid]) for rid in orphans}

    def merged_results(self):
        """Results in request-id order, once every request has finished."""
        if any(self.outstanding[r] for r in self.alive):
            raise RuntimeError("requests still outstanding")
        return [self.done[i][1] for i in sorted(self.done)]
