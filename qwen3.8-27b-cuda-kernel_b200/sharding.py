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
