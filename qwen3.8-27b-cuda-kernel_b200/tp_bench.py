"""Benchmark of the tensor-parallel path: one request with a very long context (default 262,144 tokens, lean recipe,
27B geometry) over all ranks of the job.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \\
      qwen3.8-27b-cuda-kernel_b200/tp_bench.py --context 262144

Weights are random BQ planes of the real geometry (written once to shared memory by rank 0); every rank uploads only
its shard. The first `--real-prefill` tokens of the context are really prefilled (512-token steps, timed; -1 = all of
it, optionally within `--prefill-budget-s` seconds); what is not prefilled is filled with random int8 rows and finite
scales. Then `--steps` decode steps (one CUDA graph per step) are timed with CUDA events, max over ranks, twice: with
the all-reduce inside the row-parallel GEMM over peer memory, and with NCCL all-reduces between the GEMM and the
residual update; one 512-token prefill step at the end of the context is timed as well. Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import time
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _package():
    name = "q38b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, HERE / "__init__.py", submodule_search_locations=[str(HERE)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measure(pkg, dist, rank: int, world: int, context: int = 262144, real_prefill: int = 2048, layers: int = 64,
            recipe: str = "lean", steps: int = 20, warmup: int = 3, prefill_budget_s: float = 0.0) -> dict:
    """Builds the sharded runner on an initialised process group (or none) and times it; every rank returns the same
    dictionary. `real_prefill` < 0: the whole context is really prefilled, as far as `prefill_budget_s` seconds of
    device time allow (0 = no limit); what is left is filled with random rows like before."""
    from q38b200 import synth, tp

    shm = Path("/dev/shm") if Path("/dev/shm").is_dir() else Path("/tmp")
    path = shm / f"q38_tp_27b_{recipe}_L{layers}.q38"
    if rank == 0 and not path.exists():
        types = None
        if layers != 64:
            types = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(layers)]
        cfg = synth.model_config(**{**synth.CONFIG_27B, "layers": layers, "layer_types": types})
        t0 = time.time()
        synth.write_random_planes_q38(path, cfg, recipe=recipe, seed=11)
        print(f"tp_bench: model planes written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    if dist is not None:
        dist.barrier()
    t0 = time.time()
    runner = tp.TPRunner(pkg, path, rank, world, dist, max_tokens=512, max_context=context + 64, fused_allreduce=True)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"tp_bench: shards uploaded in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)

    rng = np.random.default_rng(3)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn):
        e0, e1 = ev(), ev()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0])

    # ---- real prefill: the head of the context, or all of it within the time budget ----
    whole = real_prefill < 0
    want = (context - 1024 if whole else min(real_prefill, context - 1024)) // 512 * 512
    pre_ms, real, short_ms, short_tokens, last_step_ms = 0.0, 0, 0.0, 0, 0.0
    for p0 in range(0, want, 512):
        toks = rng.integers(1000, 150000, size=512)
        last_step_ms = timed(lambda: runner.forward(toks, p0))
        pre_ms += last_step_ms
        real = p0 + 512
        if real <= 2048:
            short_ms, short_tokens = pre_ms, real
        if prefill_budget_s > 0 and pre_ms > 1000.0 * prefill_budget_s:  # the max over ranks: every rank stops here
            break
    # ---- the rest of the KV cache: random int8 rows, finite fp16 scales ----
    kvp = runner.kv_pool
    first_fake_page = real // 64
    per_layer = runner.pages * runner.page_bytes
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    if first_fake_page < runner.pages:
        for layer in range(max(1, sum(1 for L in runner.layers if L["attention"]))):
            a = layer * per_layer + first_fake_page * runner.page_bytes
            b = (layer + 1) * per_layer
            view = kvp[a:b]
            view.copy_(torch.randint(0, 256, (b - a,), dtype=torch.uint8, device="cuda", generator=g))
            view.view(torch.int16).bitwise_and_(0x2BFF)  # as fp16: positive, below 0.06 (int8 rows are unaffected in kind)
    torch.cuda.synchronize()

    # ---- one prefill step at the far end of the context ----
    far0 = context - 1024
    toks = rng.integers(1000, 150000, size=512)
    far_ms = timed(lambda: runner.forward(toks, far0))

    # ---- decode: the all-reduce inside the GEMM over peer memory, then NCCL all-reduce + residual update ----
    tok = 12345
    dec = {}
    for mode, fused in (("fused", True), ("nccl", False)):
        runner.use_fused = fused
        runner._graph = None
        state = {"pos": context - 512 + (0 if fused else 128)}
        for _ in range(max(warmup, 2)):
            runner.decode_replay(tok, state["pos"])
            state["pos"] += 1

        def run_steps():
            for _ in range(steps):
                runner.decode_replay(tok, state["pos"])
                state["pos"] += 1
        dec[mode] = timed(run_steps) / steps
    logits = runner.logits()
    err = runner.device_error()
    line = {
        "metric": "tp_decode_tok_per_s", "value": 1000.0 / dec["fused"], "unit": "tok/s", "n_gpus": world, "steps": steps,
        "ms_per_step": dec["fused"], "ms_per_step_nccl_allreduce": dec["nccl"], "context_tokens": context,
        "recipe": recipe, "layers": layers, "all_reduces_per_step": 2 * layers,
        "allreduce": "inside the row-parallel GEMM (peer stores, per-tile flags, sum in rank order)",
        "prefill_tok_per_s_short_context": (short_tokens / short_ms * 1000.0) if short_ms > 0 else None,
        "prefill_tokens_really_run": real, "prefill_total_s": pre_ms / 1000.0,
        "prefill_last_real_step_ms": last_step_ms, "prefill_512_at_context_end_ms": far_ms,
        "kv": (f"first {real} tokens really prefilled" + ("" if real >= want and whole else ", the rest random int8 rows")),
        "logits_finite": bool(np.isfinite(logits).all()), "device_error": err, "data": "synthetic",
    }
    runner.close()
    return line


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--context", type=int, default=262144)
    ap.add_argument("--real-prefill", type=int, default=2048, help="tokens really prefilled; -1 = the whole context")
    ap.add_argument("--prefill-budget-s", type=float, default=0.0, help="stop the real prefill after this much device time")
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--recipe", default="lean")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # NCCL prints its version banner on stdout when the first communicator comes up: stdout is pointed at stderr
        # until then, so that the JSON line stays the only thing on stdout
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    pkg = _package()
    line = measure(pkg, dist, rank, world, args.context, args.real_prefill, args.layers, args.recipe, args.steps,
                   args.warmup, args.prefill_budget_s)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
