"""q38-bench: throughput sweeps, per-op profile and GEMM autotuning on a model file.

The counterpart of the reference's bench app (src/apps/bench.cpp:70-194, options `--decode`, `--context`, `--gen`,
`--prefill`, `--profile`, `--tune`, `--json`) over this engine's ModelRunner:

    python qwen3.8-27b-cuda-kernel_b200/q38_bench.py --model M.q38                    decode (B = 1,2,4,8,16) + prefill sweep
    python qwen3.8-27b-cuda-kernel_b200/q38_bench.py --model M.q38 --decode 1,8,64 --context 4096 --gen 64
    python qwen3.8-27b-cuda-kernel_b200/q38_bench.py --model M.q38 --profile          per-op GPU time of decode and prefill steps
    python qwen3.8-27b-cuda-kernel_b200/q38_bench.py --model M.q38 --tune tuning.json sweep GEMM tile configurations, write a tuning table
    python qwen3.8-27b-cuda-kernel_b200/q38_bench.py --synthetic 27b --layers 8       no model file: random planes of the 27B geometry

Decode: `batch` sequences are prefilled to `context` tokens of ordinary-text ids (1000..150000, as the reference
draws them), then `gen` greedy decode steps run through ModelRunner::decode (CUDA graph per batch bucket); the step
time is the device time of the step (CUDA events inside the runner) and the wall time of the call. Prefill: one
sequence, chunked; tokens per second of device time. `--json` writes everything machine-readable.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

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


def ints(text: str) -> list[int]:
    return [int(x) for x in text.split(",") if x]


def random_tokens(rng, n: int, vocab: int) -> np.ndarray:
    return rng.integers(1000, min(vocab, 150000), size=n).astype(np.int32)


def prefill_all(runner, slot: int, tokens: np.ndarray, chunk: int, sampling) -> tuple[int, float]:
    """Chunked prefill of one sequence; returns (first sampled token, device milliseconds)."""
    first, ms = 0, 0.0
    for off in range(0, len(tokens), chunk):
        part = tokens[off:off + chunk]
        last = off + len(part) == len(tokens)
        toks, _ = runner.prefill([(slot, off, part, sampling if last else None, 0)])
        ms += runner.last_step_ms()
        if last:
            first = int(toks[0])
    return first, ms


def bench_decode(eng, runner, model, batch: int, context: int, gen: int, chunk: int, rng) -> dict:
    g = eng.greedy()
    nxt = []
    for s in range(batch):
        runner.reset_slot(s)
        if not runner.kv_ensure(s, context + gen + 1):
            raise SystemExit(f"KV cache too small for batch {batch} x context {context}")
        nxt.append(prefill_all(runner, s, random_tokens(rng, context, model.vocab), chunk, g)[0])
    dev_ms, t0 = 0.0, None
    for step in range(gen + 2):
        if step == 2:  # two warm-up steps (graph capture happens in the first)
            t0 = time.perf_counter()
            dev_ms = 0.0
        toks, _ = runner.decode([(s, context + step, nxt[s], g, step + 1) for s in range(batch)])
        dev_ms += runner.last_step_ms()
        nxt = [int(t) for t in toks]
    wall = time.perf_counter() - t0
    for s in range(batch):
        runner.kv_release(s)
    return {"batch": batch, "context": context, "steps": gen, "device_ms_per_step": dev_ms / gen,
            "wall_ms_per_step": 1000.0 * wall / gen, "tok_per_s": batch * gen / wall}


def bench_prefill(eng, runner, model, length: int, chunk: int, rng) -> dict:
    runner.reset_slot(0)
    if not runner.kv_ensure(0, length + 1):
        raise SystemExit(f"KV cache too small for a prompt of {length}")
    t0 = time.perf_counter()
    _, ms = prefill_all(runner, 0, random_tokens(rng, length, model.vocab), chunk, eng.greedy())
    wall = time.perf_counter() - t0
    runner.kv_release(0)
    return {"prompt": length, "chunk": chunk, "device_ms": ms, "wall_ms": 1000.0 * wall, "tok_per_s": length / (ms / 1000.0)}


def profile_steps(eng, runner, model, batch: int, context: int, chunk: int, rng) -> dict:
    """Per-op device time of one decode step of `batch` sequences and of one full prefill chunk (eager, CUDA events
    between the kernels)."""
    g = eng.greedy()
    nxt = []
    for s in range(batch):
        runner.reset_slot(s)
        assert runner.kv_ensure(s, context + chunk + 8)
        nxt.append(prefill_all(runner, s, random_tokens(rng, context, model.vocab), chunk, g)[0])
    runner.set_profiling(True)
    runner.profile(clear=True)
    for step in range(3):
        toks, _ = runner.decode([(s, context + step, nxt[s], g, step + 1) for s in range(batch)])
        nxt = [int(t) for t in toks]
    decode = {k: round(v[0] / 3, 4) for k, v in runner.profile(clear=True).items() if k != "start"}
    runner.prefill([(0, context + 3, random_tokens(rng, chunk, model.vocab), None, 0)])
    prefill = {k: round(v[0], 4) for k, v in runner.profile(clear=True).items() if k != "start"}
    runner.set_profiling(False)
    for s in range(batch):
        runner.kv_release(s)
    return {"decode_batch": batch, "context": context, "decode_ms_per_op": decode, "prefill_chunk": chunk,
            "prefill_ms_per_op": prefill}


def print_ops(title: str, ops: dict) -> None:
    total = sum(ops.values())
    print(f"{title}: {total:.3f} ms")
    for name, ms in sorted(ops.items(), key=lambda kv: -kv[1]):
        print(f"    {name:24s} {ms:9.3f} ms  {100.0 * ms / max(total, 1e-9):5.1f} %")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="", help="a .q38 model file")
    ap.add_argument("--synthetic", default="", choices=["", "27b"], help="no file: random BQ planes of this geometry")
    ap.add_argument("--layers", type=int, default=64, help="--synthetic: number of layers")
    ap.add_argument("--recipe", default="default")
    ap.add_argument("--decode", default="1,2,4,8,16", help="decode batch sizes")
    ap.add_argument("--context", default="512", help="context length(s) of the decode sweep")
    ap.add_argument("--gen", type=int, default=32, help="decode steps per measurement")
    ap.add_argument("--prefill", default="512,2048,8192", help="prompt lengths of the prefill sweep ('' = skip)")
    ap.add_argument("--chunk", type=int, default=512, help="prefill chunk")
    ap.add_argument("--kv", default="int8", choices=["int8", "bf16"])
    ap.add_argument("--profile", action="store_true", help="per-op GPU time of a decode and a prefill step")
    ap.add_argument("--tune", default="", metavar="FILE", help="sweep the GEMM tile configurations of the 27B shapes and write a tuning table")
    ap.add_argument("--tuning", default="", metavar="FILE", help="install a tuning table before measuring")
    ap.add_argument("--json", default="", metavar="FILE")
    args = ap.parse_args(argv)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("q38-bench needs a CUDA device")
    pkg = _package()
    from q38b200 import engine as eng
    results: dict = {"device": torch.cuda.get_device_name(0)}

    if args.tune:
        import gemm_bench  # beside this file
        gemm_bench.main(["--sweep", "--save", args.tune, "--epilogue", "step"])
        results["tuning_table"] = args.tune
        if not args.model and not args.synthetic:
            return 0
    if args.tuning:
        eng.load_tuning(args.tuning)

    path = Path(args.model) if args.model else None
    if path is None:
        if not args.synthetic:
            raise SystemExit("give --model FILE or --synthetic 27b")
        from q38b200 import synth
        cfg = synth.model_config(**{**synth.CONFIG_27B, "layers": args.layers})
        path = Path(tempfile.gettempdir()) / f"q38_bench_synth_{args.recipe}_L{args.layers}.q38"
        if not path.exists():
            synth.write_random_planes_q38(path, cfg, recipe=args.recipe)
    model = eng.Model(path)
    print(model.summary())
    batches, contexts = ints(args.decode), ints(args.context)
    prompts = ints(args.prefill)
    need = max([0] + contexts) + args.gen + args.chunk + 64
    max_batch = max(batches + [1])
    kv_tokens = max(max_batch * (need + 64), max(prompts + [0]) + 128)
    runner = eng.Runner(model, eng.default_runner_options(max_batch=max_batch, prefill_chunk=args.chunk,
                                                          kv_dtype=0 if args.kv == "int8" else 1, kv_tokens=kv_tokens,
                                                          max_context=max(need, max(prompts + [0]) + 64), verbose=0))
    rng = np.random.default_rng(42)
    results["memory"] = runner.memory()
    if args.profile:
        prof = profile_steps(eng, runner, model, max_batch, contexts[0], args.chunk, rng)
        results["profile"] = prof
        print_ops(f"decode step, batch {prof['decode_batch']}, context {prof['context']}", prof["decode_ms_per_op"])
        print_ops(f"prefill step, {prof['prefill_chunk']} tokens", prof["prefill_ms_per_op"])
    else:
        results["decode"] = []
        for ctx in contexts:
            for b in batches:
                r = bench_decode(eng, runner, model, b, ctx, args.gen, args.chunk, rng)
                results["decode"].append(r)
                print(f"decode  batch {b:4d} context {ctx:6d}: {r['device_ms_per_step']:8.3f} ms/step device, "
                      f"{r['wall_ms_per_step']:8.3f} ms/step wall, {r['tok_per_s']:9.1f} tok/s")
        results["prefill"] = []
        for n in prompts:
            r = bench_prefill(eng, runner, model, n, args.chunk, rng)
            results["prefill"].append(r)
            print(f"prefill prompt {n:6d} (chunk {args.chunk}): {r['device_ms']:9.2f} ms device, {r['tok_per_s']:9.1f} tok/s")
    if pkg.kernels().q38_device_error(1):
        raise SystemExit("a device-side wait gave up during the run")
    runner.close()
    model.close()
    if args.json:
        Path(args.json).write_text(json.dumps(results, indent=1))
    return 0


if __name__ == "__main__":
    sys.path.insert(0, str(HERE))
    sys.exit(main())
