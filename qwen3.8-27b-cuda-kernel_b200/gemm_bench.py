"""Per-shape micro-benchmark and tile-configuration sweep of the BQ GEMM (q38_qgemm).

The kernel-level counterpart of the reference bench app's GEMM sweep (src/apps/bench.cpp:134-194): for each
(bits, n, k) of the 27B geometry and each token count m it times every tile configuration that accepts m,
prints weight GB/s and TFLOP/s, and with --save writes the winners as a tuning table in the JSON layout
load_tuning() reads (src/tuning.cpp:24-70).

Planes are random bytes (timing does not depend on the values); each shape is held in several copies whose
total size exceeds L2, and successive launches rotate over them, so every launch streams its weights from HBM.
Launches are captured into one CUDA graph per measurement and timed with CUDA events around the replay.

  python qwen3.8-27b-cuda-kernel_b200/gemm_bench.py --m 1,8,16,64                # auto-selected config per m
  python qwen3.8-27b-cuda-kernel_b200/gemm_bench.py --sweep --save tuning.json   # all configs, keep the best
  python qwen3.8-27b-cuda-kernel_b200/gemm_bench.py --single 69632,5120,4 --m 8 --launches 3
      # a few plain launches of one shape and nothing else: the small case to put under a profiler
"""

from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import json
import sys
from pathlib import Path

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


# (n, k, bits, name): the GEMMs of one decode step of the 27B geometry under the default recipe
SHAPES_27B = [
    (34816, 5120, 4, "mlp_gate_up"),
    (5120, 17408, 5, "mlp_down"),
    (16384, 5120, 5, "gdn_qkvz"),
    (5120, 6144, 5, "gdn_out"),
    (14336, 5120, 5, "attn_qkvg"),
    (5120, 6144, 5, "attn_o"),
    (248320, 5120, 8, "lm_head"),
]

L2_BYTES = 126 << 20


def plane_bytes(n: int, k: int, bits: int):
    slabs = (n // 64) * (k // 16)
    hi_per_slab = {4: 0, 5: 128, 6: 256, 8: 512}[bits]
    return slabs * 512, slabs * hi_per_slab, (n // 64) * (k // 64) * 128


class Planes:
    def __init__(self, pkg, n, k, bits):
        lo_b, hi_b, sc_b = plane_bytes(n, k, bits)
        self.lo = torch.randint(0, 256, (lo_b,), dtype=torch.uint8, device="cuda")
        self.hi = torch.randint(0, 256, (hi_b,), dtype=torch.uint8, device="cuda") if hi_b else None
        self.sc = (torch.rand(sc_b // 2, device="cuda") * 0.01 + 0.001).to(torch.bfloat16)
        self.desc = pkg.BQWeight(pkg.ptr(self.lo), pkg.ptr(self.hi), pkg.ptr(self.sc), bits, n, k, n)
        self.bytes = lo_b + hi_b + sc_b


class Workspace:
    def __init__(self, pkg, tokens_per_pass=512):
        sms = pkg.kernels().q38_num_sms()
        self.partials = torch.empty(2 * sms * 128 * tokens_per_pass, dtype=torch.float32, device="cuda")
        self.counters = torch.zeros(8192, dtype=torch.int32, device="cuda")
        self.desc = pkg.GemmWorkspace(pkg.ptr(self.partials), self.partials.numel(), pkg.ptr(self.counters),
                                      self.counters.numel())


def make_epilogue(pkg, kind, m, n):
    """The epilogue descriptor of one of the step's three GEMM kinds plus the tensors it points to."""
    if kind == "residual":  # out-projections and down: residual += C, bf16 copy, partial sums of squares per 128 columns
        res = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        xbf = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        part = torch.empty((m, n // 128), dtype=torch.float32, device="cuda")
        return pkg.GemmEpilogue(pkg.EPI_RESIDUAL, None, 0, 0, pkg.ptr(res), pkg.ptr(xbf), pkg.ptr(part), None, 0, 1e-6), (res, xbf, part)
    if kind == "swiglu":    # gate/up: silu(gate) * up on interleaved column pairs
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        return pkg.GemmEpilogue(pkg.EPI_SWIGLU, pkg.ptr(out), n // 2, 0, None, None, None, None, 0, 1e-6), (out,)
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    return pkg.GemmEpilogue(pkg.EPI_STORE_BF16, pkg.ptr(out), n, 0, None, None, None, None, 0, 1e-6), (out,)


def time_gemm(pkg, copies, ws, m, config, iters=20, epilogue="store"):
    K = pkg.kernels()
    w0 = copies[0].desc
    a = torch.randn((m, w0.k), device="cuda").to(torch.bfloat16)
    ep, keep = make_epilogue(pkg, epilogue, m, w0.n)
    st = torch.cuda.Stream()

    def launch(i):
        pkg.check(K.q38_qgemm(pkg.ptr(a), m, C.byref(copies[i % len(copies)].desc), C.byref(ep), C.byref(ws.desc),
                              st.cuda_stream, config))

    with torch.cuda.stream(st):
        for i in range(4):
            launch(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=st):
        for i in range(iters):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3  # microseconds per launch


def configs_for(pkg, bits):
    """Every tile configuration built for this bit width (the 512-token pass does not exist for 8-bit weights)."""
    K = pkg.kernels()
    return [c for c in range(K.q38_qgemm_num_configs()) if not (bits == 8 and K.q38_qgemm_config_name(c) == b"umma_t512")]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--m", default="1,8,16,32,64,128,256,512", help="comma-separated token counts")
    ap.add_argument("--shapes", default="", help="comma-separated shape names (default: all of the 27B geometry)")
    ap.add_argument("--config", type=int, default=-1, help="tile configuration id (-1: the dispatcher's choice)")
    ap.add_argument("--sweep", action="store_true", help="time every configuration and report the best")
    ap.add_argument("--save", default="", help="with --sweep: write the winners as a tuning table (JSON)")
    ap.add_argument("--single", default="", help="n,k,bits: launch only this shape, --launches times, untimed")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="HBM peak to print fractions of (GB/s)")
    ap.add_argument("--epilogue", default="store", choices=["store", "residual", "swiglu", "step"],
                    help="epilogue kind; 'step' = the kind each shape has in the model's step")
    args = ap.parse_args(argv)

    if not torch.cuda.is_available():
        raise SystemExit("gemm_bench needs a CUDA device")
    pkg = _package()
    K = pkg.kernels()
    ms = [int(x) for x in args.m.split(",") if x]
    ws = Workspace(pkg)

    if args.single:
        n, k, bits = (int(x) for x in args.single.split(","))
        w = Planes(pkg, n, k, bits)
        m = ms[0]
        a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ep = pkg.GemmEpilogue(pkg.EPI_STORE_BF16, pkg.ptr(out), n, 0, None, None, None, None, 0, 1e-6)
        for _ in range(args.launches):
            pkg.check(K.q38_qgemm(pkg.ptr(a), m, C.byref(w.desc), C.byref(ep), C.byref(ws.desc), None, args.config))
        torch.cuda.synchronize()
        if K.q38_device_error(1):
            raise SystemExit("device-side wait gave up")
        print(f"ok: {args.launches} launches, m={m}, {w.bytes} weight bytes per launch")
        return 0

    wanted = set(args.shapes.split(",")) if args.shapes else None
    entries = []
    for n, k, bits, name in SHAPES_27B:
        if wanted and name not in wanted:
            continue
        one = sum(plane_bytes(n, k, bits))
        copies = [Planes(pkg, n, k, bits) for _ in range(max(2, -(-2 * L2_BYTES // one)))]
        kind = args.epilogue
        if kind == "step":
            kind = {"mlp_gate_up": "swiglu", "mlp_down": "residual", "gdn_out": "residual", "attn_o": "residual"}.get(name, "store")
        for m in ms:
            cands = configs_for(pkg, bits) if args.sweep else [args.config]
            best = None
            for c in cands:
                us = time_gemm(pkg, copies, ws, m, c, epilogue=kind)
                if best is None or us < best[1]:
                    best = (c, us)
            c, us = best
            cname = K.q38_qgemm_config_name(c if c >= 0 else K.q38_qgemm_auto_config(bits, n, k, m)).decode()
            gbs = one / us / 1e3
            frac = f"  {100 * gbs / args.peak_gbs:5.1f}% of peak" if args.peak_gbs else ""
            print(f"{name:12s} bq{bits} n={n:6d} k={k:6d} m={m:4d} -> {cname:10s} {us:9.1f} us {gbs:7.0f} GB/s{frac}"
                  f" {2.0 * m * n * k / us / 1e6:7.1f} TFLOP/s", flush=True)
            entries.append({"bits": bits, "n": n, "k": k, "m_max": m, "config": c, "us": round(us, 2)})
        del copies
        torch.cuda.empty_cache()
    if K.q38_device_error(1):
        raise SystemExit("device-side wait gave up")
    if args.save:
        if not args.sweep:
            raise SystemExit("--save needs --sweep")
        Path(args.save).write_text(json.dumps({"device": torch.cuda.get_device_name(0), "entries": entries}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
