"""Micro-benchmark of the state-streaming decode kernels and of the prefill attention at the 27B geometry: paged int8 decode attention
(24 q heads / 4 kv heads, head_dim 256, 64-token pages in a shuffled page table, contexts log-uniform in
128..32768) and the Gated DeltaNet decode recurrence (48 value heads / 16 key heads, 128x128 fp32 state).

The KV pages hold random bytes with random fp16 scales and the recurrent states random floats: the timing does not
depend on the values. Each measurement is a CUDA graph of `--iters` launches timed with CUDA events; the
working set of either kernel is far larger than L2.

  python qwen3.8-27b-cuda-kernel_b200/op_bench.py                       # both kernels, 64 sequences
  python qwen3.8-27b-cuda-kernel_b200/op_bench.py --op attn --seqs 16 --launches 3 --untimed
      # a few plain launches and nothing else: the small case to put under a profiler
  python qwen3.8-27b-cuda-kernel_b200/op_bench.py --op prefill --prefix 2048,32768,131072
      # the query-tiled prefill attention: one 512-token chunk behind a cached prefix, for the 27B layer (24 q / 4 kv
      # heads) and for one rank of the 8-way tensor-parallel layout (3 q / 1 kv head, keys cut over several CTAs)
  python qwen3.8-27b-cuda-kernel_b200/op_bench.py --op scan --chunk 512
      # the chunked Gated DeltaNet recurrence over one prefill step (per-chunk preparation + state scan), with the scan's
      # products on the tensor cores (split TF32) and as fp32 FMAs
"""

from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
NQ, NKV, HD, PAGE = 24, 4, 256, 64
NK, NV = 16, 48


def _package():
    name = "q38b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, HERE / "__init__.py", submodule_search_locations=[str(HERE)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def batch_desc(pkg, seqs, pos0):
    """One new token per sequence; slot b = sequence b."""
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    t = {"seq_start": mk(list(range(seqs + 1))), "seq_slot": mk(list(range(seqs))), "seq_pos0": mk(pos0),
         "tok_pos": mk(pos0), "tok_seq": mk(list(range(seqs)))}
    desc = pkg.BatchDesc(seqs, seqs, 1, pkg.ptr(t["seq_start"]), pkg.ptr(t["seq_slot"]), pkg.ptr(t["seq_pos0"]),
                         pkg.ptr(t["tok_pos"]), pkg.ptr(t["tok_seq"]))
    return desc, t


def timed_graph(launch, iters):
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            launch(st.cuda_stream)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        for _ in range(iters):
            launch(st.cuda_stream)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def attn_case(pkg, seqs, seed):
    K = pkg.kernels()
    rng = np.random.default_rng(seed)
    ctx = np.exp(rng.uniform(np.log(128), np.log(32768), size=seqs)).astype(np.int64)
    pages_per_seq = [int((c + 1 + PAGE - 1) // PAGE) for c in ctx]
    num_pages = sum(pages_per_seq) + 1
    page_bytes = int(K.q38_kv_page_bytes(pkg.KV_INT8, NKV))
    pool = torch.randint(0, 256, (num_pages * page_bytes,), dtype=torch.uint8, device="cuda")
    # the scale rows must be finite fp16 numbers: overwrite every 16-bit word pattern's exponent via a mask
    pool.view(torch.int16).bitwise_and_(0x3BFF)
    max_pages = max(pages_per_seq)
    table = np.zeros((seqs, max_pages), dtype=np.int32)
    perm = rng.permutation(num_pages - 1) + 1
    at = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[at:at + n]
        at += n
    table_d = torch.from_numpy(table).cuda()
    kv = pkg.KvCacheDesc(pkg.ptr(pool), pkg.KV_INT8, NKV, num_pages, page_bytes, num_pages * page_bytes,
                         pkg.ptr(table_d), max_pages)
    desc, keep = batch_desc(pkg, seqs, [int(c) for c in ctx])
    q = torch.randn((seqs, NQ, HD), device="cuda").to(torch.float16)
    gate = torch.randn((seqs, NQ * HD), device="cuda").to(torch.bfloat16)
    out = torch.empty((seqs, NQ * HD), dtype=torch.bfloat16, device="cuda")
    splits = 64
    scratch = torch.empty(seqs * NQ * splits * (HD + 2), dtype=torch.float32, device="cuda")
    ap = pkg.AttentionParams(pkg.ptr(q), pkg.ptr(gate), NQ * HD, pkg.ptr(out), NQ, NKV, 0, pkg.ptr(scratch), splits)
    kv_bytes = int(sum(int(c) + 1 for c in ctx)) * NKV * (2 * HD + 16)

    def launch(stream):
        pkg.check(K.q38_attention_decode(C.byref(ap), C.byref(desc), C.byref(kv), stream))
    return launch, kv_bytes, (pool, table_d, keep, q, gate, out, scratch), f"{seqs} sequences, {int(ctx.sum())} context tokens"


def prefill_case(pkg, prefix, chunk, seed, nq=NQ, nkv=NKV, split_rows=0):
    """One sequence: a `chunk`-token prefill step behind `prefix` cached tokens (random int8 pages)."""
    K = pkg.kernels()
    rng = np.random.default_rng(seed)
    total = prefix + chunk
    pages = (total + PAGE - 1) // PAGE
    page_bytes = int(K.q38_kv_page_bytes(pkg.KV_INT8, nkv))
    pool = torch.randint(0, 256, ((pages + 1) * page_bytes,), dtype=torch.uint8, device="cuda")
    pool.view(torch.int16).bitwise_and_(0x3BFF)
    table_d = torch.from_numpy((rng.permutation(pages) + 1).astype(np.int32)[None, :]).cuda()
    kv = pkg.KvCacheDesc(pkg.ptr(pool), pkg.KV_INT8, nkv, pages + 1, page_bytes, (pages + 1) * page_bytes,
                         pkg.ptr(table_d), pages)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    t = {"seq_start": mk([0, chunk]), "seq_slot": mk([0]), "seq_pos0": mk([prefix]),
         "tok_pos": mk(list(range(prefix, total))), "tok_seq": mk([0] * chunk)}
    desc = pkg.BatchDesc(1, chunk, chunk, pkg.ptr(t["seq_start"]), pkg.ptr(t["seq_slot"]), pkg.ptr(t["seq_pos0"]),
                         pkg.ptr(t["tok_pos"]), pkg.ptr(t["tok_seq"]))
    q = torch.randn((chunk, nq, HD), device="cuda").to(torch.float16)
    gate = torch.randn((chunk, nq * HD), device="cuda").to(torch.bfloat16)
    out = torch.empty((chunk, nq * HD), dtype=torch.bfloat16, device="cuda")
    max_splits = 16
    rows = max(split_rows, 1)
    scratch = torch.empty(rows * nq * max_splits * (HD + 2), dtype=torch.float32, device="cuda")
    ap = pkg.AttentionParams(pkg.ptr(q), pkg.ptr(gate), nq * HD, pkg.ptr(out), nq, nkv, 0, pkg.ptr(scratch), max_splits,
                             split_rows)
    keys_seen = chunk * prefix + chunk * (chunk + 1) // 2
    flops = 4 * HD * nq * keys_seen

    def launch(stream):
        pkg.check(K.q38_attention_prefill(C.byref(ap), C.byref(desc), C.byref(kv), stream))
    return launch, flops, (pool, table_d, t, q, gate, out, scratch), (f"{chunk}-token chunk behind {prefix} tokens, "
                                                                     f"{nq} q / {nkv} kv heads")


def gdn_case(pkg, seqs, seed):
    K = pkg.kernels()
    g = torch.Generator(device="cuda").manual_seed(seed)
    conv_dim = (2 * NK + NV) * 128
    ld = conv_dim + NV * 128
    rec = torch.randn((seqs, 1, NV, 128, 128), generator=g, device="cuda") * 0.1
    conv = torch.zeros((seqs, 1, 3, conv_dim), dtype=torch.bfloat16, device="cuda")
    st = pkg.GdnStateDesc(pkg.ptr(rec), pkg.ptr(conv), 1)
    dims = pkg.GdnDims(NK, NV, conv_dim, ld)
    desc, keep = batch_desc(pkg, seqs, [100] * seqs)
    qkv = torch.randn((seqs, conv_dim), generator=g, device="cuda") * 0.1
    ab = torch.randn((seqs, 2 * NV), generator=g, device="cuda")
    A = -torch.rand(NV, generator=g, device="cuda") - 0.5
    dt = torch.randn(NV, generator=g, device="cuda") * 0.5
    nw = torch.ones(128, device="cuda")
    proj = torch.randn((seqs, ld), generator=g, device="cuda").to(torch.bfloat16)
    out = torch.empty((seqs, NV * 128), dtype=torch.bfloat16, device="cuda")
    rp = pkg.GdnRecurrenceParams(pkg.ptr(qkv), pkg.ptr(ab), pkg.ptr(A), pkg.ptr(dt), pkg.ptr(proj) + conv_dim * 2, ld,
                                 pkg.ptr(nw), 1e-6, pkg.ptr(out), 0)
    state_bytes = 2 * seqs * NV * 128 * 128 * 4

    def launch(stream):
        pkg.check(K.q38_gdn_recurrence(C.byref(rp), C.byref(dims), C.byref(desc), C.byref(st), stream))
    return launch, state_bytes, (rec, conv, keep, qkv, ab, A, dt, nw, proj, out), f"{seqs} sequences x {NV} heads"


def scan_case(pkg, tokens, seed):
    """One sequence: the chunked recurrence (per-chunk preparation + state scan) over a `tokens`-token prefill step of
    one GDN layer of the 27B geometry."""
    K = pkg.kernels()
    g = torch.Generator(device="cuda").manual_seed(seed)
    conv_dim = (2 * NK + NV) * 128
    ld = conv_dim + NV * 128
    rec = torch.randn((1, 1, NV, 128, 128), generator=g, device="cuda") * 0.1
    conv = torch.zeros((1, 1, 3, conv_dim), dtype=torch.bfloat16, device="cuda")
    st = pkg.GdnStateDesc(pkg.ptr(rec), pkg.ptr(conv), 1)
    dims = pkg.GdnDims(NK, NV, conv_dim, ld)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    t = {"seq_start": mk([0, tokens]), "seq_slot": mk([0]), "seq_pos0": mk([0]), "tok_pos": mk(list(range(tokens))),
         "tok_seq": mk([0] * tokens)}
    desc = pkg.BatchDesc(1, tokens, tokens, pkg.ptr(t["seq_start"]), pkg.ptr(t["seq_slot"]), pkg.ptr(t["seq_pos0"]),
                         pkg.ptr(t["tok_pos"]), pkg.ptr(t["tok_seq"]))
    qkv = torch.randn((tokens, conv_dim), generator=g, device="cuda") * 0.1
    ab = torch.randn((tokens, 2 * NV), generator=g, device="cuda")
    A = -torch.rand(NV, generator=g, device="cuda") - 0.5
    dt = torch.randn(NV, generator=g, device="cuda") * 0.5
    nw = torch.ones(128, device="cuda")
    proj = torch.randn((tokens, ld), generator=g, device="cuda").to(torch.bfloat16)
    out = torch.empty((tokens, NV * 128), dtype=torch.bfloat16, device="cuda")
    rp = pkg.GdnRecurrenceParams(pkg.ptr(qkv), pkg.ptr(ab), pkg.ptr(A), pkg.ptr(dt), pkg.ptr(proj) + conv_dim * 2, ld,
                                 pkg.ptr(nw), 1e-6, pkg.ptr(out), 0)
    need = int(K.q38_gdn_chunk_scratch_floats(tokens, 1, NV))
    scratch = torch.empty(need, dtype=torch.float32, device="cuda")
    # per (token, value head): four 64x128x128-shaped products of the scan, 2 flops per multiply-add
    flops = 4 * 2 * tokens * NV * 128 * 128

    def launch(stream):
        pkg.check(K.q38_gdn_recurrence_chunked(C.byref(rp), C.byref(dims), C.byref(desc), C.byref(st), pkg.ptr(scratch),
                                               need, stream))
    return launch, flops, (rec, conv, t, qkv, ab, A, dt, nw, proj, out, scratch), f"{tokens} tokens x {NV} heads"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="attn,gdn", help="comma-separated: attn, gdn, prefill, scan")
    ap.add_argument("--prefix", default="2048,32768,131072", help="prefill: cached tokens before the chunk")
    ap.add_argument("--chunk", type=int, default=512, help="prefill: tokens of the step")
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--launches", type=int, default=3, help="with --untimed: number of plain launches")
    ap.add_argument("--untimed", action="store_true", help="launch --launches times on the default stream and exit")
    ap.add_argument("--peak-gbs", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=7)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("op_bench needs a CUDA device")
    pkg = _package()
    K = pkg.kernels()
    for op in args.op.split(","):
        if op == "prefill":  # flash prefill attention: TFLOP/s of the visible (query, key) pairs
            for prefix in [int(x) for x in args.prefix.split(",")]:
                for nq, nkv, rows in ((NQ, NKV, 0), (3, 1, args.chunk)):  # the 27B layer; one rank of 8-way tensor parallelism
                    launch, flops, keep, what = prefill_case(pkg, prefix, args.chunk, args.seed, nq, nkv, rows)
                    if args.untimed:
                        for _ in range(args.launches):
                            launch(None)
                        torch.cuda.synchronize()
                        print(f"ok: prefill: {args.launches} launches, {what}")
                    else:
                        us = timed_graph(launch, max(2, args.iters // 4))
                        print(f"prefill {what}: {us:9.1f} us  {flops / us / 1e6:7.1f} TFLOP/s", flush=True)
                    del keep
            if K.q38_device_error(1):
                raise SystemExit("device-side wait gave up")
            continue
        if op == "scan":  # chunked GDN recurrence of one prefill step, both forms of the scan
            for tensor_cores in (1, 0):
                K.q38_gdn_set_chunk_scan_tensor_cores(tensor_cores)
                launch, flops, keep, what = scan_case(pkg, args.chunk, args.seed)
                form = "tensor cores (split TF32)" if tensor_cores else "fp32 FMA"
                if args.untimed:
                    for _ in range(args.launches):
                        launch(None)
                    torch.cuda.synchronize()
                    print(f"ok: scan [{form}]: {args.launches} launches, {what}")
                else:
                    us = timed_graph(launch, args.iters)
                    print(f"scan  {what} [{form}]: {us:8.1f} us  {flops / us / 1e6:6.1f} TFLOP/s of scan products", flush=True)
                del keep
            K.q38_gdn_set_chunk_scan_tensor_cores(1)
            if K.q38_device_error(1):
                raise SystemExit("device-side wait gave up")
            continue
        launch, nbytes, keep, what = (attn_case if op == "attn" else gdn_case)(pkg, args.seqs, args.seed)
        if args.untimed:
            for _ in range(args.launches):
                launch(None)
            torch.cuda.synchronize()
            print(f"ok: {op}: {args.launches} launches, {what}, {nbytes} algorithmic bytes per launch")
        else:
            us = timed_graph(launch, args.iters)
            gbs = nbytes / us / 1e3
            frac = f" ({100 * gbs / args.peak_gbs:.1f}% of peak)" if args.peak_gbs else ""
            print(f"{op:5s} {what}: {us:8.1f} us  {gbs:7.0f} GB/s{frac}", flush=True)
        if K.q38_device_error(1):
            raise SystemExit("device-side wait gave up")
        del keep
    return 0


if __name__ == "__main__":
    sys.exit(main())
