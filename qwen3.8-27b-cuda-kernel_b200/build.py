"""In-tree build of the native libraries (no GPU needed: nvcc cross-compiles for sm_100a).

    python qwen3.8-27b-cuda-kernel_b200/build.py [--force] [--verbose]

Outputs, next to this file:
    lib/libq38_kernels.so   every CUDA kernel + the C ABI declared in include/q38_kernels.h
    lib/libq38_engine.so    the C++20 host engine (ModelFile, KvCache, ModelRunner, Engine) + its C ABI
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = HERE / "csrc"
HOST = HERE / "host"
OBJ = HERE / "build"
LIB = HERE / "lib"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_LIB = str(Path(NVCC).resolve().parents[1] / "lib64")
CUDA_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-I", str(ROOT / "include")]
HOST_FLAGS = ["-std=c++20", "-O2", "-fPIC", "-I", str(ROOT / "include"), "-I", str(HOST / "include"),
              "-I", "/usr/local/cuda/include"]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> dict[str, Path]:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    cu_headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT / "include" / "q38_kernels.h"]
    jobs = []
    cu_objs = []
    for src in sorted(CSRC.glob("*.cu")):
        obj = OBJ / (src.stem + ".o")
        cu_objs.append(obj)
        if force or _stale(obj, [src] + cu_headers):
            extra = ["-Xptxas", "-v"] if ptxas_verbose else []
            jobs.append([NVCC, *CUDA_FLAGS, *extra, "-c", str(src), "-o", str(obj)])
    host_headers = sorted((HOST / "include").rglob("*.h")) + sorted((ROOT / "include").glob("*.h"))
    host_objs = []
    for src in sorted((HOST / "src").glob("*.cpp")):
        obj = OBJ / ("host_" + src.stem + ".o")
        host_objs.append(obj)
        if force or _stale(obj, [src] + host_headers):
            jobs.append(["g++", *HOST_FLAGS, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(lambda c: _run(c, verbose or ptxas_verbose), jobs))
    kernels_so = LIB / "libq38_kernels.so"
    if force or _stale(kernels_so, cu_objs):
        # both libraries use the one shared CUDA runtime of the process (a host application's, or torch's in the
        # tests and benchmarks): same soname, so whichever copy is loaded first serves everybody
        _run([NVCC, "-shared", "--cudart", "shared", "-o", str(kernels_so), *map(str, cu_objs),
              "-Xlinker", f"-rpath,{CUDA_LIB}"], verbose)
    out = {"kernels": kernels_so}
    if host_objs:
        engine_so = LIB / "libq38_engine.so"
        if force or _stale(engine_so, host_objs + [kernels_so]):
            _run(["g++", "-shared", "-o", str(engine_so), *map(str, host_objs), "-L", str(LIB), "-lq38_kernels",
                  f"-L{CUDA_LIB}", "-lcudart", "-ldl", "-lrt", "-lpthread",
                  f"-Wl,-rpath,$ORIGIN:{CUDA_LIB}"], verbose)
        out["engine"] = engine_so
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args()
    for name, path in build(a.force, a.verbose, a.ptxas).items():
        print(f"{name}: {path}")
