"""q38_qgemm_static: the decode GEMM for hosts that cannot allocate device memory (a plugin that only receives
its tensors, a server whose memory pool is sealed at start-up). Its stream-K workspace is a fixed array inside
the library, so the call takes inputs and outputs only. Checked here against q38_qgemm with a caller-owned
workspace: the same kernel and grid, so the results must be bit-identical, on two calls in a row (the second
call finds the array as the first one left it). Collected last on purpose."""

import ctypes as C

import numpy as np
import pytest
import torch

import q38_testlib as tl
from q38_testlib import pkg

pytestmark = pytest.mark.gpu


def test_static_workspace_gemm_matches_the_caller_workspace_gemm_twice():
    K = pkg.kernels()
    rng = np.random.default_rng(17)
    ws = tl.Workspace()
    # the last shape has more than four 128-column tiles per SM: the even cut over all SMs, two partial tiles per CTA
    for bits, n, k in ((4, 1536, 512), (5, 5120, 1024), (8, 256, 6144), (4, 76800, 256)):
        w = tl.DeviceBQ(tl.make_bq(n, k, bits, seed=bits, std=0.05, fast=True))
        for m in (1, 7, 16):
            a = tl.to_dev_bf16(rng.standard_normal((m, k)))
            want = torch.empty((m, n), dtype=torch.float32, device="cuda")
            ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(want), n, 0, None, None, None, None, 0, 1e-6)
            pkg.check(K.q38_qgemm(pkg.ptr(a), m, C.byref(w.desc), C.byref(ep), C.byref(ws.desc), None, -1))
            for call in range(2):
                got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
                ep2 = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(got), n, 0, None, None, None, None, 0, 1e-6)
                pkg.check(K.q38_qgemm_static(pkg.ptr(a), m, C.byref(w.desc), C.byref(ep2), None))
                torch.cuda.synchronize()
                assert torch.equal(got, want), (bits, n, k, m, call)
    assert K.q38_device_error(1) == 0
    # sizes beyond the built-in workspace are refused before anything is launched
    a = torch.zeros((17, 512), dtype=torch.bfloat16, device="cuda")
    w = tl.DeviceBQ(tl.make_bq(128, 512, 4, seed=1, fast=True))
    out = torch.zeros((17, 128), dtype=torch.float32, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(out), 128, 0, None, None, None, None, 0, 1e-6)
    assert K.q38_qgemm_static(pkg.ptr(a), 17, C.byref(w.desc), C.byref(ep), None) == -1
    assert b"outside the built-in workspace" in K.q38_last_error()
