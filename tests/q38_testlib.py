"""Shared test plumbing: the package, the CPU oracle (ctypes), the optional reference build, and helpers
that put BQ weights / descriptors on the device. The oracle is only ever the checker here."""

from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import torch

import __graft_entry__ as entry

ROOT = Path(__file__).resolve().parents[1]
pkg = entry.load_package()
from q38b200 import bqformat as bq  # noqa: E402
from q38b200 import synth  # noqa: E402

F32P = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def _np(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class CpuOps:
    """ctypes view of a library that exports the oracle operations under `prefix` (orc_ or ref_)."""

    def __init__(self, path: Path, prefix: str):
        self.lib = C.CDLL(str(path))
        self.p = prefix
        self.is_ref = prefix == "ref_"

    def fn(self, name, restype=None):
        f = getattr(self.lib, self.p + name)
        f.restype = restype
        return f

    def dequant(self, packed: bq.Packed) -> np.ndarray:
        lo = np.frombuffer(packed.lo, dtype=np.uint8)
        hi = np.frombuffer(packed.hi, dtype=np.uint8) if packed.hi else None
        sc = np.frombuffer(packed.scales, dtype=np.uint16)
        out = np.empty((packed.n, packed.k), dtype=np.float32)
        self.fn("bq_dequant")(_vp(lo), _vp(hi), _vp(sc), C.c_int(packed.bits), C.c_int64(packed.n),
                              C.c_int64(packed.k), _vp(out))
        return out

    def codes(self, packed: bq.Packed):
        lo = np.frombuffer(packed.lo, dtype=np.uint8)
        hi = np.frombuffer(packed.hi, dtype=np.uint8) if packed.hi else None
        sc = np.frombuffer(packed.scales, dtype=np.uint16)
        codes = np.empty((packed.n, packed.k), dtype=np.int32)
        sbits = np.empty((packed.n, packed.k // 64), dtype=np.uint16)
        self.fn("bq_codes")(_vp(lo), _vp(hi), _vp(sc), C.c_int(packed.bits), C.c_int64(packed.n), C.c_int64(packed.k),
                            _vp(codes), _vp(sbits))
        return codes, sbits

    def norm_partials(self, row: np.ndarray) -> np.ndarray:
        row = _np(row, np.float32)
        out = np.empty(row.shape[-1] // 128, dtype=np.float32)
        self.fn("norm_partials")(_vp(row), C.c_int(row.shape[-1]), _vp(out))
        return out

    def norm_row_scale(self, partials: np.ndarray, hidden: int, eps: float) -> float:
        partials = _np(partials, np.float32)
        return float(self.fn("norm_row_scale", C.c_float)(_vp(partials), C.c_int(partials.size), C.c_int(hidden),
                                                          C.c_float(eps)))

    def qgemm(self, a, w, row_scale, epilogue, out=None, ldo=0, residual=None, xbf=None, partials=None, exact=False):
        a = _np(a, np.float32)
        w = _np(w, np.float32)
        m, k = a.shape
        n = w.shape[0]
        rs = None if row_scale is None else _np(row_scale, np.float32)
        self.fn("qgemm")(_vp(a), C.c_int(m), _vp(w), C.c_int(n), C.c_int(k), _vp(rs), C.c_int(epilogue), _vp(out),
                         C.c_int(ldo), _vp(residual), _vp(xbf), _vp(partials), C.c_int(int(exact)))

    def int8_group_roundtrip(self, x: np.ndarray) -> np.ndarray:
        x = _np(x, np.float32).copy()
        self.fn("int8_group_roundtrip")(_vp(x), C.c_int(x.size))
        return x

    def gdn_token(self, lk, lv, eps, proj_row, ab_row, conv_w, A, dt_bias, norm_w, state_s, state_conv, exact=False):
        out = np.empty(lv * 128, dtype=np.float32)
        self.fn("gdn_token")(C.c_int(lk), C.c_int(lv), C.c_float(eps), _vp(_np(proj_row, np.float32)),
                             _vp(_np(ab_row, np.float32)), _vp(_np(conv_w, np.float32)), _vp(_np(A, np.float32)),
                             _vp(_np(dt_bias, np.float32)), _vp(_np(norm_w, np.float32)), _vp(state_s),
                             _vp(state_conv), _vp(out), C.c_int(int(exact)))
        return out


    def sample_penalties(self, logits: np.ndarray, history, presence: float, repetition: float, cap: int) -> np.ndarray:
        """Penalised copy of one logits row (every distinct history token once)."""
        out = _np(logits, np.float32).copy()
        h = _np(history, np.int32)
        self.fn("sample_penalties")(_vp(out), C.c_int(out.size), _vp(h), C.c_int(h.size), C.c_int(cap),
                                    C.c_float(presence), C.c_float(repetition))
        return out

    def sample_draws(self, logits: np.ndarray, temperature, top_k, top_p, min_p, seeds, steps):
        """Tokens and log-probabilities of len(seeds) draws from one (already penalised) logits row."""
        lg = _np(logits, np.float32)
        sd, st = _np(seeds, np.uint64), _np(steps, np.int32)
        toks = np.empty(sd.size, dtype=np.int32)
        lps = np.empty(sd.size, dtype=np.float32)
        self.fn("sample_draws")(_vp(lg), C.c_int(lg.size), C.c_float(temperature), C.c_int(top_k), C.c_float(top_p),
                                C.c_float(min_p), _vp(sd), _vp(st), C.c_int(sd.size), _vp(toks), _vp(lps))
        return toks, lps


class OracleKv:
    """Dequantised KV store of one sequence and one layer, [kv_heads][capacity][256], for either library."""

    def __init__(self, ops: CpuOps, kv_heads: int, capacity: int):
        self.ops, self.kv_heads, self.capacity = ops, kv_heads, capacity
        if ops.is_ref:
            create = ops.fn("kv_create", C.c_void_p)
            self.handle = C.c_void_p(create(C.c_int(kv_heads), C.c_int(capacity)))
            kp = ops.fn("kv_k", C.POINTER(C.c_float))(self.handle)
            vp = ops.fn("kv_v", C.POINTER(C.c_float))(self.handle)
            self.k = np.ctypeslib.as_array(kp, shape=(kv_heads, capacity, 256))
            self.v = np.ctypeslib.as_array(vp, shape=(kv_heads, capacity, 256))
        else:
            self.handle = None
            self.k = np.zeros((kv_heads, capacity, 256), dtype=np.float32)
            self.v = np.zeros((kv_heads, capacity, 256), dtype=np.float32)

    def append(self, nq, eps, theta, proj_row, pos, q_norm, k_norm, kv_dtype=2, exact=False) -> np.ndarray:
        q_out = np.empty(nq * 256, dtype=np.float32)
        args = [C.c_int(nq), C.c_int(self.kv_heads), C.c_float(eps), C.c_double(theta), _vp(_np(proj_row, np.float32)),
                C.c_int(pos), _vp(_np(q_norm, np.float32)), _vp(_np(k_norm, np.float32)), _vp(q_out)]
        if self.ops.is_ref:
            args += [self.handle]
        else:
            args += [_vp(self.k), _vp(self.v), C.c_int(self.capacity)]
        args += [C.c_int(kv_dtype), C.c_int(int(exact))]
        self.ops.fn("qk_norm_rope_append")(*args)
        return q_out

    def attend(self, nq, q, gate, pos, exact=False) -> np.ndarray:
        out = np.empty(nq * 256, dtype=np.float32)
        args = [C.c_int(nq), C.c_int(self.kv_heads), _vp(_np(q, np.float32)), _vp(_np(gate, np.float32)), C.c_int(pos)]
        if self.ops.is_ref:
            args += [self.handle]
        else:
            args += [_vp(self.k), _vp(self.v), C.c_int(self.capacity)]
        args += [_vp(out), C.c_int(int(exact))]
        self.ops.fn("attention_token")(*args)
        return out


_oracle = None


def oracle() -> CpuOps:
    global _oracle
    if _oracle is None:
        so = ROOT / "oracle" / "_build" / "libq38_oracle.so"
        src = ROOT / "oracle" / "q38_oracle.cpp"
        if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
            subprocess.run(["make", "-s", "-C", str(ROOT / "oracle"), "all"], check=True)
        _oracle = CpuOps(so, "orc_")
    return _oracle


def reference_ops():
    """The reference's own CPU code (oracle/_ref), or None where it has not been built."""
    so = ROOT / "oracle" / "_ref" / "libq38_ref.so"
    return CpuOps(so, "ref_") if so.exists() else None


def reference_binary():
    exe = ROOT / "oracle" / "_ref" / "qwen38-ref"
    return exe if exe.exists() else None


# ---- device helpers -------------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


class DeviceBQ:
    """A packed BQ tensor uploaded to the GPU plus its C descriptor."""

    def __init__(self, packed: bq.Packed, rows: int | None = None, device="cuda"):
        self.packed = packed
        self.lo = torch.frombuffer(bytearray(packed.lo), dtype=torch.uint8).to(device)
        self.hi = torch.frombuffer(bytearray(packed.hi), dtype=torch.uint8).to(device) if packed.hi else None
        self.sc = torch.frombuffer(bytearray(packed.scales), dtype=torch.uint8).to(device)
        self.desc = pkg.BQWeight(pkg.ptr(self.lo), pkg.ptr(self.hi), pkg.ptr(self.sc), packed.bits, packed.n, packed.k,
                                 rows if rows is not None else packed.n)


def make_bq(n: int, k: int, bits: int, seed: int, std: float = 0.02, grid: int = 24, fast: bool = False) -> bq.Packed:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((n, k), generator=g) * std
    codes, scales = (bq.quantize_absmax(w, bits) if fast else bq.quantize_matrix(w, bits, grid))
    return bq.pack(codes, scales, bits)


class Workspace:
    def __init__(self, floats: int = 2 * 148 * 128 * 512, counters: int = 65536, device="cuda"):
        self.partials = torch.empty(floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.desc = pkg.GemmWorkspace(pkg.ptr(self.partials), floats, pkg.ptr(self.counters), counters)


class Batch:
    """Ragged batch metadata on the device from (slot, pos0, n) triples."""

    def __init__(self, seqs, device="cuda"):
        seq_start, seq_slot, seq_pos0, tok_pos, tok_seq = [0], [], [], [], []
        for b, (slot, pos0, n) in enumerate(seqs):
            seq_slot.append(slot)
            seq_pos0.append(pos0)
            tok_pos += [pos0 + i for i in range(n)]
            tok_seq += [b] * n
            seq_start.append(seq_start[-1] + n)
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        self.seq_start, self.seq_slot, self.seq_pos0 = mk(seq_start), mk(seq_slot), mk(seq_pos0)
        self.tok_pos, self.tok_seq = mk(tok_pos), mk(tok_seq)
        self.num_tokens = seq_start[-1]
        self.desc = pkg.BatchDesc(len(seqs), seq_start[-1], max(n for _, _, n in seqs), pkg.ptr(self.seq_start),
                                  pkg.ptr(self.seq_slot), pkg.ptr(self.seq_pos0), pkg.ptr(self.tok_pos),
                                  pkg.ptr(self.tok_seq))


class KvPool:
    """A paged KV pool with an explicit block table (tests choose the page ids)."""

    def __init__(self, kv_heads: int, layers: int, num_pages: int, slots: int, max_pages_per_seq: int, dtype=0,
                 device="cuda"):
        self.kv_heads, self.layers, self.num_pages, self.dtype = kv_heads, layers, num_pages, dtype
        self.page_bytes = int(pkg.kernels().q38_kv_page_bytes(dtype, kv_heads))
        self.layer_stride = self.page_bytes * num_pages
        self.pool = torch.zeros(self.layer_stride * layers, dtype=torch.uint8, device=device)
        self.table = torch.zeros((slots, max_pages_per_seq), dtype=torch.int32, device=device)
        self.max_pages_per_seq = max_pages_per_seq

    @property
    def desc(self):
        return pkg.KvCacheDesc(pkg.ptr(self.pool), self.dtype, self.kv_heads, self.num_pages, self.page_bytes,
                               self.layer_stride, pkg.ptr(self.table), self.max_pages_per_seq)

    def read_sequence(self, layer: int, slot: int, length: int):
        """Dequantised K, V [kv_heads][length][256] fp32 as the attention kernels see them."""
        table = self.table[slot].cpu().numpy()
        k = np.zeros((self.kv_heads, length, 256), dtype=np.float32)
        v = np.zeros_like(k)
        for p in range((length + 63) // 64):
            base = layer * self.layer_stride + int(table[p]) * self.page_bytes
            page = self.pool[base:base + self.page_bytes].cpu().numpy()
            n = min(64, length - 64 * p)
            H = self.kv_heads
            if self.dtype == 0:
                kq = page[:H * 64 * 256].view(np.int8).reshape(H, 64, 256).astype(np.float32)
                vq = page[H * 64 * 256:2 * H * 64 * 256].view(np.int8).reshape(H, 64, 256).astype(np.float32)
                sc = page[2 * H * 64 * 256:].view(np.float16).astype(np.float32)
                ks, vs = sc[:H * 64 * 4].reshape(H, 64, 4), sc[H * 64 * 4:].reshape(H, 64, 4)
                kd = kq * np.repeat(ks, 64, axis=2)
                vd = vq * np.repeat(vs, 64, axis=2)
            else:
                raw = torch.from_numpy(page.view(np.int16).copy()).view(torch.bfloat16).to(torch.float32).numpy()
                kd = raw[:H * 64 * 256].reshape(H, 64, 256)
                vd = raw[H * 64 * 256:].reshape(H, 64, 256)
            k[:, 64 * p:64 * p + n] = kd[:, :n]
            v[:, 64 * p:64 * p + n] = vd[:, :n]
        return k, v


def to_dev_bf16(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).cuda()
