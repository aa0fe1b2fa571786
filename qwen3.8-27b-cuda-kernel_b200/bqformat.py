"""BQ group-wise 4/5/6/8-bit weights and the `.q38` container: quantise, pack, unpack, read, write.

This is the data-format side of the drop-in: files written here are byte-compatible with the
reference's converter output (reference docs/FORMAT.md sections 1-2; reference tools/bqpack.py and
tools/convert.py are the producers there, src/model_file.cpp and src/bq_host.cpp the readers), so
the reference CPU model and this engine can be run on the very same file.

Layout facts used below (reference docs/FORMAT.md 2.2-2.5):
  * slab = 16 (k) x 64 (n); slabs are stored n-block-major: index = nb * (K / 16) + kb;
  * lane L = 4 g + t of a slab owns column n = 64 nb + 8 j + g and rows k = 16 kb + 2 t + 8 h + e,
    as 16 pairs q = 2 j + h of two elements e;
  * lo plane: 16 bytes per lane = 4 little-endian words, pair q in word q >> 2 at nibble q & 3
    (element 0 in the low half-word, element 1 in the high half-word);
  * hi plane: 5-bit -> one word per lane (bit q / bit 16 + q); 6-bit -> two words per lane (2-bit
    fields at 2 (q & 7) / 16 + 2 (q & 7)); 8-bit -> a second nibble plane;
  * scales: bf16, 64 per (nb, k-group) block, column 8 j + g stored at position 8 g + j.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

GROUP = 64
MAGIC = b"QW38MDL1"
BITS = (4, 5, 6, 8)

# bits per role, reference tools/convert.py:38-54
RECIPES = {
    "default": {"attn.qkvg": 5, "attn.o": 5, "gdn.qkvz": 5, "gdn.out": 5, "mlp.gate_up": 4, "mlp.down": 5,
                "lm_head": 8},
    "lean": {"attn.qkvg": 4, "attn.o": 4, "gdn.qkvz": 4, "gdn.out": 4, "mlp.gate_up": 4, "mlp.down": 4,
             "lm_head": 6},
    "quality": {"attn.qkvg": 5, "attn.o": 6, "gdn.qkvz": 5, "gdn.out": 6, "mlp.gate_up": 4, "mlp.down": 6,
                "lm_head": 8},
    "q8": {"attn.qkvg": 8, "attn.o": 8, "gdn.qkvz": 8, "gdn.out": 8, "mlp.gate_up": 8, "mlp.down": 8,
           "lm_head": 8},
}


def _bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


# ---------------------------------------------------------------------------------------------------
# quantiser (reference docs/FORMAT.md 2.7, tools/bqpack.py:40-102): per (row, 64-group) the scale
# with the least squared error among candidates that map the signed extreme onto either end of the
# code range, each stretched over `grid` factors in [0.80, 1.06] and refitted by least squares; the
# winner is rounded to bf16 and the codes are recomputed against the rounded scale.
# ---------------------------------------------------------------------------------------------------
@torch.no_grad()
def quantize_groups(x: torch.Tensor, bits: int, grid: int = 24):
    """x [G, 64] fp32 -> (codes int16 [G, 64], scales fp32 [G], bf16-representable)."""
    assert x.dim() == 2 and x.shape[1] == GROUP
    lo_code, hi_code = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    x = x.to(torch.float32)
    extreme = x.gather(1, x.abs().argmax(dim=1, keepdim=True)).squeeze(1)
    live = extreme != 0
    ext = torch.where(live, extreme, torch.ones_like(extreme))
    best_err = torch.full_like(ext, float("inf"))
    best = torch.zeros_like(ext)
    stretch = torch.linspace(0.80, 1.06, grid, device=x.device)
    for end in (float(lo_code), float(hi_code)):
        for f in stretch:
            s0 = ext / (end * f)
            c0 = torch.clamp(torch.round(x / s0[:, None]), lo_code, hi_code)
            dot, sq = (c0 * x).sum(dim=1), (c0 * c0).sum(dim=1)
            s1 = _bf16_round(torch.where(sq > 0, dot / sq.clamp_min(1e-30), s0))
            s1 = torch.where(s1 == 0, _bf16_round(s0), s1)
            c1 = torch.clamp(torch.round(x / s1[:, None]), lo_code, hi_code)
            err = ((c1 * s1[:, None] - x) ** 2).sum(dim=1)
            take = err < best_err
            best_err = torch.where(take, err, best_err)
            best = torch.where(take, s1, best)
    best = torch.where(live, best, torch.zeros_like(best))
    div = torch.where(best != 0, best, torch.ones_like(best))
    codes = torch.clamp(torch.round(x / div[:, None]), lo_code, hi_code)
    codes = torch.where(best[:, None] != 0, codes, torch.zeros_like(codes))
    return codes.to(torch.int16), best


@torch.no_grad()
def quantize_matrix(w: torch.Tensor, bits: int, grid: int = 24, row_chunk: int = 2048):
    """w [N, K] -> (codes int16 [N, K], scales fp32 [N, K / 64])."""
    assert bits in BITS
    n, k = w.shape
    assert k % GROUP == 0
    codes = torch.empty((n, k), dtype=torch.int16, device=w.device)
    scales = torch.empty((n, k // GROUP), dtype=torch.float32, device=w.device)
    for r0 in range(0, n, row_chunk):
        r1 = min(n, r0 + row_chunk)
        c, s = quantize_groups(w[r0:r1].to(torch.float32).reshape(-1, GROUP), bits, grid)
        codes[r0:r1] = c.reshape(r1 - r0, k)
        scales[r0:r1] = s.reshape(r1 - r0, k // GROUP)
    return codes, scales


@torch.no_grad()
def quantize_absmax(w: torch.Tensor, bits: int):
    """Fast quantiser (scale = amax / (2^(b-1) - 1), bf16) for large synthetic benchmark weights."""
    n, k = w.shape
    g = w.to(torch.float32).reshape(n, k // GROUP, GROUP)
    s = _bf16_round(g.abs().amax(dim=2) / float((1 << (bits - 1)) - 1))
    div = torch.where(s != 0, s, torch.ones_like(s))
    c = torch.clamp(torch.round(g / div[:, :, None]), -(1 << (bits - 1)), (1 << (bits - 1)) - 1)
    return c.reshape(n, k).to(torch.int16), s


def dequantize(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """bf16(code * scale) as fp32 — the exact weight value every reader must reproduce."""
    return _bf16_round(codes.to(torch.float32) * scales.to(torch.float32).repeat_interleave(GROUP, dim=1))


# ---------------------------------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------------------------------
@dataclass
class Packed:
    bits: int
    n: int
    k: int
    lo: bytes
    hi: bytes
    scales: bytes


def plane_bytes(n: int, k: int, bits: int):
    return n * k // 2, n * k * (bits - 4) // 8, n * (k // GROUP) * 2


def _to_lanes(u: np.ndarray) -> np.ndarray:
    """[N, K] -> [slab, lane 32, pair 16, elem 2] in plane order."""
    n, k = u.shape
    nb, kb = n // 64, k // 16
    #  n = 64 nb + 8 j + g ; k = 16 kb + 8 h + 2 t + e
    v = u.reshape(nb, 8, 8, kb, 2, 4, 2)             # nb j g kb h t e
    v = np.transpose(v, (0, 3, 2, 5, 1, 4, 6))       # nb kb g t j h e
    return np.ascontiguousarray(v).reshape(nb * kb, 32, 16, 2)


def _from_lanes(v: np.ndarray, n: int, k: int) -> np.ndarray:
    nb, kb = n // 64, k // 16
    v = v.reshape(nb, kb, 8, 4, 8, 2, 2)             # nb kb g t j h e
    v = np.transpose(v, (0, 4, 2, 1, 5, 3, 6))       # nb j g kb h t e
    return np.ascontiguousarray(v).reshape(n, k)


def _nibble_words(vals: np.ndarray) -> np.ndarray:
    """[slab, 32, 16, 2] of 4-bit values -> [slab, 32, 4] u32 words."""
    v = vals.astype(np.uint32).reshape(vals.shape[0], 32, 4, 4, 2)
    sh = (4 * np.arange(4, dtype=np.uint32))[None, None, None, :]
    return ((v[..., 0] << sh) | (v[..., 1] << (sh + 16))).sum(axis=-1, dtype=np.uint32)


def _nibbles_of(words: np.ndarray) -> np.ndarray:
    w = words.astype(np.uint32)[..., None]
    sh = 4 * np.arange(4, dtype=np.uint32)
    e0, e1 = (w >> sh) & 15, (w >> (sh + 16)) & 15
    return np.stack([e0, e1], axis=-1).reshape(words.shape[0], 32, 16, 2)


def _pack_on_device(codes: torch.Tensor, scales: torch.Tensor, bits: int) -> Packed:
    """pack() as tensor arithmetic on the device the codes live on (same bytes; a 27B-sized matrix packs in well
    under a second on a GPU where the numpy path needs half a minute)."""
    n, k = codes.shape
    dev = codes.device
    nb, kb = n // 64, k // 16
    u = codes.to(torch.int64) + (1 << (bits - 1))
    #  n = 64 nb + 8 j + g ; k = 16 kb + 8 h + 2 t + e  ->  [slab, lane (g t), pair (j h), e]
    lanes = u.reshape(nb, 8, 8, kb, 2, 4, 2).permute(0, 3, 2, 5, 1, 4, 6).reshape(nb * kb, 32, 16, 2)

    def words(v, shifts):  # v [..., P, 2], shifts [P]: sum_p (v0 << s_p) | (v1 << (s_p + 16)) as little-endian u32 bytes
        w = ((v[..., 0] << shifts) | (v[..., 1] << (shifts + 16))).sum(dim=-1)
        return (w & 0xFFFFFFFF).to(torch.int32).contiguous().cpu().numpy().astype("<u4").tobytes()

    ar = lambda cnt, step: step * torch.arange(cnt, dtype=torch.int64, device=dev)
    lo = words((lanes & 15).reshape(-1, 32, 4, 4, 2), ar(4, 4))
    top = lanes >> 4
    if bits == 4:
        hi = b""
    elif bits == 5:
        hi = words(top, ar(16, 1))
    elif bits == 6:
        hi = words(top.reshape(-1, 32, 2, 8, 2), ar(8, 2))
    else:
        hi = words(top.reshape(-1, 32, 4, 4, 2), ar(4, 4))
    s16 = scales.to(torch.float32).to(torch.bfloat16).view(torch.int16)
    s16 = s16.reshape(nb, 8, 8, k // GROUP).permute(0, 3, 2, 1).contiguous().cpu().numpy()
    return Packed(bits, n, k, lo, hi, s16.astype("<i2").tobytes())


def pack(codes: torch.Tensor, scales: torch.Tensor, bits: int) -> Packed:
    assert bits in BITS
    n, k = codes.shape
    assert n % 128 == 0 and k % GROUP == 0, (n, k)
    if codes.is_cuda:
        return _pack_on_device(codes, scales, bits)
    u = (codes.to(torch.int32).cpu().numpy() + (1 << (bits - 1))).astype(np.uint32)
    assert int(u.max()) < (1 << bits)
    lanes = _to_lanes(u)
    lo = _nibble_words(lanes & 15).astype("<u4").tobytes()
    top = lanes >> 4
    if bits == 4:
        hi = b""
    elif bits == 5:
        q = np.arange(16, dtype=np.uint32)
        hi = ((top[..., 0] << q) | (top[..., 1] << (q + 16))).sum(axis=-1, dtype=np.uint32).astype("<u4").tobytes()
    elif bits == 6:
        t2 = top.reshape(top.shape[0], 32, 2, 8, 2)
        r = 2 * np.arange(8, dtype=np.uint32)
        hi = ((t2[..., 0] << r) | (t2[..., 1] << (r + 16))).sum(axis=-1, dtype=np.uint32).astype("<u4").tobytes()
    else:
        hi = _nibble_words(top).astype("<u4").tobytes()
    s16 = scales.to(torch.float32).cpu().to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    s16 = s16.reshape(n // 64, 8, 8, k // GROUP)      # nb j g group
    s16 = np.transpose(s16, (0, 3, 2, 1))             # nb group g j
    return Packed(bits, n, k, lo, hi, np.ascontiguousarray(s16).astype("<u2").tobytes())


def unpack(p: Packed):
    """-> (codes int16 [N, K], scales fp32 [N, K / 64])"""
    n, k, bits = p.n, p.k, p.bits
    slabs = (n // 64) * (k // 16)
    u = _nibbles_of(np.frombuffer(p.lo, dtype="<u4").reshape(slabs, 32, 4))
    if bits == 5:
        w = np.frombuffer(p.hi, dtype="<u4").reshape(slabs, 32).astype(np.uint32)[..., None]
        q = np.arange(16, dtype=np.uint32)
        u = u | (np.stack([(w >> q) & 1, (w >> (q + 16)) & 1], axis=-1) << 4)
    elif bits == 6:
        w = np.frombuffer(p.hi, dtype="<u4").reshape(slabs, 32, 2).astype(np.uint32)[..., None]
        r = 2 * np.arange(8, dtype=np.uint32)
        h = np.stack([(w >> r) & 3, (w >> (r + 16)) & 3], axis=-1).reshape(slabs, 32, 16, 2)
        u = u | (h << 4)
    elif bits == 8:
        u = u | (_nibbles_of(np.frombuffer(p.hi, dtype="<u4").reshape(slabs, 32, 4)) << 4)
    codes = torch.from_numpy((_from_lanes(u, n, k).astype(np.int32) - (1 << (bits - 1))).astype(np.int16))
    s16 = np.frombuffer(p.scales, dtype="<u2").reshape(n // 64, k // GROUP, 8, 8)   # nb group g j
    s16 = np.ascontiguousarray(np.transpose(s16, (0, 3, 2, 1))).reshape(n, k // GROUP)
    scales = torch.from_numpy(s16.astype(np.int16)).view(torch.bfloat16).to(torch.float32)
    return codes, scales


# ---------------------------------------------------------------------------------------------------
# .q38 container (reference docs/FORMAT.md 1; writer: tools/convert.py:341-449; reader:
# src/model_file.cpp:141-237)
# ---------------------------------------------------------------------------------------------------
def _up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class Q38Writer:
    """Collects tensors, then writes header + 256-byte-aligned payloads."""

    def __init__(self, config: dict, recipe: str = "default"):
        self.config = dict(config)
        self.recipe = recipe
        self.records: dict[str, dict] = {}
        self.blobs: list[tuple[int, bytes]] = []
        self.cursor = 0

    def _place(self, blob: bytes):
        self.cursor = _up(self.cursor, 256)
        at = self.cursor
        self.blobs.append((at, blob))
        self.cursor += len(blob)
        return at

    def add_direct(self, name: str, t: torch.Tensor, dtype: str):
        if dtype == "bf16":
            blob = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        else:
            blob = t.to(torch.float32).contiguous().numpy().astype("<f4").tobytes()
        self.records[name] = {"dtype": dtype, "shape": list(t.shape), "offset": self._place(blob),
                              "bytes": len(blob)}

    def add_bq(self, name: str, w: torch.Tensor, bits: int, grid: int = 24, quantizer=None, device="cpu"):
        rows, k = w.shape
        n = _up(rows, 128)
        if n != rows:
            w = torch.cat([w, torch.zeros(n - rows, k, dtype=w.dtype)], dim=0)
        w = w.to(device)
        codes, scales = (quantizer or (lambda m, b: quantize_matrix(m, b, grid)))(w, bits)
        self.add_packed(name, pack(codes, scales, bits), rows)
        return codes, scales

    def add_packed(self, name: str, p: Packed, rows: int | None = None):
        planes = {"lo": [self._place(p.lo), len(p.lo)]}
        if p.hi:
            planes["hi"] = [self._place(p.hi), len(p.hi)]
        planes["scales"] = [self._place(p.scales), len(p.scales)]
        rec = {"dtype": f"bq{p.bits}", "shape": [p.n, p.k], "group_size": GROUP, "planes": planes}
        if rows is not None and rows != p.n:
            rec["rows"] = rows
        self.records[name] = rec

    def write(self, path: str | Path):
        header = {"format": "qwen38-model", "format_version": 1, "config": self.config,
                  "recipe": {"name": self.recipe}, "tensors": self.records, "resources": {},
                  "provenance": {"source": "synthetic", "converter": "qwen38-b200 bqformat.Q38Writer"}}
        hb = json.dumps(header, indent=1).encode("utf-8")
        start = _up(16 + len(hb), 4096)
        with open(path, "wb") as f:
            f.write(MAGIC + struct.pack("<Q", len(hb)) + hb)
            f.write(b"\0" * (start - f.tell()))
            for at, blob in self.blobs:
                f.seek(start + at)
                f.write(blob)
            f.seek(start + self.cursor)
            f.truncate()


class Q38File:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        if self._f.read(8) != MAGIC:
            raise ValueError(f"{path} is not a .q38 file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(hlen))
        self.data_start = _up(16 + hlen, 4096)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.config = self.header["config"]
        self.tensors = self.header["tensors"]

    def raw(self, off: int, size: int) -> bytes:
        return self._mm[self.data_start + off:self.data_start + off + size]

    def direct(self, name: str) -> torch.Tensor:
        rec = self.tensors[name]
        raw = self.raw(rec["offset"], rec["bytes"])
        if rec["dtype"] == "bf16":
            return torch.from_numpy(np.frombuffer(raw, dtype="<i2").copy()).view(torch.bfloat16).reshape(rec["shape"])
        return torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()).reshape(rec["shape"])

    def packed(self, name: str) -> Packed:
        rec = self.tensors[name]
        pl = rec["planes"]
        n, k = rec["shape"]
        return Packed(int(rec["dtype"][2:]), n, k, self.raw(*pl["lo"]), self.raw(*pl["hi"]) if "hi" in pl else b"",
                      self.raw(*pl["scales"]))

    def rows(self, name: str) -> int:
        rec = self.tensors[name]
        return rec.get("rows", rec["shape"][0])

    def dequant(self, name: str) -> torch.Tensor:
        """Padded [N, K] fp32 (bf16-exact) weight."""
        return dequantize(*unpack(self.packed(name)))
