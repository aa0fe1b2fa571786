// In-register decoder of BQ 4/5/6/8-bit weight slabs (format: reference docs/FORMAT.md 2.1-2.5).
//
// One warp lane owns 16 bytes of a slab's lo plane (+ 4 / 8 / 16 bytes of its hi plane): 16 pairs
// q = 2 j + h of weights for column 8 j + g and rows 2 t + 8 h + {0, 1} (g = lane >> 2, t = lane & 3).
// decode_slab() turns them into 16 packed bf16x2 values w[q] = bf16(code * scale), bit-exact with the
// format definition W = bf16(float(c) * float(s)): the unsigned code u is placed in the mantissa of the
// bf16 number 128 (0x4300 | u == 128 + u exactly, u < 128), the bias 128 + 2^(b-1) is removed with an
// exact bf16 subtraction, and one bf16 multiply by the group scale performs the single rounding.
#pragma once

#include <utility>

#include "common.cuh"

namespace q38 {

template <int BITS>
struct BqGeom {
  static_assert(BITS == 4 || BITS == 5 || BITS == 6 || BITS == 8, "BQ bit width");
  static constexpr int kHiSlabBytes = BITS == 4 ? 0 : BITS == 5 ? 128 : BITS == 6 ? 256 : 512;
  static constexpr int kHiLaneWords = kHiSlabBytes / 128;  // u32 words per lane: 0, 1, 2, 4
  static constexpr int kLoGroupBytes = 4 * 512;            // one 64-wide k-group of one 64-column block
  static constexpr int kHiGroupBytes = 4 * kHiSlabBytes;
  static constexpr int kScGroupBytes = 128;
};

__device__ __forceinline__ uint32_t bf16x2_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 bits_bf16x2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

template <int SH>
__device__ __forceinline__ uint32_t shr_mul(uint32_t x) {
  return x >> SH;
}
template <int SH>
__device__ __forceinline__ uint32_t shl_mul(uint32_t x) {
  return x << SH;
}

// Bit masks of the decoder, handed to the kernels as launch arguments. A three-input logic instruction takes one
// immediate at most; with the masks as compile-time constants the compiler spends two instructions on
// (x & nibble) | magic, with the masks in registers (values it cannot see) it spends one.
struct DecodeConsts {
  uint32_t nib;     // 0x000F000F
  uint32_t magic;   // 0x43004300: bf16x2 (128, 128)
  uint32_t himask;  // 0x00100010 (5 bit) / 0x00300030 (6 bit)
};
inline DecodeConsts decode_consts(int bits) { return DecodeConsts{0x000F000Fu, 0x43004300u, bits == 6 ? 0x00300030u : 0x00100010u}; }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t b, uint32_t c) {  // a | (b & c)
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xF8;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <int BITS, int Q>
__device__ __forceinline__ uint32_t decode_pair(const uint32_t (&lo)[4], const uint32_t (&hi)[4], uint32_t s2,
                                                const DecodeConsts& dc) {
  constexpr uint32_t kMagic = 0x43004300u;  // bf16x2 (128, 128)
  constexpr int p = Q & 3;
  uint32_t v = lop3_and_or(shr_mul<4 * p>(lo[Q >> 2]), dc.nib, dc.magic);
  __nv_bfloat162 c;
  if constexpr (BITS == 4) {
    c = __hsub2(bits_bf16x2(v), bits_bf16x2(0x43084308u));  // 136
  } else if constexpr (BITS == 5) {
    uint32_t h;
    if constexpr (Q >= 4) h = shr_mul<Q - 4>(hi[0]);
    else h = shl_mul<4 - Q>(hi[0]);
    v = lop3_or_and(v, h, dc.himask);
    c = __hsub2(bits_bf16x2(v), bits_bf16x2(0x43104310u));  // 144
  } else if constexpr (BITS == 6) {
    constexpr int r = Q & 7;
    uint32_t h;
    if constexpr (2 * r >= 4) h = shr_mul<2 * r - 4>(hi[Q >> 3]);
    else h = shl_mul<4 - 2 * r>(hi[Q >> 3]);
    v = lop3_or_and(v, h, dc.himask);
    c = __hsub2(bits_bf16x2(v), bits_bf16x2(0x43204320u));  // 160
  } else {
    const uint32_t vh = lop3_and_or(shr_mul<4 * p>(hi[Q >> 2]), dc.nib, dc.magic);
    // code = 16 * (hi - 8) + lo, every intermediate is a small integer (exact in bf16)
    const __nv_bfloat162 top = __hsub2(bits_bf16x2(vh), bits_bf16x2(0x43084308u));
    const __nv_bfloat162 low = __hsub2(bits_bf16x2(v), bits_bf16x2(kMagic));
    c = __hfma2(top, bits_bf16x2(0x41804180u), low);  // 16.0
  }
  return bf16x2_bits(__hmul2(c, bits_bf16x2(s2)));
}

template <int BITS, int... Q>
__device__ __forceinline__ void decode_all(const uint32_t (&lo)[4], const uint32_t (&hi)[4], const uint32_t (&s2)[8],
                                           uint32_t (&w)[16], const DecodeConsts& dc,
                                           std::integer_sequence<int, Q...>) {
  ((w[Q] = decode_pair<BITS, Q>(lo, hi, s2[Q >> 1], dc)), ...);
}

// lo: the lane's four lo words. hi: the lane's hi words (BqGeom::kHiLaneWords of them are read).
// s2[j]: the scale of column 8 j + g duplicated into both halves of a bf16x2.
template <int BITS>
__device__ __forceinline__ void decode_slab(const uint32_t (&lo)[4], const uint32_t (&hi)[4], const uint32_t (&s2)[8],
                                            uint32_t (&w)[16], const DecodeConsts& dc) {
  decode_all<BITS>(lo, hi, s2, w, dc, std::make_integer_sequence<int, 16>{});
}

// Half a slab = the lane's pairs of four adjacent columns j = 4 f + j', j' = 0..3, given as lo[0..1] = its lo words
// 2 f, 2 f + 1; hi[] = the matching hi words moved to the front (5 bit: the word shifted right by 8 f; 6 bit: word
// f; 8 bit: words 2 f, 2 f + 1); s2[0..3] = the four columns' scales. decode_fragment<F> decodes the pairs of
// columns j' = 2 F, 2 F + 1 in the register order of an mma.m16n8k16 A fragment:
// a0 = (row g, k 2t..) a1 = (row g + 8, k 2t..) a2 = (row g, k 2t + 8..) a3 = (row g + 8, k 2t + 8..).
template <int BITS, int F>
__device__ __forceinline__ void decode_fragment(const uint32_t (&lo)[4], const uint32_t (&hi)[4], const uint32_t (&s2)[8],
                                                const DecodeConsts& dc, uint32_t& a0, uint32_t& a1, uint32_t& a2,
                                                uint32_t& a3) {
  a0 = decode_pair<BITS, 4 * F + 0>(lo, hi, s2[2 * F], dc);
  a2 = decode_pair<BITS, 4 * F + 1>(lo, hi, s2[2 * F], dc);
  a1 = decode_pair<BITS, 4 * F + 2>(lo, hi, s2[2 * F + 1], dc);
  a3 = decode_pair<BITS, 4 * F + 3>(lo, hi, s2[2 * F + 1], dc);
}

// Expands the lane's eight scales (one 16-byte read: columns 8 j + g, j = 0..7) into duplicated pairs.
__device__ __forceinline__ void expand_scales(const uint4& sv, uint32_t (&s2)[8]) {
  const uint32_t words[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    s2[2 * i] = __byte_perm(words[i], 0, 0x1010);
    s2[2 * i + 1] = __byte_perm(words[i], 0, 0x3232);
  }
}

}  // namespace q38
