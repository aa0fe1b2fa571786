// Full-attention layers: fused q/k-norm + partial RoPE + KV quantise + paged append, split-KV GQA
// flash-decoding with the merge + sigmoid output gate, and chunked-prefill causal attention over the
// paged int8 / bf16 KV cache.
//
// Replaces kernels::qk_norm_rope_append, attention_decode(+_splits) and attention_prefill of the
// reference (src/kernels/kernels.h:140-179; src/kernels/qk_norm_rope.cu, attention_decode.cu,
// attention_prefill.cu). Page layout per (layer, page): K [kv_head][64][256], V same, then (int8) fp16
// scales K [kv_head][64][4], V same (reference docs/FORMAT.md 3.1).
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "host_util.h"

namespace q38 {
namespace {

constexpr int kHd = Q38_HEAD_DIM;
constexpr int kPage = Q38_PAGE_TOKENS;

struct KvView {
  uint8_t* pool;
  int int8;
  int kv_heads;
  int num_pages;
  size_t page_bytes;
  size_t layer_stride;
  const int* block_table;
  int max_pages_per_seq;

  __device__ __forceinline__ size_t elem() const { return int8 ? 1 : 2; }
  __device__ __forceinline__ size_t k_off(int head, int tok) const { return ((size_t)head * kPage + tok) * kHd * elem(); }
  __device__ __forceinline__ size_t v_off(int head, int tok) const {
    return (size_t)kv_heads * kPage * kHd * elem() + k_off(head, tok);
  }
  __device__ __forceinline__ size_t ks_off(int head, int tok) const {
    return 2 * (size_t)kv_heads * kPage * kHd + ((size_t)head * kPage + tok) * 8;
  }
  __device__ __forceinline__ size_t vs_off(int head, int tok) const {
    return ks_off(head, tok) + (size_t)kv_heads * kPage * 8;
  }
  // base of the (layer, page) block holding position `pos` of `slot`; nullptr if the table entry is invalid
  __device__ __forceinline__ uint8_t* page_of(int layer, int slot, int pos) const {
    const int page = block_table[(size_t)slot * max_pages_per_seq + pos / kPage];
    if (page < 0 || page >= num_pages) return nullptr;
    return pool + (size_t)layer * layer_stride + (size_t)page * page_bytes;
  }
};

KvView make_view(const q38_kv_cache_desc& d) {
  KvView v;
  v.pool = d.pool;
  v.int8 = d.dtype == Q38_KV_INT8;
  v.kv_heads = d.kv_heads;
  v.num_pages = d.num_pages;
  v.page_bytes = d.page_bytes;
  v.layer_stride = d.layer_stride;
  v.block_table = d.block_table;
  v.max_pages_per_seq = d.max_pages_per_seq;
  return v;
}

struct RopeTable {
  float inv_freq[32];  // evaluated on the host exactly as the CPU oracle does (src/ref/ops.cpp:104)
};

// ---------------------------------------------------------------------------------------------------
// qk_norm_rope_append: one CTA per token, one warp per head (nq query heads, nkv key heads, nkv value
// heads); a lane owns 8 consecutive dims. Rounding points (reference src/kernels/qk_norm_rope.cu:38-89,
// oracle src/ref/ops.cpp:79-142): q -> fp16; K (after norm + RoPE) and V (raw) -> int8 with one fp16
// scale = amax / 127 per 64 dims, q = clamp(rint(x / scale), +-127); or bf16.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ proj, int ld_proj,
                                                            const float* __restrict__ q_norm,
                                                            const float* __restrict__ k_norm, float eps, int nq, int nkv,
                                                            __half* __restrict__ q_out, int layer, RopeTable rope,
                                                            const int* __restrict__ tok_pos,
                                                            const int* __restrict__ tok_seq,
                                                            const int* __restrict__ seq_slot, KvView kv) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= nq + 2 * nkv) return;
  const int pos = tok_pos[m];
  const bool is_q = warp < nq, is_k = !is_q && warp < nq + nkv;
  const int head = is_q ? warp : is_k ? warp - nq : warp - nq - nkv;
  const size_t col = is_q ? (size_t)head * kHd : is_k ? (size_t)(2 * nq + head) * kHd : (size_t)(2 * nq + nkv + head) * kHd;
  const uint4 raw = *reinterpret_cast<const uint4*>(proj + (size_t)m * ld_proj + col + 8 * lane);
  const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float x[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __low2float(rp[i]);
    x[2 * i + 1] = __high2float(rp[i]);
  }
  if (is_q || is_k) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / float(kHd) + eps);
    const float* w = (is_q ? q_norm : k_norm) + 8 * lane;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = x[i] * r * w[i];
    // partial RoPE on dims (i, i + 32), i < 32: lanes 0-3 hold dims 0..31, lanes 4-7 hold dims 32..63
    float other[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], 4);
    if (lane < 8) {
      const bool low = lane < 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int fi = 8 * (lane & 3) + i;
        const float angle = float(pos) * rope.inv_freq[fi];
        const float c = cosf(angle), s = sinf(angle);
        // low half: x1 c - x2 s ; high half: x2 c + x1 s
        x[i] = low ? x[i] * c - other[i] * s : x[i] * c + other[i] * s;
      }
    }
  }
  if (is_q) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(q_out + ((size_t)m * nq + head) * kHd + 8 * lane) = *reinterpret_cast<uint4*>(h);
    return;
  }
  const int slot = seq_slot[tok_seq[m]];
  uint8_t* page = kv.page_of(layer, slot, pos);
  if (page == nullptr) {
    report_error(0x201);
    return;
  }
  const int tok = pos % kPage;
  if (kv.int8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    // one scale per 64 dims = 8 lanes
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const __half sh = __float2half_rn(amax / 127.0f);
    const float scale = __half2float(sh);
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float q = 0.0f;
      if (scale > 0.0f) q = fminf(fmaxf(rintf(x[i] / scale), -127.0f), 127.0f);
      packed[i >> 2] |= (uint32_t(int(q)) & 255u) << (8 * (i & 3));
    }
    uint8_t* dst = page + (is_k ? kv.k_off(head, tok) : kv.v_off(head, tok)) + 8 * lane;
    *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
    if ((lane & 7) == 0) {
      uint8_t* sdst = page + (is_k ? kv.ks_off(head, tok) : kv.vs_off(head, tok)) + 2 * (lane >> 3);
      *reinterpret_cast<__half*>(sdst) = sh;
    }
  } else {
    __nv_bfloat162 b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    uint8_t* dst = page + (is_k ? kv.k_off(head, tok) : kv.v_off(head, tok)) + 16 * lane;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(b);
  }
}

// ---------------------------------------------------------------------------------------------------
// Token attention (generic path): one CTA per (split, kv head, row). A row is one query token with its
// causal length L; the GROUP query heads of the kv head share every K/V byte read. Warps stride over
// the keys of the split, a lane owns 8 dims; online softmax in the log2 domain; the warps' states are
// merged through shared memory. With num_splits == 1 the CTA normalises, applies the sigmoid gate and
// writes bf16 itself; otherwise it writes (acc[256], m, l) per head to the scratch for the merge kernel.
// Serves decode (row = sequence, L = pos0 + 1) and, as the first prefill implementation, every prompt
// token of a chunk (row = token, L = pos + 1).
// ---------------------------------------------------------------------------------------------------
constexpr int kAttnWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

template <int GROUP, bool INT8>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_token_kernel(
    const __half* __restrict__ q, const __nv_bfloat16* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ out,
    int nq, int layer, float* __restrict__ scratch, int max_splits, int num_splits, int decode_rows,
    const int* __restrict__ seq_start, const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, KvView kv) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int m, slot, L;
  if (decode_rows) {
    m = seq_start[row];
    slot = seq_slot[row];
    L = seq_pos0[row] + 1;
  } else {
    m = row;
    slot = seq_slot[tok_seq[row]];
    L = tok_pos[row] + 1;
  }
  // keys of this split (whole pages except possibly the last)
  const int pages = (L + kPage - 1) / kPage;
  const int pages_per_split = (pages + num_splits - 1) / num_splits;
  const int t0 = min(L, split * pages_per_split * kPage), t1 = min(L, (split + 1) * pages_per_split * kPage);

  float qv[GROUP][8];
#pragma unroll
  for (int h = 0; h < GROUP; ++h) {
    const uint4 raw = *reinterpret_cast<const uint4*>(q + ((size_t)m * nq + kvh * GROUP + h) * kHd + 8 * lane);
    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(hp[i]);
      qv[h][2 * i] = f.x * (kLog2e / 16.0f);  // 1 / sqrt(256), log2 domain
      qv[h][2 * i + 1] = f.y * (kLog2e / 16.0f);
    }
  }
  float mx[GROUP], l[GROUP], acc[GROUP][8];
#pragma unroll
  for (int h = 0; h < GROUP; ++h) {
    mx[h] = -INFINITY;
    l[h] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;
  }

  for (int t = t0 + warp; t < t1; t += kAttnWarps) {
    const uint8_t* page = kv.page_of(layer, slot, t);
    if (page == nullptr) {
      report_error(0x202);
      break;
    }
    const int tok = t % kPage;
    float kx[8], vx[8];
    if constexpr (INT8) {
      const uint2 kr = *reinterpret_cast<const uint2*>(page + kv.k_off(kvh, tok) + 8 * lane);
      const uint2 vr = *reinterpret_cast<const uint2*>(page + kv.v_off(kvh, tok) + 8 * lane);
      const float ks = __half2float(*reinterpret_cast<const __half*>(page + kv.ks_off(kvh, tok) + 2 * (lane >> 3)));
      const float vs = __half2float(*reinterpret_cast<const __half*>(page + kv.vs_off(kvh, tok) + 2 * (lane >> 3)));
      const uint32_t kw[2] = {kr.x, kr.y}, vw[2] = {vr.x, vr.y};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        kx[i] = float(int8_t(kw[i >> 2] >> (8 * (i & 3)))) * ks;
        vx[i] = float(int8_t(vw[i >> 2] >> (8 * (i & 3)))) * vs;
      }
    } else {
      const uint4 kr = *reinterpret_cast<const uint4*>(page + kv.k_off(kvh, tok) + 16 * lane);
      const uint4 vr = *reinterpret_cast<const uint4*>(page + kv.v_off(kvh, tok) + 16 * lane);
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr);
      const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vr);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kx[2 * i] = __low2float(kp[i]);
        kx[2 * i + 1] = __high2float(kp[i]);
        vx[2 * i] = __low2float(vp[i]);
        vx[2 * i + 1] = __high2float(vp[i]);
      }
    }
#pragma unroll
    for (int h = 0; h < GROUP; ++h) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += qv[h][i] * kx[i];
      s = warp_sum(s);
      const float mn = fmaxf(mx[h], s);
      const float corr = exp2f(mx[h] - mn), p = exp2f(s - mn);
      mx[h] = mn;
      l[h] = l[h] * corr + p;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = acc[h][i] * corr + p * vx[i];
    }
  }

  // merge the warps' states: shared [warp][GROUP][256 + 2]
  __shared__ float sm_acc[kAttnWarps][GROUP][kHd];
  __shared__ float sm_ml[kAttnWarps][GROUP][2];
#pragma unroll
  for (int h = 0; h < GROUP; ++h) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[warp][h][8 * lane + i] = acc[h][i];
    if (lane == 0) {
      sm_ml[warp][h][0] = mx[h];
      sm_ml[warp][h][1] = l[h];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GROUP * kHd; idx += kAttnWarps * 32) {
    const int h = idx / kHd, d = idx % kHd;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm_ml[w][h][0]);
    float ll = 0.0f, a = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
      ll += sm_ml[w][h][1] * c;
      a += sm_acc[w][h][d] * c;
    }
    const int qh = kvh * GROUP + h;
    if (num_splits == 1) {
      const float g = __bfloat162float(gate[(size_t)m * ld_gate + (size_t)qh * kHd + d]);
      out[(size_t)m * nq * kHd + (size_t)qh * kHd + d] = __float2bfloat16_rn(a / ll * sigmoid_f(g));
    } else {
      float* dst = scratch + (((size_t)row * nq + qh) * max_splits + split) * (kHd + 2);
      dst[d] = a;
      if (d == 0) {
        dst[kHd] = mm;
        dst[kHd + 1] = ll;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
#ifndef Q38_ATTN_MIN_PAGES_PER_SPLIT
#define Q38_ATTN_MIN_PAGES_PER_SPLIT 8
#endif
constexpr int kMinPagesPerSplit = Q38_ATTN_MIN_PAGES_PER_SPLIT;  // 64-token pages

// Decode attention over int8 KV on tensor cores: one CTA per (split, kv head, sequence), two CTAs per SM.
//   * a producer lane walks the sequence's block-table row and brings one (page, kv head) per stage with four
//     1-D bulk copies: K 16 KB, V 16 KB and their two 512-byte scale rows are each contiguous in the page;
//   * each of the 4 consumer warps owns 16 of the page's 64 tokens. S = K Q^T runs as m16n8k16 f16 MMAs with the
//     tokens as rows and the (<= 8) query heads of the kv head as the 8 columns; the int8 bytes become exact
//     fp16 integers in registers (byte permute into 0x64xx = 1024 + x, minus 1152), and the per-(token, 64-dim)
//     K scale multiplies each 64-dim partial sum in fp32. The order of dims inside an MMA k-step is permuted
//     so that a lane reads 16 contiguous bytes per token (Q fragments use the same permutation);
//   * online softmax in the log2 domain on the accumulator fragments; P is scaled by the V scales, cast to
//     fp16 and transposed in registers (movmatrix) to become the B operand of O^T = V^T P^T, whose A operand
//     pairs two tokens of one dim (bytes of two V rows permuted together);
//   * the warps' (m, l, O) are merged through shared memory; a single split finishes in place (normalise,
//     sigmoid gate, bf16), otherwise the state goes to the scratch for attn_merge_kernel.
// K/V bytes are read from HBM exactly once per GQA group (reference design point: attention_decode.cu).
// ---------------------------------------------------------------------------------------------------
constexpr int kMmaWarps = 4;
constexpr int kMmaThreads = (kMmaWarps + 1) * 32;
constexpr int kMmaStages = 3;
constexpr int kStageK = 0, kStageV = 16384, kStageKs = 32768, kStageVs = 33280, kStageBytes = 33792;
constexpr int kMmaSmem = kMmaStages * kStageBytes + 256;

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// two biased bytes (x + 128) of one word -> half2 (x0, x1)
template <int SEL>
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t w) {
  const uint32_t h = __byte_perm(w, 0x64646464u, SEL);
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half(0x6480)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// byte I of two words -> half2 (wa.byte, wb.byte)
template <int I>
__device__ __forceinline__ uint32_t byte_pair_to_half2(uint32_t wa, uint32_t wb) {
  constexpr uint32_t sel = I | (I << 4) | ((4 + I) << 8) | (I << 12);
  const uint32_t h = (__byte_perm(wa, wb, sel) & 0x00FF00FFu) | 0x64006400u;
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half(0x6480)));
  return *reinterpret_cast<const uint32_t*>(&r);
}

__global__ void __launch_bounds__(kMmaThreads, 2) attn_decode_mma_kernel(
    const __half* __restrict__ q, const __nv_bfloat16* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ out,
    int nq, int group, int layer, float* __restrict__ scratch, int max_splits, int num_splits, int decode_rows,
    const int* __restrict__ seq_start, const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, KvView kv) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  extern __shared__ __align__(128) uint8_t dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm + kMmaStages * kStageBytes);
  uint64_t* empty = full + kMmaStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMmaStages);
  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // a row is a sequence's single new token (decode) or one prompt token of a chunk with its causal length (prefill)
  const int m = decode_rows ? seq_start[row] : row;
  const int slot = decode_rows ? seq_slot[row] : seq_slot[tok_seq[row]];
  const int L = (decode_rows ? seq_pos0[row] : tok_pos[row]) + 1;
  const int pages = (L + kPage - 1) / kPage;
  // a split takes at least kMinPagesPerSplit pages: a short sequence of a ragged batch uses fewer of the launch's
  // splits (the others leave at once) instead of paying a CTA's fixed cost for one or two pages
  const int pages_per_split = max(kMinPagesPerSplit, (pages + num_splits - 1) / num_splits);
  const int p0 = min(pages, split * pages_per_split), p1 = min(pages, (split + 1) * pages_per_split);
  if (p0 >= p1 && num_splits > 1) {  // a split beyond this sequence's pages: an empty state for the merge, nothing else
    if (tid < group) {
      float* dst = scratch + (((size_t)row * nq + (size_t)kvh * group + tid) * max_splits + split) * (kHd + 2);
      dst[kHd] = -INFINITY;
      dst[kHd + 1] = 0.0f;
    }
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < kMmaStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kMmaWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kMmaWarps) {
    if (lane == 0) {
      // decode reads every page once; the prompt tokens of a chunk re-read each other's pages out of L2
      const uint64_t pol = decode_rows ? policy_evict_first() : policy_evict_normal();
      const int* table = kv.block_table + (size_t)slot * kv.max_pages_per_seq;
      for (int p = p0, it = 0; p < p1; ++p, ++it) {
        const int s = it % kMmaStages;
        if (*abort_flag || !mbar_wait(&empty[s], ((it / kMmaStages) & 1) ^ 1, 0x211)) {
          *abort_flag = 1;
          break;
        }
        const int page = table[p];
        if (page < 0 || page >= kv.num_pages) {
          report_error(0x212);
          *abort_flag = 1;
          break;
        }
        const uint8_t* base = kv.pool + (size_t)layer * kv.layer_stride + (size_t)page * kv.page_bytes;
        uint8_t* st = dsm + (size_t)s * kStageBytes;
        mbar_expect_tx(&full[s], 2 * 16384 + 2 * 512);
        bulk_g2s(st + kStageK, base + kv.k_off(kvh, 0), 16384, &full[s], pol);
        bulk_g2s(st + kStageV, base + kv.v_off(kvh, 0), 16384, &full[s], pol);
        bulk_g2s(st + kStageKs, base + kv.ks_off(kvh, 0), 512, &full[s], pol);
        bulk_g2s(st + kStageVs, base + kv.vs_off(kvh, 0), 512, &full[s], pol);
      }
    }
    return;
  }

  const int g = lane >> 2, t = lane & 3;
  // Q fragments: head g of the group, dims 64 grp + 16 t + 4 s + {0..3}
  uint32_t qf[4][4][2];
  {
    const bool live = g < group;
    const __half* qrow = q + ((size_t)m * nq + (size_t)kvh * group + (live ? g : 0)) * kHd;
#pragma unroll
    for (int grp = 0; grp < 4; ++grp)
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint2 v = *reinterpret_cast<const uint2*>(qrow + 64 * grp + 16 * t + 4 * s);
        qf[grp][s][0] = live ? v.x : 0u;
        qf[grp][s][1] = live ? v.y : 0u;
      }
  }
  float o[16][4];
#pragma unroll
  for (int T = 0; T < 16; ++T)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[T][c] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // heads 2t and 2t + 1
  constexpr float kScale = kLog2e / 16.0f;

  for (int p = p0, it = 0; p < p1; ++p, ++it) {
    const int s = it % kMmaStages;
    bool ok = !*abort_flag && mbar_wait(&full[s], (it / kMmaStages) & 1, 0x213);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) *abort_flag = 1;
    const int tok0 = 16 * warp, tbase = p * kPage + tok0;
    if (ok && tbase < L) {
      const uint8_t* st = dsm + (size_t)s * kStageBytes;
      const uint8_t* Ks = st + kStageK + (size_t)tok0 * kHd;
      const uint8_t* Vs = st + kStageV + (size_t)tok0 * kHd;
      const __half* Ksc = reinterpret_cast<const __half*>(st + kStageKs) + tok0 * 4;
      const __half* Vsc = reinterpret_cast<const __half*>(st + kStageVs) + tok0 * 4;
      // ---- S = K Q^T ----
      float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint4 ka = *reinterpret_cast<const uint4*>(Ks + g * kHd + 64 * grp + 16 * t);
        const uint4 kb = *reinterpret_cast<const uint4*>(Ks + (g + 8) * kHd + 64 * grp + 16 * t);
        const uint32_t wa[4] = {ka.x ^ 0x80808080u, ka.y ^ 0x80808080u, ka.z ^ 0x80808080u, ka.w ^ 0x80808080u};
        const uint32_t wb[4] = {kb.x ^ 0x80808080u, kb.y ^ 0x80808080u, kb.z ^ 0x80808080u, kb.w ^ 0x80808080u};
        float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int ss = 0; ss < 4; ++ss)
          mma_f16_16816(d, bytes_to_half2<0x4140>(wa[ss]), bytes_to_half2<0x4140>(wb[ss]),
                        bytes_to_half2<0x4342>(wa[ss]), bytes_to_half2<0x4342>(wb[ss]), qf[grp][ss][0], qf[grp][ss][1]);
        const float ksa = __half2float(Ksc[g * 4 + grp]), ksb = __half2float(Ksc[(g + 8) * 4 + grp]);
        sacc[0] += ksa * d[0];
        sacc[1] += ksa * d[1];
        sacc[2] += ksb * d[2];
        sacc[3] += ksb * d[3];
      }
      // ---- online softmax over the block's 16 tokens ----
      const bool va = tbase + g < L, vb = tbase + g + 8 < L;
      const float s0 = va ? sacc[0] * kScale : -INFINITY, s1 = va ? sacc[1] * kScale : -INFINITY;
      const float s2 = vb ? sacc[2] * kScale : -INFINITY, s3 = vb ? sacc[3] * kScale : -INFINITY;
      float bm0 = fmaxf(s0, s2), bm1 = fmaxf(s1, s3);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, off));
        bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, off));
      }
      const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
      const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
      const float pr0 = exp2f(s0 - mn0), pr1 = exp2f(s1 - mn1), pr2 = exp2f(s2 - mn0), pr3 = exp2f(s3 - mn1);
      float ls0 = pr0 + pr2, ls1 = pr1 + pr3;
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, off);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, off);
      }
      m0 = mn0;
      m1 = mn1;
      l0 = l0 * c0 + ls0;
      l1 = l1 * c1 + ls1;
#pragma unroll
      for (int T = 0; T < 16; ++T) {
        o[T][0] *= c0;
        o[T][1] *= c1;
        o[T][2] *= c0;
        o[T][3] *= c1;
      }
      // ---- O^T += V^T P^T ----
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const float vsa = __half2float(Vsc[g * 4 + grp]), vsb = __half2float(Vsc[(g + 8) * 4 + grp]);
        const __half2 pa = __floats2half2_rn(pr0 * vsa, pr1 * vsa), pb = __floats2half2_rn(pr2 * vsb, pr3 * vsb);
        const uint32_t b0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&pa));
        const uint32_t b1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&pb));
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int J = 2 * grp + jj;
          const uint8_t* vp = Vs + 32 * J + 4 * g;
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vp + (2 * t) * kHd) ^ 0x80808080u;
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vp + (2 * t + 1) * kHd) ^ 0x80808080u;
          const uint32_t w2 = *reinterpret_cast<const uint32_t*>(vp + (2 * t + 8) * kHd) ^ 0x80808080u;
          const uint32_t w3 = *reinterpret_cast<const uint32_t*>(vp + (2 * t + 9) * kHd) ^ 0x80808080u;
          mma_f16_16816(o[2 * J], byte_pair_to_half2<0>(w0, w1), byte_pair_to_half2<1>(w0, w1),
                        byte_pair_to_half2<0>(w2, w3), byte_pair_to_half2<1>(w2, w3), b0, b1);
          mma_f16_16816(o[2 * J + 1], byte_pair_to_half2<2>(w0, w1), byte_pair_to_half2<3>(w0, w1),
                        byte_pair_to_half2<2>(w2, w3), byte_pair_to_half2<3>(w2, w3), b0, b1);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // ---- merge the four warps (shared memory aliases the drained stages) ----
  named_bar_sync(1, kMmaWarps * 32);
  float* sm_acc = reinterpret_cast<float*>(dsm);                       // [warp][8 heads][256]
  float* sm_ml = sm_acc + kMmaWarps * 8 * kHd;                         // [warp][8 heads][2]
#pragma unroll
  for (int T = 0; T < 16; ++T)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int dim = 32 * (T >> 1) + 4 * g + 2 * (T & 1) + (c >> 1);
      const int head = 2 * t + (c & 1);
      sm_acc[((size_t)warp * 8 + head) * kHd + dim] = o[T][c];
    }
  if (g == 0) {
    sm_ml[(warp * 8 + 2 * t) * 2] = m0;
    sm_ml[(warp * 8 + 2 * t) * 2 + 1] = l0;
    sm_ml[(warp * 8 + 2 * t + 1) * 2] = m1;
    sm_ml[(warp * 8 + 2 * t + 1) * 2 + 1] = l1;
  }
  named_bar_sync(1, kMmaWarps * 32);
  for (int idx = tid; idx < group * kHd; idx += kMmaWarps * 32) {
    const int h = idx / kHd, d = idx % kHd;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mm = fmaxf(mm, sm_ml[(w * 8 + h) * 2]);
    float ll = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float mw = sm_ml[(w * 8 + h) * 2];
      const float c = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
      ll += sm_ml[(w * 8 + h) * 2 + 1] * c;
      acc += sm_acc[((size_t)w * 8 + h) * kHd + d] * c;
    }
    const int qh = kvh * group + h;
    if (num_splits == 1) {
      const float gt = __bfloat162float(gate[(size_t)m * ld_gate + (size_t)qh * kHd + d]);
      out[(size_t)m * nq * kHd + (size_t)qh * kHd + d] = __float2bfloat16_rn(acc / ll * sigmoid_f(gt));
    } else {
      float* dst = scratch + (((size_t)row * nq + qh) * max_splits + split) * (kHd + 2);
      dst[d] = acc;
      if (d == 0) {
        dst[kHd] = mm;
        dst[kHd + 1] = ll;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Chunked-prefill attention over int8 pages, query-tiled (flash attention 2 on the tensor cores).
// Replaces the reference's attention_prefill kernel (src/kernels/attention_prefill.cu:154-313) for int8 KV.
//
// One CTA per (KV split, kv head, tile of `tq` consecutive prompt tokens of one sequence). The tile's rows are its
// (token, query head of the kv head's group) pairs, at most 128 = eight warps of 16 rows (eight warps are two per
// scheduler, which leaves each thread the full 255 registers for the 16 x 256 fp32 output block it carries). Thread 0
// streams the (page, kv head) blocks of the keys the tile may see (causal: positions 0 .. last token of the tile)
// through a two-stage shared-memory ring with the same four bulk copies per page as the decode kernel: two pages up
// front, then the page after next as soon as a stage has been converted. Every K / V byte is fetched once per tile
// instead of once per prompt token and query row.
// Per page the eight warps first turn the raw block into fp16 tiles K, V [64 keys][256] in shared memory, each element
// fp16(int8) * fp16(scale of its key and 64-dim group) - the rounding of the reference's prefill kernel - once for
// the whole tile (the raw stage goes back to the producer at that point); then every warp runs S = Q K^T for its 16
// rows (Q fragments by ldmatrix from the staged fp16 query rows, K fragments by ldmatrix), the online softmax in the
// log2 domain on the accumulator fragments (the O accumulator is rescaled only when a row maximum of the warp
// moved), and O += P V with P straight from the S registers and V by transposing ldmatrix. Keys beyond a row's
// position are masked; pages entirely beyond a warp's last position cost it nothing but the two barriers. A single
// split normalises, applies the sigmoid output gate and writes bf16; with several splits the (O, m, l) states go to
// the scratch for attn_merge_kernel.
// ---------------------------------------------------------------------------------------------------
constexpr int kPfWarps = 8;
constexpr int kPfRows = kPfWarps * 16;
constexpr int kPfConsumers = kPfWarps * 32;
constexpr int kPfThreads = kPfConsumers;
constexpr int kPfStages = 2;
constexpr int kPfHStride = 2 * kHd + 16;       // bytes per fp16 row of the K / V / Q tiles: 16 mod 128, ldmatrix rows on distinct banks
constexpr int kPfOStride = kHd + 4;            // floats per staged output row
constexpr int kPfRingBytes = kPfStages * kStageBytes;
constexpr int kPfTileBytes = kPage * kPfHStride;
constexpr int kPfKhOff = kPfRingBytes, kPfVhOff = kPfKhOff + kPfTileBytes, kPfQOff = kPfVhOff + kPfTileBytes;
constexpr int kPfBarOff = kPfQOff + kPfRows * kPfHStride;
static_assert(kPfRows * kPfOStride * 4 <= kPfQOff, "the output staging aliases the ring and the K / V tiles");
constexpr int kPfSmem = kPfBarOff + 256;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 16 int8 values (one 16-byte word group, biased by the caller's XOR) -> 16 fp16 values times `scale`, stored as 32 bytes
__device__ __forceinline__ void dequant16_to_half(const uint4& raw, __half scale, uint8_t* dst) {
  const __half2 sc = __half2half2(scale);
  const uint32_t w[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
  uint32_t outw[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = bytes_to_half2<0x4140>(w[i]), hi = bytes_to_half2<0x4342>(w[i]);
    const __half2 a = __hmul2(*reinterpret_cast<const __half2*>(&lo), sc);
    const __half2 b = __hmul2(*reinterpret_cast<const __half2*>(&hi), sc);
    outw[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
    outw[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
  *reinterpret_cast<uint4*>(dst + 16) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
}

// 8 bf16 values (16 bytes) -> 8 fp16 values (exact for every magnitude an fp16 holds; K and V rows are O(1))
__device__ __forceinline__ uint4 bf16x8_to_half(const uint4& raw) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    o[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// kInt8: int8 pages with fp16 scales, brought in by bulk copies through the raw ring and dequantised; otherwise bf16
// pages, read with plain 16-byte loads and converted on the way into the same fp16 tiles (no ring: this is not the
// benchmarked cache type, the loads of a page are simply exposed).
template <bool kInt8>
__global__ void __launch_bounds__(kPfThreads, 1) attn_prefill_tile_kernel(
    const __half* __restrict__ q, const __nv_bfloat16* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ out,
    int nq, int group, int layer, int tq, int tiles_per_seq, float* __restrict__ scratch, int max_splits, int num_splits,
    const int* __restrict__ seq_start, const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0, KvView kv) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  extern __shared__ __align__(128) uint8_t dsm[];
  uint8_t* Kh = dsm + kPfKhOff;
  uint8_t* Vh = dsm + kPfVhOff;
  uint8_t* qs = dsm + kPfQOff;
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm + kPfBarOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(full + kPfStages);
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int b = blockIdx.z / tiles_per_seq, ti = blockIdx.z % tiles_per_seq;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s_first = seq_start[b], n_seq = seq_start[b + 1] - s_first;
  const int i0 = ti * tq;
  if (i0 >= n_seq) return;                       // this sequence's chunk has fewer tiles
  const int nt = min(tq, n_seq - i0);            // tokens of the tile
  const int rows = nt * group;                   // (token, head) rows, <= 128
  const int m0 = s_first + i0;                   // first token row of the tile in the step's arrays
  const int pos0 = seq_pos0[b] + i0;             // its position; row r sees keys 0 .. pos0 + r / group
  const int slot = seq_slot[b];
  const int L = pos0 + nt;
  const int pages = (L + kPage - 1) / kPage;
  const int pages_per_split = (pages + num_splits - 1) / num_splits;
  const int p0 = min(pages, split * pages_per_split), p1 = min(pages, (split + 1) * pages_per_split);
  if (p0 >= p1) {  // (only with several splits) nothing to do here: empty states for the merge
    for (int r = tid; r < rows; r += kPfThreads) {
      float* dst = scratch + (((size_t)(m0 + r / group) * nq + (size_t)kvh * group + r % group) * max_splits + split) * (kHd + 2);
      dst[kHd] = -INFINITY;
      dst[kHd + 1] = 0.0f;
    }
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < kPfStages; ++s) mbar_init(&full[s], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  // Requests page p of the tile's key range into ring stage `s` (thread 0 only; the stage must be free).
  auto request_page = [&](int p, int s) {
    const int page = kv.block_table[(size_t)slot * kv.max_pages_per_seq + p];
    if (page < 0 || page >= kv.num_pages) {
      report_error(0x222);
      *abort_flag = 1;
      return;
    }
    const uint64_t pol = policy_evict_normal();  // the tiles of a chunk share their pages through L2
    const uint8_t* base = kv.pool + (size_t)layer * kv.layer_stride + (size_t)page * kv.page_bytes;
    uint8_t* st = dsm + (size_t)s * kStageBytes;
    mbar_expect_tx(&full[s], 2 * 16384 + 2 * 512);
    bulk_g2s(st + kStageK, base + kv.k_off(kvh, 0), 16384, &full[s], pol);
    bulk_g2s(st + kStageV, base + kv.v_off(kvh, 0), 16384, &full[s], pol);
    bulk_g2s(st + kStageKs, base + kv.ks_off(kvh, 0), 512, &full[s], pol);
    bulk_g2s(st + kStageVs, base + kv.vs_off(kvh, 0), 512, &full[s], pol);
  };
  // stage the tile's query rows (fp16), zero rows beyond the tile
  for (int i = tid; i < kPfRows * (kHd / 8); i += kPfThreads) {
    const int r = i / (kHd / 8), c = i % (kHd / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows)
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(m0 + r / group) * nq + (size_t)kvh * group + r % group) * kHd + 8 * c);
    *reinterpret_cast<uint4*>(qs + (size_t)r * kPfHStride + 16 * c) = v;
  }
  __syncthreads();

  if (kInt8 && tid == 0) {  // barriers are initialised (the __syncthreads above): the first two pages
    request_page(p0, 0);
    if (p0 + 1 < p1) request_page(p0 + 1, 1);
  }

  const int g = lane >> 2, t = lane & 3;
  const int ra = 16 * warp + g, rb = ra + 8;                   // this lane's two rows of the tile
  const bool warp_live = 16 * warp < rows;
  const int pos_a = ra < rows ? pos0 + ra / group : -1;        // last key position a row may see (-1: padding row)
  const int pos_b = rb < rows ? pos0 + rb / group : -1;
  const int warp_first = pos0 + (16 * warp) / group;           // smallest / largest position among the warp's rows
  const int warp_last = pos0 + (min(rows, 16 * warp + 16) - 1) / group;
  // ldmatrix lane addresses: Q A-fragments (rows 16 w + (lane & 15), dims + 8 (lane >> 4)); K fragments (keys
  // 8 (mi >> 1) + (lane & 7), dims + 8 (mi & 1), mi = lane >> 3); V fragments transposed (keys 8 (mi & 1) + .., dims + 8 (mi >> 1))
  const int mi = lane >> 3;
  const uint32_t q_addr = smem_u32(qs) + (uint32_t)(16 * warp + (lane & 15)) * kPfHStride + 16u * (lane >> 4);
  const uint32_t k_addr = smem_u32(Kh) + (uint32_t)(8 * (mi >> 1) + (lane & 7)) * kPfHStride + 16u * (mi & 1);
  const uint32_t v_addr = smem_u32(Vh) + (uint32_t)(8 * (mi & 1) + (lane & 7)) * kPfHStride + 16u * (mi >> 1);
  float o[32][4];
#pragma unroll
  for (int T = 0; T < 32; ++T)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[T][c] = 0.0f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;  // l: this lane's share of the row sums
  constexpr float kScale = kLog2e / 16.0f;

  for (int p = p0, it = 0; p < p1; ++p, ++it) {
    const int s = it % kPfStages;
    bool ok = !*abort_flag && (!kInt8 || mbar_wait(&full[s], (it / kPfStages) & 1, 0x223));
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) *abort_flag = 1;
    // ---- the page's K and V as fp16 tiles, once for all rows of the tile ----
    if constexpr (!kInt8) {
      if (ok) {
        const int page = kv.block_table[(size_t)slot * kv.max_pages_per_seq + p];  // the same entry in every thread
        if (page < 0 || page >= kv.num_pages) {
          if (tid == 0) report_error(0x222);
          *abort_flag = 1;
          ok = false;
        } else {
          const uint8_t* base = kv.pool + (size_t)layer * kv.layer_stride + (size_t)page * kv.page_bytes;
          const uint8_t* ksrc = base + kv.k_off(kvh, 0);
          const uint8_t* vsrc = base + kv.v_off(kvh, 0);
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int u = tid + kPfConsumers * r;  // 16-byte group: key u / 32, dims 8 (u % 32) ..
            const int key = u >> 5, ch = u & 31;
            uint4 kh = make_uint4(0u, 0u, 0u, 0u), vh = kh;  // positions nobody has written yet stay zero
            if (p * kPage + key < L) {
              kh = bf16x8_to_half(__ldg(reinterpret_cast<const uint4*>(ksrc) + u));
              vh = bf16x8_to_half(__ldg(reinterpret_cast<const uint4*>(vsrc) + u));
            }
            *reinterpret_cast<uint4*>(Kh + (size_t)key * kPfHStride + 16 * ch) = kh;
            *reinterpret_cast<uint4*>(Vh + (size_t)key * kPfHStride + 16 * ch) = vh;
          }
        }
      }
    }
    if (kInt8 && ok) {
      const uint8_t* st = dsm + (size_t)s * kStageBytes;
      const __half* Ksc = reinterpret_cast<const __half*>(st + kStageKs);
      const __half* Vsc = reinterpret_cast<const __half*>(st + kStageVs);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int u = tid + kPfConsumers * r;  // 16-byte group: key u / 16, dims 16 (u % 16) ..
        const int key = u >> 4, ch = u & 15;
        if (p * kPage + key < L) {
          dequant16_to_half(*reinterpret_cast<const uint4*>(st + kStageK + 16 * u), Ksc[key * 4 + (ch >> 2)],
                            Kh + (size_t)key * kPfHStride + 32 * ch);
          dequant16_to_half(*reinterpret_cast<const uint4*>(st + kStageV + 16 * u), Vsc[key * 4 + (ch >> 2)],
                            Vh + (size_t)key * kPfHStride + 32 * ch);
        } else {  // positions nobody has written yet: whatever the page holds must not reach the products (0 x NaN)
          const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(Kh + (size_t)key * kPfHStride + 32 * ch) = zero;
          *reinterpret_cast<uint4*>(Kh + (size_t)key * kPfHStride + 32 * ch + 16) = zero;
          *reinterpret_cast<uint4*>(Vh + (size_t)key * kPfHStride + 32 * ch) = zero;
          *reinterpret_cast<uint4*>(Vh + (size_t)key * kPfHStride + 32 * ch + 16) = zero;
        }
      }
    }
    __syncthreads();  // the fp16 tiles are complete, the raw stage is free: the page after next streams in during the products
    if (kInt8 && tid == 0 && p + kPfStages < p1 && !*abort_flag) request_page(p + kPfStages, s);

    const int kbase = p * kPage;
    if (ok && warp_live && kbase <= warp_last) {
      // ---- S = Q K^T: this warp's 16 rows x 64 keys (8 n-tiles), 16 k-steps of 16 dims ----
      float sacc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[j][c] = 0.0f;
#pragma unroll 4
      for (int kk = 0; kk < 16; ++kk) {
        uint32_t qa[4];
        ldmatrix_x4(qa, q_addr + 32u * kk);
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {  // keys 16 jp .. 16 jp + 15
          uint32_t kb[4];
          ldmatrix_x4(kb, k_addr + (uint32_t)(16 * jp) * kPfHStride + 32u * kk);
          mma_f16_16816(sacc[2 * jp], qa[0], qa[1], qa[2], qa[3], kb[0], kb[1]);
          mma_f16_16816(sacc[2 * jp + 1], qa[0], qa[1], qa[2], qa[3], kb[2], kb[3]);
        }
      }
      // ---- online softmax (log2 domain); keys beyond a row's position are masked on pages that reach that far ----
      const bool need_mask = kbase + kPage - 1 > warp_first;
      float bm_a = -INFINITY, bm_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float v = sacc[j][c] * kScale;
          if (need_mask) {
            const int key = kbase + 8 * j + 2 * t + (c & 1);
            if (key > ((c & 2) ? pos_b : pos_a)) v = -INFINITY;
          }
          sacc[j][c] = v;
          if (c & 2) bm_b = fmaxf(bm_b, v);
          else bm_a = fmaxf(bm_a, v);
        }
      bm_a = fmaxf(bm_a, __shfl_xor_sync(0xffffffffu, bm_a, 1));
      bm_a = fmaxf(bm_a, __shfl_xor_sync(0xffffffffu, bm_a, 2));
      bm_b = fmaxf(bm_b, __shfl_xor_sync(0xffffffffu, bm_b, 1));
      bm_b = fmaxf(bm_b, __shfl_xor_sync(0xffffffffu, bm_b, 2));
      const float mn_a = fmaxf(m_a, bm_a), mn_b = fmaxf(m_b, bm_b);
      const float ref_a = mn_a == -INFINITY ? 0.0f : mn_a, ref_b = mn_b == -INFINITY ? 0.0f : mn_b;  // no inf - inf
      const float c_a = exp2f(m_a - ref_a), c_b = exp2f(m_b - ref_b);
      float ps_a = 0.0f, ps_b = 0.0f;
      uint32_t pf[8][2];  // P as fp16 pairs: [n-tile][rows g / g + 8]
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float e0 = exp2f(sacc[j][0] - ref_a), e1 = exp2f(sacc[j][1] - ref_a);
        const float e2 = exp2f(sacc[j][2] - ref_b), e3 = exp2f(sacc[j][3] - ref_b);
        ps_a += e0 + e1;
        ps_b += e2 + e3;
        const __half2 ha = __floats2half2_rn(e0, e1), hb = __floats2half2_rn(e2, e3);
        pf[j][0] = *reinterpret_cast<const uint32_t*>(&ha);
        pf[j][1] = *reinterpret_cast<const uint32_t*>(&hb);
      }
      l_a = l_a * c_a + ps_a;
      l_b = l_b * c_b + ps_b;
      const bool moved = (m_a != mn_a) || (m_b != mn_b);
      m_a = mn_a;
      m_b = mn_b;
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int T = 0; T < 32; ++T) {
          o[T][0] *= c_a;
          o[T][1] *= c_a;
          o[T][2] *= c_b;
          o[T][3] *= c_b;
        }
      }
      // ---- O += P V: 4 k-steps of 16 keys, 32 n-tiles of 8 dims (two per transposing ldmatrix) ----
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int dp = 0; dp < 16; ++dp) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, v_addr + (uint32_t)(16 * ks) * kPfHStride + 32u * dp);
          mma_f16_16816(o[2 * dp], pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1], vb[0], vb[1]);
          mma_f16_16816(o[2 * dp + 1], pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();  // every warp is through with the fp16 tiles before the next page overwrites them
  }

  // ---- finish: row sums across the four lanes of a row, then through shared memory (ring and tiles are drained) for
  //      coalesced gate reads and stores ----
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  float* os = reinterpret_cast<float*>(dsm);
  const float inv_a = (num_splits == 1 && l_a > 0.0f) ? 1.0f / l_a : 1.0f;
  const float inv_b = (num_splits == 1 && l_b > 0.0f) ? 1.0f / l_b : 1.0f;
#pragma unroll
  for (int T = 0; T < 32; ++T) {
    *reinterpret_cast<float2*>(os + (size_t)ra * kPfOStride + 8 * T + 2 * t) = make_float2(o[T][0] * inv_a, o[T][1] * inv_a);
    *reinterpret_cast<float2*>(os + (size_t)rb * kPfOStride + 8 * T + 2 * t) = make_float2(o[T][2] * inv_b, o[T][3] * inv_b);
  }
  __syncwarp();
  for (int rr = 0; rr < 16; ++rr) {
    const int r = 16 * warp + rr;
    if (r >= rows) break;
    const int m = m0 + r / group, qh = kvh * group + r % group;
    const float4 x0 = *reinterpret_cast<const float4*>(os + (size_t)r * kPfOStride + 8 * lane);
    const float4 x1 = *reinterpret_cast<const float4*>(os + (size_t)r * kPfOStride + 8 * lane + 4);
    const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    if (num_splits == 1) {
      const uint4 graw = *reinterpret_cast<const uint4*>(gate + (size_t)m * ld_gate + (size_t)qh * kHd + 8 * lane);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
      __nv_bfloat162 res[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        res[i] = __floats2bfloat162_rn(x[2 * i] * sigmoid_f(__low2float(gp[i])), x[2 * i + 1] * sigmoid_f(__high2float(gp[i])));
      *reinterpret_cast<uint4*>(out + (size_t)m * nq * kHd + (size_t)qh * kHd + 8 * lane) = *reinterpret_cast<uint4*>(res);
    } else {
      float* dst = scratch + (((size_t)m * nq + qh) * max_splits + split) * (kHd + 2);
      *reinterpret_cast<float2*>(dst + 8 * lane) = make_float2(x[0], x[1]);
      *reinterpret_cast<float2*>(dst + 8 * lane + 2) = make_float2(x[2], x[3]);
      *reinterpret_cast<float2*>(dst + 8 * lane + 4) = make_float2(x[4], x[5]);
      *reinterpret_cast<float2*>(dst + 8 * lane + 6) = make_float2(x[6], x[7]);
      // the row's (m, l) sit in the lanes that own it: rows 16 w + g (first half) and + 8 (second half)
      const float mr = __shfl_sync(0xffffffffu, rr < 8 ? m_a : m_b, 4 * (rr & 7));
      const float lr = __shfl_sync(0xffffffffu, rr < 8 ? l_a : l_b, 4 * (rr & 7));
      if (lane == 0) {
        dst[kHd] = mr;
        dst[kHd + 1] = lr;
      }
    }
  }
}

// Merge of the splits + normalisation + sigmoid gate -> bf16 (reference attention_decode.cu:241-257).
__global__ void __launch_bounds__(kHd) attn_merge_kernel(const float* __restrict__ scratch, int max_splits,
                                                         int num_splits, const __nv_bfloat16* __restrict__ gate,
                                                         int ld_gate, __nv_bfloat16* __restrict__ out, int nq,
                                                         const int* __restrict__ seq_start) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int qh = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  const int m = seq_start ? seq_start[row] : row;  // decode: a sequence's token row; prefill tiles: the token row itself
  const float* base = scratch + ((size_t)row * nq + qh) * max_splits * (kHd + 2);
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, base[(size_t)s * (kHd + 2) + kHd]);
  float ll = 0.0f, a = 0.0f;
  for (int s = 0; s < num_splits; ++s) {
    const float* p = base + (size_t)s * (kHd + 2);
    const float ms = p[kHd];
    if (ms == -INFINITY) continue;  // an empty split: its accumulator row was never written
    const float c = exp2f(ms - mm);
    ll += p[kHd + 1] * c;
    a += p[d] * c;
  }
  const float g = __bfloat162float(gate[(size_t)m * ld_gate + (size_t)qh * kHd + d]);
  out[(size_t)m * nq * kHd + (size_t)qh * kHd + d] = __float2bfloat16_rn(a / ll * sigmoid_f(g));
}

template <int GROUP>
int launch_token_attention(const q38_attention_params& p, const q38_batch_desc& b, const q38_kv_cache_desc& kvd,
                           bool decode, int splits, cudaStream_t s) {
  const KvView kv = make_view(kvd);
  const int rows = decode ? b.num_seqs : b.num_tokens;
  const dim3 grid(splits, p.num_kv_heads, rows);
  const __half* q = reinterpret_cast<const __half*>(p.q);
  const __nv_bfloat16* gate = reinterpret_cast<const __nv_bfloat16*>(p.gate);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
  if (kv.int8)
    (void)launch_kernel(attn_token_kernel<GROUP, true>, dim3(grid), dim3(kAttnWarps * 32), 0, s, 
        q, gate, p.ld_gate, out, p.num_q_heads, p.attn_layer, p.split_scratch, p.max_splits, splits, decode ? 1 : 0,
        b.seq_start, b.seq_slot, b.seq_pos0, b.tok_pos, b.tok_seq, kv);
  else
    (void)launch_kernel(attn_token_kernel<GROUP, false>, dim3(grid), dim3(kAttnWarps * 32), 0, s, 
        q, gate, p.ld_gate, out, p.num_q_heads, p.attn_layer, p.split_scratch, p.max_splits, splits, decode ? 1 : 0,
        b.seq_start, b.seq_slot, b.seq_pos0, b.tok_pos, b.tok_seq, kv);
  Q38_LAUNCH_OK("attn_token_kernel");
  if (splits > 1) {
    (void)launch_kernel(attn_merge_kernel, dim3(p.num_q_heads, rows), dim3(kHd), 0, s, p.split_scratch, p.max_splits, splits, gate, p.ld_gate,
                                                               out, p.num_q_heads, b.seq_start);
    Q38_LAUNCH_OK("attn_merge_kernel");
  }
  return Q38_OK;
}

int dispatch_group(int group, const q38_attention_params& p, const q38_batch_desc& b, const q38_kv_cache_desc& kv,
                   bool decode, int splits, cudaStream_t s) {
  switch (group) {
    case 1: return launch_token_attention<1>(p, b, kv, decode, splits, s);
    case 2: return launch_token_attention<2>(p, b, kv, decode, splits, s);
    case 3: return launch_token_attention<3>(p, b, kv, decode, splits, s);
    case 4: return launch_token_attention<4>(p, b, kv, decode, splits, s);
    case 5: return launch_token_attention<5>(p, b, kv, decode, splits, s);
    case 6: return launch_token_attention<6>(p, b, kv, decode, splits, s);
    case 7: return launch_token_attention<7>(p, b, kv, decode, splits, s);
    case 8: return launch_token_attention<8>(p, b, kv, decode, splits, s);
    default: set_error("attention: GQA group %d is not implemented (1..8)", group); return Q38_ERR_INVALID;
  }
}

int check_attention(const q38_attention_params* p, const q38_batch_desc* b, const q38_kv_cache_desc* kv) {
  Q38_REQUIRE(p && b && kv, "attention: null argument");
  Q38_REQUIRE(p->q && p->gate && p->out, "attention: null pointer");
  Q38_REQUIRE(p->num_kv_heads > 0 && p->num_q_heads % p->num_kv_heads == 0, "attention: heads %d / %d",
              p->num_q_heads, p->num_kv_heads);
  Q38_REQUIRE(kv->kv_heads == p->num_kv_heads, "attention: kv head count mismatch");
  Q38_REQUIRE(kv->pool && kv->block_table && kv->max_pages_per_seq > 0, "attention: kv cache descriptor");
  return Q38_OK;
}

}  // namespace

unsigned int attention_error(bool clear) { return read_tu_error(clear); }
unsigned int* attention_error_address() { return tu_error_address(); }

}  // namespace q38

using namespace q38;

extern "C" int q38_qk_norm_rope_append(const q38_qk_norm_rope_params* p, const q38_batch_desc* batch,
                                       const q38_kv_cache_desc* kv, void* stream) {
  Q38_REQUIRE(p && batch && kv, "qk_norm_rope_append: null argument");
  if (batch->num_tokens == 0) return Q38_OK;
  const int warps = p->num_q_heads + 2 * p->num_kv_heads;
  Q38_REQUIRE(warps > 0 && warps <= 32, "qk_norm_rope_append: %d heads per token exceed one CTA", warps);
  Q38_REQUIRE(kv->kv_heads == p->num_kv_heads, "qk_norm_rope_append: kv head count mismatch");
  Q38_REQUIRE(p->ld_proj % 8 == 0, "qk_norm_rope_append: ld_proj must be a multiple of 8");
  RopeTable rope;
  for (int i = 0; i < 32; ++i) rope.inv_freq[i] = 1.0f / std::pow(float(p->rope_theta), float(2 * i) / 64.0f);
  (void)launch_kernel(qk_norm_rope_kernel, dim3(batch->num_tokens), dim3(warps * 32), 0, as_stream(stream), 
      reinterpret_cast<const __nv_bfloat16*>(p->proj), p->ld_proj, p->q_norm, p->k_norm, p->eps, p->num_q_heads,
      p->num_kv_heads, reinterpret_cast<__half*>(p->q_out), p->attn_layer, rope, batch->tok_pos, batch->tok_seq,
      batch->seq_slot, make_view(*kv));
  Q38_LAUNCH_OK("qk_norm_rope_kernel");
  return Q38_OK;
}

// Split count of the decode launcher. Context lengths of a ragged batch differ by orders of magnitude and the count is
// fixed per captured graph, so it is chosen for balance, not for occupancy: about sixteen work items per SM, so
// that the longest sequence's share per CTA is small against the whole step; splits beyond a short sequence's
// pages cost one early-exiting CTA each.
extern "C" int q38_attention_decode_splits(int batch_seqs, int kv_heads, int num_sms, int max_splits) {
  const int ctas = batch_seqs * kv_heads;
  if (ctas <= 0) return 1;
  int s = (16 * num_sms + ctas - 1) / ctas;
  if (s < 1) s = 1;
  if (s > max_splits) s = max_splits;
  if (s > 256) s = 256;
  return s;
}

extern "C" int q38_attention_decode(const q38_attention_params* p, const q38_batch_desc* batch,
                                    const q38_kv_cache_desc* kv, void* stream) {
  const int rc = check_attention(p, batch, kv);
  if (rc != Q38_OK) return rc;
  if (batch->num_seqs == 0) return Q38_OK;
  Q38_REQUIRE(batch->num_tokens == batch->num_seqs, "attention_decode: one token per sequence expected");
  int splits = q38_attention_decode_splits(batch->num_seqs, p->num_kv_heads, num_sms(), p->max_splits);
  if (!p->split_scratch) splits = 1;
  const int group = p->num_q_heads / p->num_kv_heads;
  if (kv->dtype != Q38_KV_INT8) return dispatch_group(group, *p, *batch, *kv, true, splits, as_stream(stream));
  Q38_REQUIRE(group >= 1 && group <= 8, "attention: GQA group %d is not implemented (1..8)", group);
  static const cudaError_t attr =
      cudaFuncSetAttribute(attn_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
  Q38_CUDA_OK(attr);
  const cudaStream_t s = as_stream(stream);
  const __nv_bfloat16* gate = reinterpret_cast<const __nv_bfloat16*>(p->gate);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p->out);
  (void)launch_kernel(attn_decode_mma_kernel, dim3(splits, p->num_kv_heads, batch->num_seqs), dim3(kMmaThreads), kMmaSmem, s, 
      reinterpret_cast<const __half*>(p->q), gate, p->ld_gate, out, p->num_q_heads, group, p->attn_layer,
      p->split_scratch, p->max_splits, splits, 1, batch->seq_start, batch->seq_slot, batch->seq_pos0, batch->tok_pos,
      batch->tok_seq, make_view(*kv));
  Q38_LAUNCH_OK("attn_decode_mma_kernel");
  if (splits > 1) {
    (void)launch_kernel(attn_merge_kernel, dim3(p->num_q_heads, batch->num_seqs), dim3(kHd), 0, s, p->split_scratch, p->max_splits, splits, gate,
                                                                           p->ld_gate, out, p->num_q_heads,
                                                                           batch->seq_start);
    Q38_LAUNCH_OK("attn_merge_kernel");
  }
  return Q38_OK;
}

extern "C" int q38_attention_prefill(const q38_attention_params* p, const q38_batch_desc* batch,
                                     const q38_kv_cache_desc* kv, void* stream) {
  const int rc = check_attention(p, batch, kv);
  if (rc != Q38_OK) return rc;
  if (batch->num_tokens == 0) return Q38_OK;
  const int group = p->num_q_heads / p->num_kv_heads;
  const bool int8 = kv->dtype == Q38_KV_INT8;
  if (batch->max_tokens_per_seq > 1 && group >= 1 && group <= kPfRows) {
    // chunks of more than one token: the query-tiled kernel. With few tiles for the GPU (one long request, or a
    // tensor-parallel rank with one kv head) the keys are cut over several CTAs per tile when the caller's scratch
    // (laid out [token][q head][max_splits][258]) allows it.
    static const cudaError_t attr_pf =
        cudaFuncSetAttribute(attn_prefill_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem);
    static const cudaError_t attr_pf16 =
        cudaFuncSetAttribute(attn_prefill_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem);
    Q38_CUDA_OK(attr_pf);
    Q38_CUDA_OK(attr_pf16);
    const int tq = kPfRows / group;
    const int tiles_per_seq = (batch->max_tokens_per_seq + tq - 1) / tq;
    const int tiles = (batch->num_tokens + tq - 1) / tq + batch->num_seqs;  // upper bound of the live tiles
    int splits = 1;
    if (p->split_scratch && p->max_splits > 1 && p->scratch_rows >= batch->num_tokens) {
      // The cut that gives every CTA the fewest keys per wave of CTAs: s / ceil(tiles * kv heads * s / SMs) is largest
      // (thirteen tiles of one kv head: eleven cuts fill one wave of 143 CTAs, sixteen would need two waves of longer
      // tails). One sequence: the tile count is exact; otherwise it is the upper bound above. Up to two waves.
      const int live = (batch->num_seqs == 1 ? tiles_per_seq : tiles) * p->num_kv_heads;
      const int sms = num_sms(), cap = std::min(p->max_splits, 16);
      double best = 0.0;
      for (int c = 1; c <= cap; ++c) {
        const int waves = (live * c + sms - 1) / sms;
        if (waves > 2) break;
        const double gain = double(c) / waves;
        if (gain > best * 1.02) {  // a further cut must pay for its share of the merge
          best = gain;
          splits = c;
        }
      }
    }
    const cudaStream_t s = as_stream(stream);
    const __nv_bfloat16* gate = reinterpret_cast<const __nv_bfloat16*>(p->gate);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p->out);
    (void)launch_kernel(int8 ? attn_prefill_tile_kernel<true> : attn_prefill_tile_kernel<false>,
                        dim3(splits, p->num_kv_heads, batch->num_seqs * tiles_per_seq), dim3(kPfThreads), kPfSmem, s,
                        reinterpret_cast<const __half*>(p->q), gate, p->ld_gate, out, p->num_q_heads, group, p->attn_layer,
                        tq, tiles_per_seq, p->split_scratch, p->max_splits, splits, batch->seq_start, batch->seq_slot,
                        batch->seq_pos0, make_view(*kv));
    Q38_LAUNCH_OK("attn_prefill_tile_kernel");
    if (splits > 1) {
      (void)launch_kernel(attn_merge_kernel, dim3(p->num_q_heads, batch->num_tokens), dim3(kHd), 0, s, p->split_scratch,
                          p->max_splits, splits, gate, p->ld_gate, out, p->num_q_heads, static_cast<const int*>(nullptr));
      Q38_LAUNCH_OK("attn_merge_kernel");
    }
    return Q38_OK;
  }
  if (!int8) return dispatch_group(group, *p, *batch, *kv, false, 1, as_stream(stream));
  // single-token chunks: the decode kernel, one CTA per (kv head, token)
  Q38_REQUIRE(group >= 1 && group <= 8, "attention: GQA group %d is not implemented (1..8)", group);
  static const cudaError_t attr =
      cudaFuncSetAttribute(attn_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
  Q38_CUDA_OK(attr);
  (void)launch_kernel(attn_decode_mma_kernel, dim3(1, p->num_kv_heads, batch->num_tokens), dim3(kMmaThreads), kMmaSmem, as_stream(stream), 
      reinterpret_cast<const __half*>(p->q), reinterpret_cast<const __nv_bfloat16*>(p->gate), p->ld_gate,
      reinterpret_cast<__nv_bfloat16*>(p->out), p->num_q_heads, group, p->attn_layer, p->split_scratch, p->max_splits, 1,
      0, batch->seq_start, batch->seq_slot, batch->seq_pos0, batch->tok_pos, batch->tok_seq, make_view(*kv));
  Q38_LAUNCH_OK("attn_decode_mma_kernel");
  return Q38_OK;
}
