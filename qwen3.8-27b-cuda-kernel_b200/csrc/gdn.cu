// Gated DeltaNet layers: a/b gate projection, fused causal conv(4) + SiLU + q/k L2 norm with the conv
// state carry, and the 128x128 fp32 recurrent-state update with the gated RMSNorm, over ragged
// sequences. Replaces kernels::gdn_ab, gdn_conv and gdn_recurrence of the reference
// (src/kernels/kernels.h:184-228, src/kernels/gdn.cu). State layouts (reference docs/FORMAT.md 3.2):
// recurrent fp32 [slot][gdn_layer][v_head][128 dv][128 dk]; conv bf16 [slot][gdn_layer][3][conv_dim],
// tap 0 oldest.
#include <algorithm>

#include "common.cuh"
#include "host_util.h"

namespace q38 {
extern int g_chunk_scan_tensor_cores;  // 1: the chunk scan runs its products on the tensor cores (TF32)
namespace {

constexpr int kDk = 128, kDv = 128;

// ---------------------------------------------------------------------------------------------------
// gdn_ab: ab[m][j] = rs[m] * sum_k xbf[m][k] * w[j][k]  (fp32; rows j < nv are b, the rest a).
// One CTA per (8 weight rows, 8 tokens); the 8 warps split K, every lane issues 16 independent 16-byte loads
// per step (8 weight rows + 8 token rows) for 512 FMAs, and the warps' partial sums meet in shared memory.
// ---------------------------------------------------------------------------------------------------
constexpr int kAbRows = 8, kAbTokens = 8;
__global__ void __launch_bounds__(256) gdn_ab_kernel(const __nv_bfloat16* __restrict__ xbf, int m, int hidden,
                                                     const __nv_bfloat16* __restrict__ w, int rows,
                                                     const float* __restrict__ partials_in, float eps,
                                                     float* __restrict__ ab_out) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  __shared__ float red[8][kAbRows * kAbTokens];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j0 = blockIdx.x * kAbRows, m0 = blockIdx.y * kAbTokens;
  float acc[kAbRows][kAbTokens];
#pragma unroll
  for (int r = 0; r < kAbRows; ++r)
#pragma unroll
    for (int t = 0; t < kAbTokens; ++t) acc[r][t] = 0.0f;
  for (int c = warp * 32 + lane; c < hidden / 8; c += 256) {
    float wf[kAbRows][8], xf[kAbTokens][8];
#pragma unroll
    for (int r = 0; r < kAbRows; ++r) {
      const int j = min(j0 + r, rows - 1);
      const uint4 v = reinterpret_cast<const uint4*>(w + (size_t)j * hidden)[c];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        wf[r][2 * i] = __low2float(p[i]);
        wf[r][2 * i + 1] = __high2float(p[i]);
      }
    }
#pragma unroll
    for (int t = 0; t < kAbTokens; ++t) {
      const int mm = min(m0 + t, m - 1);
      const uint4 v = reinterpret_cast<const uint4*>(xbf + (size_t)mm * hidden)[c];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xf[t][2 * i] = __low2float(p[i]);
        xf[t][2 * i + 1] = __high2float(p[i]);
      }
    }
#pragma unroll
    for (int r = 0; r < kAbRows; ++r)
#pragma unroll
      for (int t = 0; t < kAbTokens; ++t)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][t] += wf[r][i] * xf[t][i];
  }
#pragma unroll
  for (int r = 0; r < kAbRows; ++r)
#pragma unroll
    for (int t = 0; t < kAbTokens; ++t) {
      const float v = warp_sum(acc[r][t]);
      if (lane == 0) red[warp][r * kAbTokens + t] = v;
    }
  __syncthreads();
  if (threadIdx.x < kAbRows * kAbTokens) {
    const int r = threadIdx.x / kAbTokens, t = threadIdx.x % kAbTokens;
    if (j0 + r < rows && m0 + t < m) {
      float total = 0.0f;
#pragma unroll
      for (int wi = 0; wi < 8; ++wi) total += red[wi][threadIdx.x];
      float rs = 1.0f;
      if (partials_in) {
        const int blocks = hidden / 128;
        float sum = 0.0f;
        for (int b = 0; b < blocks; ++b) sum += partials_in[(size_t)(m0 + t) * blocks + b];
        rs = 1.0f / sqrtf(sum / float(hidden) + eps);
      }
      ab_out[(size_t)(m0 + t) * rows + j0 + r] = total * rs;
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// gdn_conv: depthwise causal conv (width 4) + SiLU over the [q | k | v] channels; q/k heads are
// L2-normalised (x * rsqrt(sum x^2 + 1e-6)), q additionally scaled by 1/sqrt(128).
// Token-parallel: one CTA per (128-channel head block, 1 or 8 consecutive tokens). The three previous inputs of a channel
// come from the same chunk's earlier rows of `proj`, or from the conv state for the first tokens of a
// sequence's chunk. A second small kernel then rolls the conv state forward by the chunk.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdn_conv_kernel(const __nv_bfloat16* __restrict__ proj, int ld_proj,
                                                       const float* __restrict__ conv_w, float* __restrict__ qkv,
                                                       int conv_dim, int key_dim, int layer, int num_layers,
                                                       __nv_bfloat16* __restrict__ conv_state,
                                                       const int* __restrict__ seq_start,
                                                       const int* __restrict__ seq_slot,
                                                       const int* __restrict__ tok_seq, int roll_state, int num_tokens,
                                                       int tokens_per_cta, int one_token_each) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  __shared__ float red[4];
  const int c = blockIdx.x * 128 + threadIdx.x;
  const float4 w = *reinterpret_cast<const float4*>(conv_w + (size_t)c * 4);
  const int m_end = min(num_tokens, (int(blockIdx.y) + 1) * tokens_per_cta);
  for (int m = blockIdx.y * tokens_per_cta; m < m_end; ++m) {
    // one_token_each (a decode batch: every sequence has exactly one token, so token m is sequence m's and the first of
    // its run): two dependent loads fewer on the way to the taps
    const int b = one_token_each ? m : tok_seq[m];
    const int i = one_token_each ? 0 : m - seq_start[b];  // index of the token inside its sequence's chunk
    __nv_bfloat16* st = conv_state + ((size_t)seq_slot[b] * num_layers + layer) * 3 * conv_dim;
    float x[4];
    __nv_bfloat16 xb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // x[j] = input 3 - j steps back
      const int back = 3 - j;
      xb[j] = back <= i ? proj[(size_t)(m - back) * ld_proj + c] : st[(size_t)(3 + i - back) * conv_dim + c];
      x[j] = __bfloat162float(xb[j]);
    }
    if (roll_state) {  // one token per sequence: this thread is the only reader of its channel's taps, so it also rolls them
      st[c] = xb[1];
      st[(size_t)conv_dim + c] = xb[2];
      st[(size_t)2 * conv_dim + c] = xb[3];
    }
    float acc = 0.0f;
    acc += w.x * x[0];
    acc += w.y * x[1];
    acc += w.z * x[2];
    acc += w.w * x[3];
    float y = silu_f(acc);
    if (c < 2 * key_dim) {  // block-uniform: the 128 channels of a CTA are one q or k head
      const float ss = warp_sum(y * y);
      __syncthreads();  // the previous token's readers of red[] are done
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      const float total = red[0] + red[1] + red[2] + red[3];
      y *= 1.0f / sqrtf(total + 1e-6f);
      if (c < key_dim) y *= 0.08838834764831845f;  // 1 / sqrt(128)
    }
    qkv[(size_t)m * conv_dim + c] = y;
  }
}

// The same for prefill-sized steps: one CTA per (128-channel head block, 8 consecutive tokens), state not rolled here.
// A thread requests its channel's eleven inputs of the window (rows m0 - 3 .. m0 + 7 of `proj`) and the tokens' sequence
// data before it computes anything, so the CTA pays one round trip to memory instead of one per token; the taps a
// sequence's first three tokens take from the conv state are fetched on demand. The arithmetic per token is that of
// gdn_conv_kernel, in the same order.
constexpr int kConvBlock = 8;
__global__ void __launch_bounds__(128) gdn_conv_block_kernel(const __nv_bfloat16* __restrict__ proj, int ld_proj,
                                                             const float* __restrict__ conv_w, float* __restrict__ qkv,
                                                             int conv_dim, int key_dim, int layer, int num_layers,
                                                             const __nv_bfloat16* __restrict__ conv_state,
                                                             const int* __restrict__ seq_start,
                                                             const int* __restrict__ seq_slot,
                                                             const int* __restrict__ tok_seq, int num_tokens) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  __shared__ float red[kConvBlock][4];
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int m0 = blockIdx.y * kConvBlock;
  const int nt = min(kConvBlock, num_tokens - m0);
  const float4 w = *reinterpret_cast<const float4*>(conv_w + (size_t)c * 4);
  float win[kConvBlock + 3];  // inputs of rows m0 - 3 + k
#pragma unroll
  for (int k = 0; k < kConvBlock + 3; ++k) {
    const int row = m0 - 3 + k;
    win[k] = row >= 0 && row < num_tokens ? __bfloat162float(proj[(size_t)row * ld_proj + c]) : 0.0f;
  }
  int seq[kConvBlock], idx[kConvBlock];
#pragma unroll
  for (int t = 0; t < kConvBlock; ++t) seq[t] = t < nt ? tok_seq[m0 + t] : 0;
#pragma unroll
  for (int t = 0; t < kConvBlock; ++t) idx[t] = t < nt ? m0 + t - seq_start[seq[t]] : 3;  // index inside its sequence's chunk
  float y[kConvBlock];
#pragma unroll
  for (int t = 0; t < kConvBlock; ++t) {
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = win[t + j];  // input 3 - j steps back
    if (t < nt && idx[t] < 3) {  // the sequence's chunk starts here: older inputs come from its conv state
      const __nv_bfloat16* st = conv_state + ((size_t)seq_slot[seq[t]] * num_layers + layer) * 3 * conv_dim;
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int back = 3 - j;
        if (back > idx[t]) x[j] = __bfloat162float(st[(size_t)(3 + idx[t] - back) * conv_dim + c]);
      }
    }
    float acc = 0.0f;
    acc += w.x * x[0];
    acc += w.y * x[1];
    acc += w.z * x[2];
    acc += w.w * x[3];
    y[t] = silu_f(acc);
  }
  if (c < 2 * key_dim) {  // block-uniform: the 128 channels of a CTA are one q or k head
#pragma unroll
    for (int t = 0; t < kConvBlock; ++t) {
      const float ss = warp_sum(y[t] * y[t]);
      if ((threadIdx.x & 31) == 0) red[t][threadIdx.x >> 5] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kConvBlock; ++t) {
      const float total = red[t][0] + red[t][1] + red[t][2] + red[t][3];
      y[t] *= 1.0f / sqrtf(total + 1e-6f);
      if (c < key_dim) y[t] *= 0.08838834764831845f;  // 1 / sqrt(128)
    }
  }
#pragma unroll
  for (int t = 0; t < kConvBlock; ++t)
    if (t < nt) qkv[(size_t)(m0 + t) * conv_dim + c] = y[t];
}

__global__ void __launch_bounds__(128) gdn_conv_state_kernel(const __nv_bfloat16* __restrict__ proj, int ld_proj,
                                                             int conv_dim, int layer, int num_layers,
                                                             __nv_bfloat16* __restrict__ conv_state,
                                                             const int* __restrict__ seq_start,
                                                             const int* __restrict__ seq_slot) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
  const int s = seq_start[b], n = seq_start[b + 1] - s;
  if (n <= 0) return;
  __nv_bfloat16* st = conv_state + ((size_t)seq_slot[b] * num_layers + layer) * 3 * conv_dim;
  __nv_bfloat16 old[3], nw[3];
#pragma unroll
  for (int t = 0; t < 3; ++t) old[t] = st[(size_t)t * conv_dim + c];
#pragma unroll
  for (int t = 0; t < 3; ++t) {  // history = [old0 old1 old2 x0 .. x(n-1)], keep its last three
    const int idx = n + t;
    nw[t] = idx < 3 ? old[idx] : proj[(size_t)(s + idx - 3) * ld_proj + c];
  }
#pragma unroll
  for (int t = 0; t < 3; ++t) st[(size_t)t * conv_dim + c] = nw[t];
}

// ---------------------------------------------------------------------------------------------------
// gdn_recurrence: one CTA per (v head, sequence). The 128x128 fp32 state lives in registers for the
// whole chunk: 16 warps x 8 rows, a lane owns 4 consecutive columns of each row, so a row is one
// coalesced 512-byte access. Per token (reference src/kernels/gdn.cu:275-334, oracle
// src/ref/ops.cpp:210-240):
//   beta = sigmoid(b); decay = exp(A * softplus(a + dt_bias));
//   S *= decay; kv = S k; delta = beta (v - kv); S += delta k^T; o = S q;
//   out = bf16(o * rsqrt(mean(o^2) + eps) * norm_w * silu(z)).
// ---------------------------------------------------------------------------------------------------
constexpr int kRecWarps = 16;
constexpr int kRowsPerWarp = kDv / kRecWarps;

__global__ void __launch_bounds__(kRecWarps * 32, 1) gdn_recurrence_kernel(
    const float* __restrict__ qkv, int conv_dim, const float* __restrict__ ab, const float* __restrict__ A,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ z, int ld_z,
    const float* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ out, int layer, int num_layers, int nk,
    int nv, float* __restrict__ recurrent, const int* __restrict__ seq_start, const int* __restrict__ seq_slot) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int vh = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s0 = seq_start[b], s1 = seq_start[b + 1];
  if (s1 <= s0) return;
  const int kh = vh / (nv / nk);
  float* S = recurrent + (((size_t)seq_slot[b] * num_layers + layer) * nv + vh) * kDv * kDk;
  const int row0 = warp * kRowsPerWarp;
  float4 st[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) st[r] = *reinterpret_cast<const float4*>(S + (size_t)(row0 + r) * kDk + 4 * lane);

  __shared__ float o_sm[kDv];
  __shared__ float red[kRecWarps];
  const float a_h = A[vh], dt_h = dt_bias[vh];
  const size_t q_off = (size_t)kh * kDk, k_off = (size_t)nk * kDk + (size_t)kh * kDk, v_off = (size_t)2 * nk * kDk + (size_t)vh * kDv;

  for (int m = s0; m < s1; ++m) {
    const float* row = qkv + (size_t)m * conv_dim;
    const float4 q4 = *reinterpret_cast<const float4*>(row + q_off + 4 * lane);
    const float4 k4 = *reinterpret_cast<const float4*>(row + k_off + 4 * lane);
    const float bb = ab[(size_t)m * 2 * nv + vh], aa = ab[(size_t)m * 2 * nv + nv + vh];
    const float beta = 1.0f / (1.0f + expf(-bb));
    const float xsp = aa + dt_h;
    const float sp = xsp > 20.0f ? xsp : log1pf(expf(xsp));
    const float decay = expf(a_h * sp);
    float ov[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float4 sv = st[r];
      sv.x *= decay;
      sv.y *= decay;
      sv.z *= decay;
      sv.w *= decay;
      const float kv = warp_sum(sv.x * k4.x + sv.y * k4.y + sv.z * k4.z + sv.w * k4.w);
      const float delta = beta * (row[v_off + row0 + r] - kv);
      sv.x += delta * k4.x;
      sv.y += delta * k4.y;
      sv.z += delta * k4.z;
      sv.w += delta * k4.w;
      st[r] = sv;
      ov[r] = warp_sum(sv.x * q4.x + sv.y * q4.y + sv.z * q4.z + sv.w * q4.w);
    }
    // gated RMSNorm over the 128 outputs of the head
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) ss += ov[r] * ov[r];
    if (lane == 0) red[warp] = ss;
    if (lane < kRowsPerWarp) {
      float mine = ov[0];
#pragma unroll
      for (int r = 1; r < kRowsPerWarp; ++r)
        if (lane == r) mine = ov[r];
      o_sm[row0 + lane] = mine;
    }
    __syncthreads();
    if (threadIdx.x < kDv) {
      float total = 0.0f;
#pragma unroll
      for (int w = 0; w < kRecWarps; ++w) total += red[w];
      const float r = 1.0f / sqrtf(total / float(kDv) + eps);
      const int d = threadIdx.x;
      const float zz = __bfloat162float(z[(size_t)m * ld_z + (size_t)vh * kDv + d]);
      out[(size_t)m * nv * kDv + (size_t)vh * kDv + d] = __float2bfloat16_rn(o_sm[d] * r * norm_w[d] * silu_f(zz));
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) *reinterpret_cast<float4*>(S + (size_t)(row0 + r) * kDk + 4 * lane) = st[r];
}


// ---------------------------------------------------------------------------------------------------
// gdn_recurrence for decode batches (every sequence advances by at most one token): the step is a pure
// stream over the recurrent state (64 KB read + 64 KB written per (sequence, head), a few hundred FMAs per
// thread), so it is organised around the memory pipeline instead of one CTA per (sequence, head):
//   * one persistent CTA per SM walks the (sequence, head) items cta, cta + grid, ...;
//   * a producer warp brings each item's state and its token's q / k / v / z rows into a three-slot
//     shared-memory ring with 1-D bulk (TMA) copies, so up to three states per SM are in flight while
//     a fourth is being computed;
//   * 16 compute warps take the state into registers (a slot is handed back as soon as it has been read),
//     run exactly the arithmetic of gdn_recurrence_kernel for one token, and write the new state straight
//     from registers with 16-byte stores.
// ---------------------------------------------------------------------------------------------------
constexpr int kDecSlots = 3;
constexpr int kDecStateBytes = kDv * kDk * 4;
constexpr int kDecQOff = kDecStateBytes, kDecKOff = kDecQOff + 512, kDecVOff = kDecKOff + 512, kDecZOff = kDecVOff + 512;
constexpr int kDecSlotBytes = kDecStateBytes + 2048;
constexpr int kDecTxBytes = kDecStateBytes + 3 * 512 + 256;
constexpr int kDecSmemBytes = 128 + kDecSlots * kDecSlotBytes + 2 * (kDv + 2 * kRecWarps) * 4 + 2 * kDecSlots * 8 + 16;
constexpr int kDecThreads = (kRecWarps + 1) * 32;

__global__ void __launch_bounds__(kDecThreads, 1) gdn_recurrence_decode_kernel(
    const float* __restrict__ qkv, int conv_dim, const float* __restrict__ ab, const float* __restrict__ A,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ z, int ld_z,
    const float* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ out, int layer, int num_layers, int nk,
    int nv, float* __restrict__ recurrent, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
    int num_seqs) {
  extern __shared__ uint8_t dec_smem_raw[];
  uint8_t* smem = dec_smem_raw + ((128 - (smem_u32(dec_smem_raw) & 127)) & 127);
  uint8_t* slots = smem;
  // outputs, partial sums of squares and the warps' wait results of an item: two sets used in turn, so that one barrier
  // per item is enough (a warp may start the next item while the others still read this one's set)
  float* o_sm_all = reinterpret_cast<float*>(smem + kDecSlots * kDecSlotBytes);
  float* red_all = o_sm_all + 2 * kDv;
  int* okf_all = reinterpret_cast<int*>(red_all + 2 * kRecWarps);
  uint64_t* full = reinterpret_cast<uint64_t*>(okf_all + 2 * kRecWarps);
  uint64_t* empty = full + kDecSlots;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kDecSlots);  // [0] compute warps, [1] producer

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = num_seqs * nv;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kRecWarps);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kRecWarps) {
    // ------------------------------ producer ------------------------------
    const uint64_t pol = policy_evict_first();
    uint32_t it = 0;
    bool waited = false;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int b = item / nv, vh = item - b * nv;
      const int m = seq_start[b];
      if (seq_start[b + 1] <= m) continue;
      const int slot = it % kDecSlots;
      int ok = 1;
      if (lane == 0) {
        ok = (!abort_flag[0] && mbar_wait(&empty[slot], ((it / kDecSlots) & 1) ^ 1, 0x401)) ? 1 : 0;
        if (ok) mbar_expect_tx(&full[slot], kDecTxBytes);
        else abort_flag[1] = 1;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      uint8_t* dst = slots + (size_t)slot * kDecSlotBytes;
      const float* S = recurrent + (((size_t)seq_slot[b] * num_layers + layer) * nv + vh) * kDv * kDk;
      const float* row = qkv + (size_t)m * conv_dim;
      const int kh = vh / (nv / nk);
      if (lane < 4)
        bulk_g2s(dst + lane * (kDecStateBytes / 4), reinterpret_cast<const uint8_t*>(S) + lane * (kDecStateBytes / 4),
                 kDecStateBytes / 4, &full[slot], pol);
      if (!waited) {  // the state and the batch metadata are older than the previous kernel; the token rows may not be
        pdl_wait();
        waited = true;
      }
      if (lane == 4)
        bulk_g2s(dst + kDecQOff, row + (size_t)kh * kDk, 512, &full[slot], pol);
      else if (lane == 5)
        bulk_g2s(dst + kDecKOff, row + (size_t)nk * kDk + (size_t)kh * kDk, 512, &full[slot], pol);
      else if (lane == 6)
        bulk_g2s(dst + kDecVOff, row + (size_t)2 * nk * kDk + (size_t)vh * kDv, 512, &full[slot], pol);
      else if (lane == 7)
        bulk_g2s(dst + kDecZOff, z + (size_t)m * ld_z + (size_t)vh * kDv, 256, &full[slot], pol);
      __syncwarp();
      ++it;
    }
    return;
  }

  // ------------------------------ compute warps ------------------------------
  pdl_wait();
  pdl_launch_dependents();
  const int row0 = warp * kRowsPerWarp;
  const int tid = threadIdx.x;
  uint32_t it = 0;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int b = item / nv, vh = item - b * nv;
    const int m = seq_start[b];
    if (seq_start[b + 1] <= m) continue;
    const int slot = it % kDecSlots;
    // scalars of this (token, head): requested before the wait so that their latency hides behind it
    const float bb = ab[(size_t)m * 2 * nv + vh], aa = ab[(size_t)m * 2 * nv + nv + vh];
    const float a_h = A[vh], dt_h = dt_bias[vh];
    const float nw = tid < kDv ? norm_w[tid] : 0.0f;
    float* S = recurrent + (((size_t)seq_slot[b] * num_layers + layer) * nv + vh) * kDv * kDk;
    // a wait that runs out marks the launch as failed; the warps leave the loop together below
    const bool ok = mbar_wait(&full[slot], (it / kDecSlots) & 1, 0x402);
    if (!ok) abort_flag[0] = 1;
    float* o_sm = o_sm_all + (it & 1u) * kDv;
    float* red = red_all + (it & 1u) * kRecWarps;
    int* okf = okf_all + (it & 1u) * kRecWarps;
    const uint8_t* src = slots + (size_t)slot * kDecSlotBytes;
    float4 st[kRowsPerWarp];
    float vv[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      st[r] = *reinterpret_cast<const float4*>(src + (size_t)(row0 + r) * kDk * 4 + 16 * lane);
      vv[r] = *reinterpret_cast<const float*>(src + kDecVOff + 4 * (row0 + r));
    }
    const float4 q4 = *reinterpret_cast<const float4*>(src + kDecQOff + 16 * lane);
    const float4 k4 = *reinterpret_cast<const float4*>(src + kDecKOff + 16 * lane);
    const float zz = tid < kDv ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + kDecZOff + 2 * tid)) : 0.0f;
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[slot]);  // everything of the slot is in registers now

    const float beta = 1.0f / (1.0f + expf(-bb));
    const float xsp = aa + dt_h;
    const float sp = xsp > 20.0f ? xsp : log1pf(expf(xsp));
    const float decay = expf(a_h * sp);
    float ov[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float4 sv = st[r];
      sv.x *= decay;
      sv.y *= decay;
      sv.z *= decay;
      sv.w *= decay;
      const float kv = warp_sum(sv.x * k4.x + sv.y * k4.y + sv.z * k4.z + sv.w * k4.w);
      const float delta = beta * (vv[r] - kv);
      sv.x += delta * k4.x;
      sv.y += delta * k4.y;
      sv.z += delta * k4.z;
      sv.w += delta * k4.w;
      st[r] = sv;
      ov[r] = warp_sum(sv.x * q4.x + sv.y * q4.y + sv.z * q4.z + sv.w * q4.w);
    }
    if (ok) {
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r)
        *reinterpret_cast<float4*>(S + (size_t)(row0 + r) * kDk + 4 * lane) = st[r];
    }
    // gated RMSNorm over the 128 outputs of the head
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) ss += ov[r] * ov[r];
    if (lane == 0) {
      red[warp] = ss;
      okf[warp] = ok ? 1 : 0;
    }
    if (lane < kRowsPerWarp) {
      float mine = ov[0];
#pragma unroll
      for (int r = 1; r < kRowsPerWarp; ++r)
        if (lane == r) mine = ov[r];
      o_sm[row0 + lane] = mine;
    }
    named_bar_sync(1, kRecWarps * 32);
    // a wait of any warp ran out: all of them leave after this item (the item's set was written before the barrier, so
    // every warp reads the same value)
    int stop = 0;
#pragma unroll
    for (int w = 0; w < kRecWarps; ++w) stop |= okf[w] ^ 1;
    if (tid < kDv && ok) {
      float total = 0.0f;
#pragma unroll
      for (int w = 0; w < kRecWarps; ++w) total += red[w];
      const float r = 1.0f / sqrtf(total / float(kDv) + eps);
      out[(size_t)m * nv * kDv + (size_t)vh * kDv + tid] = __float2bfloat16_rn(o_sm[tid] * r * nw * silu_f(zz));
    }
    if (stop) break;
    ++it;
  }
}


// ---------------------------------------------------------------------------------------------------
// gdn_recurrence for prefill chunks: the chunked (WY) form of the gated delta rule. The token recurrence
//     S_t = a_t S_{t-1} + beta_t (v_t - a_t S_{t-1} k_t) k_t^T,   o_t = S_t q_t        (S is [dv][dk])
// is sequential in t; over a chunk of C = 64 tokens with lg_i = sum_{t<=i} log a_t it is equivalent to
//     A[i][j] = beta_i e^{lg_i - lg_j} (k_i . k_j)  (j < i)          P[i][j] = e^{lg_i - lg_j} (q_i . k_j)  (j <= i)
//     (I + A) U0 = diag(beta) V         (I + A) W = diag(beta e^{lg}) K                       (prep, no state)
//     U = U0 - W S_0^T      O = diag(e^{lg}) Q S_0^T + P U      S_C = e^{lg_C} S_0 + U^T diag(e^{lg_C - lg}) K
// so everything that does not touch the state is computed for all chunks in parallel (gdn_chunk_prep_kernel,
// one CTA per (chunk, v head, sequence)), and the sequential part is four small matrix products per chunk with
// the state resident in shared memory (gdn_chunk_scan_kernel, one CTA per (v head, sequence)). All arithmetic
// is fp32 on the CUDA cores; every exponent is <= 0, so nothing overflows however strong the decay is.
// Tokens beyond a sequence's ragged tail are treated as beta = 0, log a = 0, q = k = v = 0 (no effect).
// Scratch per (chunk slot, v head): U0 [64][128], W [64][128], P [64][64], lg [64] floats; the chunk slots of
// sequence b start at seq_start[b] / 64 + b (never fewer than the chunks before it, so slots do not collide).
// ---------------------------------------------------------------------------------------------------
constexpr int kCh = 64;
constexpr int kLd = 132;   // padded row stride (floats) of 128-wide shared tiles: 16-byte reads of 8 rows hit 32 banks
constexpr int kLdP = 68;   // the same for 64-wide tiles
constexpr int kChunkFloats = 2 * kCh * 128 + kCh * kCh + kCh;
constexpr int kChunkThreads = 512;

__device__ __forceinline__ void token_gates(const float* __restrict__ ab, int m, int nv, int vh, float a_h, float dt_h,
                                            float& beta, float& log_decay) {
  const float bb = ab[(size_t)m * 2 * nv + vh], aa = ab[(size_t)m * 2 * nv + nv + vh];
  beta = 1.0f / (1.0f + expf(-bb));
  const float xsp = aa + dt_h;
  const float sp = xsp > 20.0f ? xsp : log1pf(expf(xsp));
  log_decay = a_h * sp;
}

// rows [0, nc) of a [.][128] fp32 row block -> shared [64][kLd], rows >= nc zero; optional per-row scale
__device__ __forceinline__ void load_rows_128(float* dst, const float* __restrict__ src, size_t ld, int nc,
                                              const float* row_scale, int tid) {
  for (int i = tid; i < kCh * 32; i += kChunkThreads) {
    const int r = i >> 5, c4 = i & 31;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nc) {
      v = *reinterpret_cast<const float4*>(src + (size_t)r * ld + 4 * c4);
      if (row_scale) {
        const float sc = row_scale[r];
        v.x *= sc;
        v.y *= sc;
        v.z *= sc;
        v.w *= sc;
      }
    }
    *reinterpret_cast<float4*>(dst + r * kLd + 4 * c4) = v;
  }
}

// The same copy as asynchronous 16-byte copies (cp.async): no register staging, so all of a tile's requests are in
// flight at once and the copy overlaps whatever the threads do until they wait for its group.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the destination is zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void rows_async_128(float* dst, const float* __restrict__ src, size_t ld, int nc, int tid) {
  for (int i = tid; i < kCh * 32; i += kChunkThreads) {
    const int r = i >> 5, c4 = i & 31;
    cp_async16(dst + r * kLd + 4 * c4, src + (size_t)(r < nc ? r : 0) * ld + 4 * c4, r < nc);
  }
}

constexpr int kPrepSmemBytes = (2 * kCh * kLd + kCh * kLdP + 3 * kCh) * 4;

__global__ void __launch_bounds__(kChunkThreads, 1) gdn_chunk_prep_kernel(
    const float* __restrict__ qkv, int conv_dim, const float* __restrict__ ab, const float* __restrict__ A,
    const float* __restrict__ dt_bias, int nk, int nv, const int* __restrict__ seq_start, float* __restrict__ scratch) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  extern __shared__ float prep_sm[];
  float* Ks = prep_sm;
  float* Qs = Ks + kCh * kLd;
  float* As = Qs + kCh * kLd;  // [64][kLdP]
  float* beta_s = As + kCh * kLdP;
  float* lg_s = beta_s + kCh;
  float* la_s = lg_s + kCh;
  const int c = blockIdx.x, vh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int s0 = seq_start[b], n = seq_start[b + 1] - s0;
  if (c * kCh >= n) return;
  const int nc = min(kCh, n - c * kCh), m0 = s0 + c * kCh;
  const int kh = vh / (nv / nk);
  float* out = scratch + ((size_t)(s0 / kCh + b + c) * nv + vh) * kChunkFloats;
  float* U0g = out;
  float* Wg = out + kCh * 128;
  float* Pg = out + 2 * kCh * 128;
  float* lgg = Pg + kCh * kCh;

  const float* rows = qkv + (size_t)m0 * conv_dim;
  load_rows_128(Qs, rows + (size_t)kh * kDk, conv_dim, nc, nullptr, tid);
  load_rows_128(Ks, rows + (size_t)nk * kDk + (size_t)kh * kDk, conv_dim, nc, nullptr, tid);
  if (tid < kCh) {
    float be = 0.0f, la = 0.0f;
    if (tid < nc) token_gates(ab, m0 + tid, nv, vh, A[vh], dt_bias[vh], be, la);
    beta_s[tid] = be;
    la_s[tid] = la;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.0f;
    for (int i = 0; i < kCh; ++i) {
      run += la_s[i];
      lg_s[i] = run;
    }
  }
  __syncthreads();
  if (tid < kCh) lgg[tid] = lg_s[tid];

  // ---- G = K K^T and Q K^T: thread = rows {2 ty, 2 ty + 1} x columns {tx + 16 jj} ----
  {
    const int ty = tid >> 4, tx = tid & 15;
    float ag[2][4], ap[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) ag[i][jj] = ap[i][jj] = 0.0f;
#pragma unroll 4
    for (int kk = 0; kk < 128; kk += 4) {
      float4 ak[2], aq[2], bk[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        ak[i] = *reinterpret_cast<const float4*>(Ks + (2 * ty + i) * kLd + kk);
        aq[i] = *reinterpret_cast<const float4*>(Qs + (2 * ty + i) * kLd + kk);
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) bk[jj] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * jj) * kLd + kk);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          ag[i][jj] += ak[i].x * bk[jj].x + ak[i].y * bk[jj].y + ak[i].z * bk[jj].z + ak[i].w * bk[jj].w;
          ap[i][jj] += aq[i].x * bk[jj].x + aq[i].y * bk[jj].y + aq[i].z * bk[jj].z + aq[i].w * bk[jj].w;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int r = 2 * ty + i, col = tx + 16 * jj;
        const float e = col <= r ? expf(lg_s[r] - lg_s[col]) : 0.0f;
        As[r * kLdP + col] = col < r ? beta_s[r] * e * ag[i][jj] : 0.0f;
        Pg[r * kCh + col] = e * ap[i][jj];
      }
  }
  __syncthreads();

  // ---- forward substitution (I + A) X = RHS: one thread per column of [diag(beta) V | diag(beta e^lg) K] ----
  if (tid < 256) {
    float x[kCh];
    if (tid < 128) {
      const float* vcol = rows + (size_t)2 * nk * kDk + (size_t)vh * kDv + tid;
#pragma unroll
      for (int i = 0; i < kCh; ++i) x[i] = i < nc ? beta_s[i] * vcol[(size_t)i * conv_dim] : 0.0f;
    } else {
#pragma unroll
      for (int i = 0; i < kCh; ++i) x[i] = beta_s[i] * expf(lg_s[i]) * Ks[i * kLd + tid - 128];
    }
#pragma unroll
    for (int i = 1; i < kCh; ++i) {
      float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;  // four chains: the row's sum is not one serial dependency
#pragma unroll
      for (int j0 = 0; j0 < i; j0 += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(As + i * kLdP + j0);  // entries at j >= i are zero
        c0 += a4.x * x[j0];
        if (j0 + 1 < i) c1 += a4.y * x[j0 + 1];
        if (j0 + 2 < i) c2 += a4.z * x[j0 + 2];
        if (j0 + 3 < i) c3 += a4.w * x[j0 + 3];
      }
      x[i] -= (c0 + c1) + (c2 + c3);
    }
    float* dst = tid < 128 ? U0g + tid : Wg + (tid - 128);
#pragma unroll
    for (int i = 0; i < kCh; ++i) dst[i * 128] = x[i];
  }
}

constexpr int kScanSmemBytes = (128 * kLd + 4 * kCh * kLd + kCh * kLdP + 3 * kCh) * 4;

// VSPLIT = 1: one CTA per (v head, sequence) updates all 128 state rows and finishes the output (gated RMSNorm)
// itself. VSPLIT = 2: two CTAs per head, 64 state rows each (the rows are independent given k, q, beta, decay); the
// un-normalised outputs go to scratch and gdn_norm_gate_kernel finishes them, because the norm runs over all 128
// outputs of a token. The split doubles the CTAs of the sequential part when a step has few (head, sequence) pairs.
template <int VSPLIT>
__global__ void __launch_bounds__(kChunkThreads, 1) gdn_chunk_scan_kernel(
    const float* __restrict__ qkv, int conv_dim, const __nv_bfloat16* __restrict__ z, int ld_z,
    const float* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ out, int layer, int num_layers, int nk,
    int nv, float* __restrict__ recurrent, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
    const float* __restrict__ scratch, float* __restrict__ o_scratch) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  constexpr int NV = kDv / VSPLIT;  // state rows (v) of this CTA
  constexpr int TV = 4 / VSPLIT;    // v per thread in the [tokens][v] products: v = lane + 32 jj
  extern __shared__ float scan_sm[];
  float* Ss = scan_sm;               // [NV v][kLd]
  float* Ws = Ss + NV * kLd;         // [64][kLd]
  float* Qs = Ws + kCh * kLd;
  float* Kd = Qs + kCh * kLd;        // K rows
  float* Us = Kd + kCh * kLd;        // U0, then U: [64][kLd], NV columns used
  float* Ps = Us + kCh * kLd;        // [64][kLdP]
  float* lg_s = Ps + kCh * kLdP;
  float* eg_s = lg_s + kCh;          // e^{lg_t}
  float* kd_s = eg_s + kCh;          // e^{lg_C - lg_j}
  const int vh = blockIdx.x / VSPLIT, vbase = (blockIdx.x % VSPLIT) * NV, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s0 = seq_start[b], n = seq_start[b + 1] - s0;
  if (n <= 0) return;
  const int kh = vh / (nv / nk);
  float* S = recurrent + ((((size_t)seq_slot[b] * num_layers + layer) * nv + vh) * kDv + vbase) * kDk;
  for (int i = tid; i < NV * 32; i += kChunkThreads)
    *reinterpret_cast<float4*>(Ss + (i >> 5) * kLd + 4 * (i & 31)) = *reinterpret_cast<const float4*>(S + (size_t)i * 4);
  const int chunks = (n + kCh - 1) / kCh;
  float nw[TV];
#pragma unroll
  for (int jj = 0; jj < TV; ++jj) nw[jj] = norm_w[vbase + lane + 32 * jj];

  for (int c = 0; c < chunks; ++c) {
    const int nc = min(kCh, n - c * kCh), m0 = s0 + c * kCh;
    const float* in = scratch + ((size_t)(s0 / kCh + b + c) * nv + vh) * kChunkFloats;
    __syncthreads();  // the previous chunk's state update (or the initial state load) is complete
    if (tid < kCh) {
      const float lg = in[2 * kCh * 128 + kCh * kCh + tid], lgc = in[2 * kCh * 128 + kCh * kCh + kCh - 1];
      lg_s[tid] = lg;
      eg_s[tid] = expf(lg);
      kd_s[tid] = expf(lgc - lg);
    }
    __syncthreads();
    const float* rows = qkv + (size_t)m0 * conv_dim;
    // group 1: what the two state products need (W, Q, U0); group 2: P and K, which land while those run
    rows_async_128(Ws, in + kCh * 128, 128, kCh, tid);
    rows_async_128(Qs, rows + (size_t)kh * kDk, conv_dim, nc, tid);
    for (int i = tid; i < kCh * (NV / 4); i += kChunkThreads) {
      const int r = i / (NV / 4), c4 = i % (NV / 4);
      cp_async16(Us + r * kLd + 4 * c4, in + (size_t)r * 128 + vbase + 4 * c4, true);
    }
    cp_async_commit();
    rows_async_128(Kd, rows + (size_t)nk * kDk + (size_t)kh * kDk, conv_dim, nc, tid);
    for (int i = tid; i < kCh * 16; i += kChunkThreads)
      cp_async16(Ps + (i >> 4) * kLdP + 4 * (i & 15), in + 2 * kCh * 128 + (size_t)i * 4, true);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // [64 tokens][NV v] products: threads 0-255 compute X = W S0^T, threads 256-511 Y = Q S0^T at the same time.
    // Thread tile 8 tokens (8 gw + i) x TV v (lane + 32 jj): with TV = 4, 12 shared-memory reads feed 128 FMAs, which
    // keeps the products FMA-bound instead of shared-memory-bound.
    const int grp = warp >> 3, gw = warp & 7;  // grp 0: X / upper half of P U, grp 1: Y / lower half + output
    const int t0 = 8 * gw;
    float acc[8][TV];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int jj = 0; jj < TV; ++jj) acc[i][jj] = 0.0f;
    {
      const float* Am = grp == 0 ? Ws : Qs;
#pragma unroll 2
      for (int kk = 0; kk < 128; kk += 4) {
        float4 bv[TV];
#pragma unroll
        for (int jj = 0; jj < TV; ++jj) bv[jj] = *reinterpret_cast<const float4*>(Ss + (lane + 32 * jj) * kLd + kk);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 av = *reinterpret_cast<const float4*>(Am + (t0 + i) * kLd + kk);
#pragma unroll
          for (int jj = 0; jj < TV; ++jj)
            acc[i][jj] += av.x * bv[jj].x + av.y * bv[jj].y + av.z * bv[jj].z + av.w * bv[jj].w;
        }
      }
    }
    if (grp == 0) {  // (a) U = U0 - X
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int jj = 0; jj < TV; ++jj) Us[(t0 + i) * kLd + lane + 32 * jj] -= acc[i][jj];
    } else {         // (b) Y scaled by e^{lg_t}
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int jj = 0; jj < TV; ++jj) acc[i][jj] *= eg_s[t0 + i];
    }
    cp_async_wait<0>();
    __syncthreads();  // U complete; nobody reads W any more; P and K have landed

    // ---- (c) O = Y + P U. P is lower triangular: tokens 8 gw .. 8 gw + 7 need j < 8 gw + 8; the two thread groups
    // split that range (group 1 continues on top of Y, group 0 starts from zero and hands its part over through
    // the W buffer).
    {
      const int j_end = 8 * gw + 8;
      const int j_mid = (j_end / 2) & ~3;
      const int ja = grp == 0 ? j_mid : 0, jb = grp == 0 ? j_end : j_mid;
      if (grp == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int jj = 0; jj < TV; ++jj) acc[i][jj] = 0.0f;
      }
      for (int j = ja; j < jb; j += 4) {
        float uv[4][TV];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int jj = 0; jj < TV; ++jj) uv[q][jj] = Us[(j + q) * kLd + lane + 32 * jj];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 pv = *reinterpret_cast<const float4*>(Ps + (t0 + i) * kLdP + j);
#pragma unroll
          for (int jj = 0; jj < TV; ++jj)
            acc[i][jj] += pv.x * uv[0][jj] + pv.y * uv[1][jj] + pv.z * uv[2][jj] + pv.w * uv[3][jj];
        }
      }
      if (grp == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int jj = 0; jj < TV; ++jj) Ws[(t0 + i) * kLd + lane + 32 * jj] = acc[i][jj];
      }
    }
    __syncthreads();  // group 0's part of P U is in the W buffer; every read of S0 is done
    if (grp == 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int jj = 0; jj < TV; ++jj) acc[i][jj] += Ws[(t0 + i) * kLd + lane + 32 * jj];
        const int t = t0 + i;
        const size_t m = (size_t)(m0 + t);
        if constexpr (VSPLIT == 1) {
          // gated RMSNorm over the 128 outputs of each token (a warp holds whole tokens)
          float sq = 0.0f;
#pragma unroll
          for (int jj = 0; jj < TV; ++jj) sq += acc[i][jj] * acc[i][jj];
          const float ss = warp_sum(sq);
          if (t < nc) {
            const float r = 1.0f / sqrtf(ss / float(kDv) + eps);
#pragma unroll
            for (int jj = 0; jj < TV; ++jj) {
              const int d = lane + 32 * jj;
              const float zz = __bfloat162float(z[m * ld_z + (size_t)vh * kDv + d]);
              out[m * nv * kDv + (size_t)vh * kDv + d] = __float2bfloat16_rn(acc[i][jj] * r * nw[jj] * silu_f(zz));
            }
          }
        } else if (t < nc) {
#pragma unroll
          for (int jj = 0; jj < TV; ++jj)
            o_scratch[m * nv * kDv + (size_t)vh * kDv + vbase + lane + 32 * jj] = acc[i][jj];
        }
      }
    }

    // ---- (d) S = e^{lg_C} S0 + U^T diag(e^{lg_C - lg}) K: thread tile v = TV vq + i, k = 4 ko + {0..3} and 64 + 4 ko + {0..3}
    {
      const int vq = tid >> 4, ko = tid & 15;
      float sacc[TV][8];
#pragma unroll
      for (int i = 0; i < TV; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) sacc[i][e] = 0.0f;
#pragma unroll 4
      for (int j = 0; j < kCh; ++j) {
        const float kdj = kd_s[j];  // e^{lg_C - lg_j}: the decay from token j to the end of the chunk
        float uu[TV];
#pragma unroll
        for (int i = 0; i < TV; ++i) uu[i] = Us[j * kLd + TV * vq + i] * kdj;
        const float4 k0 = *reinterpret_cast<const float4*>(Kd + j * kLd + 4 * ko);
        const float4 k1 = *reinterpret_cast<const float4*>(Kd + j * kLd + 64 + 4 * ko);
        const float kk8[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
#pragma unroll
        for (int i = 0; i < TV; ++i)
#pragma unroll
          for (int e = 0; e < 8; ++e) sacc[i][e] += uu[i] * kk8[e];
      }
      const float gC = eg_s[kCh - 1];
#pragma unroll
      for (int i = 0; i < TV; ++i) {
        float* r0 = Ss + (TV * vq + i) * kLd + 4 * ko;
        float4 a = *reinterpret_cast<float4*>(r0), bq = *reinterpret_cast<float4*>(r0 + 64);
        a.x = gC * a.x + sacc[i][0];
        a.y = gC * a.y + sacc[i][1];
        a.z = gC * a.z + sacc[i][2];
        a.w = gC * a.w + sacc[i][3];
        bq.x = gC * bq.x + sacc[i][4];
        bq.y = gC * bq.y + sacc[i][5];
        bq.z = gC * bq.z + sacc[i][6];
        bq.w = gC * bq.w + sacc[i][7];
        *reinterpret_cast<float4*>(r0) = a;
        *reinterpret_cast<float4*>(r0 + 64) = bq;
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < NV * 32; i += kChunkThreads)
    *reinterpret_cast<float4*>(S + (size_t)i * 4) = *reinterpret_cast<const float4*>(Ss + (i >> 5) * kLd + 4 * (i & 31));
}

// ---------------------------------------------------------------------------------------------------
// The same scan with the four per-chunk products on the tensor cores (mma.sync m16n8k8 TF32, fp32 accumulation);
// staging, the decay factors, the forward-substituted U0 / W of the preparation kernel and the state layout are those
// of gdn_chunk_scan_kernel, which stays as the fp32 CUDA-core form of the operator. One TF32 product keeps 10 mantissa
// bits of each factor, which is not enough here: outputs that are small through cancellation moved by more than the
// operator's tolerance in a few elements per million. So every fp32 factor x is split as x = hi + lo, hi = the top 19
// bits of x (exact in TF32), lo = x - hi (exact in fp32, its own low bits below 2^-20 |x|), and a product is three
// MMAs, lo hi + hi lo + hi hi: the dropped lo lo term and lo's truncation are about 2^-20 relative, i.e. fp32-like.
// Fragment reads straight from the padded fp32 tiles in shared memory (row strides 132 / 68 floats keep the eight
// rows x four columns of a fragment on distinct banks).
//   (a) X = W S0^T and (b) Y = Q S0^T   [64 tokens][NV v], k = 128: warps 0-7 X, warps 8-15 Y, one 16-token row
//       block x NV / 16 column tiles each; U = U0 - X goes back to shared memory, Y e^{lg} stays in registers;
//   (c) O = Y e^{lg} + P U: the Y warps go on over the chunk's tokens j <= their row block (P is lower triangular);
//   (d) S = e^{lg_C} S0 + (U diag(e^{lg_C - lg}))^T K   [NV v][128 k], j = 64: all sixteen warps.
// ---------------------------------------------------------------------------------------------------
struct Tf32Pair {
  uint32_t hi, lo;
};
__device__ __forceinline__ Tf32Pair split_tf32(float x) {
  Tf32Pair p;
  p.hi = __float_as_uint(x) & 0xFFFFE000u;             // sign, exponent, 10 mantissa bits: a TF32 number
  p.lo = __float_as_uint(x - __uint_as_float(p.hi));   // exact; the tensor core reads its top 19 bits
  return p;
}
// d += A B with A = (a0..a3), B = (b0, b1) given as split pairs: the two cross terms first, the main term last
__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1);
__device__ __forceinline__ void mma3_tf32(float (&d)[4], const Tf32Pair (&a)[4], const Tf32Pair& b0, const Tf32Pair& b1) {
  mma_tf32_1688(d, a[0].lo, a[1].lo, a[2].lo, a[3].lo, b0.hi, b1.hi);
  mma_tf32_1688(d, a[0].hi, a[1].hi, a[2].hi, a[3].hi, b0.lo, b1.lo);
  mma_tf32_1688(d, a[0].hi, a[1].hi, a[2].hi, a[3].hi, b0.hi, b1.hi);
}
__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int VSPLIT>
__global__ void __launch_bounds__(kChunkThreads, 1) gdn_chunk_scan_mma_kernel(
    const float* __restrict__ qkv, int conv_dim, const __nv_bfloat16* __restrict__ z, int ld_z,
    const float* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ out, int layer, int num_layers, int nk,
    int nv, float* __restrict__ recurrent, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
    const float* __restrict__ scratch, float* __restrict__ o_scratch) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int NV = kDv / VSPLIT;   // state rows (v) of this CTA
  constexpr int NT = NV / 16;        // 8-wide column tiles per warp in (a)-(d): 4 or 8
  extern __shared__ float scan_sm[];
  float* Ss = scan_sm;               // [NV v][kLd]
  float* Ws = Ss + NV * kLd;         // [64][kLd]: W, later the chunk's outputs (VSPLIT == 1)
  float* Qs = Ws + kCh * kLd;
  float* Kd = Qs + kCh * kLd;        // K rows
  float* Us = Kd + kCh * kLd;        // U0, then U: [64][kLd], NV columns used
  float* Ps = Us + kCh * kLd;        // [64][kLdP]
  float* lg_s = Ps + kCh * kLdP;
  float* eg_s = lg_s + kCh;          // e^{lg_t}
  float* kd_s = eg_s + kCh;          // e^{lg_C - lg_j}
  const int vh = blockIdx.x / VSPLIT, vbase = (blockIdx.x % VSPLIT) * NV, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int s0 = seq_start[b], n = seq_start[b + 1] - s0;
  if (n <= 0) return;
  const int kh = vh / (nv / nk);
  float* S = recurrent + ((((size_t)seq_slot[b] * num_layers + layer) * nv + vh) * kDv + vbase) * kDk;
  for (int i = tid; i < NV * 32; i += kChunkThreads)
    *reinterpret_cast<float4*>(Ss + (i >> 5) * kLd + 4 * (i & 31)) = *reinterpret_cast<const float4*>(S + (size_t)i * 4);
  const int chunks = (n + kCh - 1) / kCh;
  // (a)-(c): product X or Y, 16-token row block mt, column tiles nt0 .. nt0 + NT - 1 of the CTA's NV columns
  const int which = warp >> 3, mt = (warp & 7) >> 1, nt0 = (warp & 1) * NT;
  // (d): state rows 16 dm .. + 15, column tiles dn0 .. dn0 + NT - 1 of the 128 k columns
  const int dm = warp / (16 / NT), dn0 = (warp % (16 / NT)) * NT;

  for (int c = 0; c < chunks; ++c) {
    const int nc = min(kCh, n - c * kCh), m0 = s0 + c * kCh;
    const float* in = scratch + ((size_t)(s0 / kCh + b + c) * nv + vh) * kChunkFloats;
    __syncthreads();  // the previous chunk's state update and output pass (or the initial state load) are complete
    if (tid < kCh) {
      const float lg = in[2 * kCh * 128 + kCh * kCh + tid], lgc = in[2 * kCh * 128 + kCh * kCh + kCh - 1];
      lg_s[tid] = lg;
      eg_s[tid] = expf(lg);
      kd_s[tid] = expf(lgc - lg);
    }
    const float* rows = qkv + (size_t)m0 * conv_dim;
    rows_async_128(Ws, in + kCh * 128, 128, kCh, tid);
    rows_async_128(Qs, rows + (size_t)kh * kDk, conv_dim, nc, tid);
    for (int i = tid; i < kCh * (NV / 4); i += kChunkThreads) {
      const int r = i / (NV / 4), c4 = i % (NV / 4);
      cp_async16(Us + r * kLd + 4 * c4, in + (size_t)r * 128 + vbase + 4 * c4, true);
    }
    cp_async_commit();
    rows_async_128(Kd, rows + (size_t)nk * kDk + (size_t)kh * kDk, conv_dim, nc, tid);
    for (int i = tid; i < kCh * 16; i += kChunkThreads)
      cp_async16(Ps + (i >> 4) * kLdP + 4 * (i & 15), in + 2 * kCh * 128 + (size_t)i * 4, true);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- (a) / (b): [16 tokens][8 NT v] += A[16][128] S0^T ----
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
    {
      const float* Am = (which == 0 ? Ws : Qs) + (16 * mt + g) * kLd + t4;
      const float* Bm = Ss + (8 * nt0 + g) * kLd + t4;
#pragma unroll 4
      for (int ks = 0; ks < 16; ++ks) {
        const Tf32Pair a[4] = {split_tf32(Am[8 * ks]), split_tf32(Am[8 * kLd + 8 * ks]), split_tf32(Am[8 * ks + 4]),
                               split_tf32(Am[8 * kLd + 8 * ks + 4])};
#pragma unroll
        for (int j = 0; j < NT; ++j)
          mma3_tf32(acc[j], a, split_tf32(Bm[(8 * j) * kLd + 8 * ks]), split_tf32(Bm[(8 * j) * kLd + 8 * ks + 4]));
      }
    }
    const int ra = 16 * mt + g, rb = ra + 8;  // this lane's two token rows of the block
    if (which == 0) {  // U = U0 - X
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int col = 8 * (nt0 + j) + 2 * t4;
        float2* pa = reinterpret_cast<float2*>(Us + ra * kLd + col);
        float2* pb = reinterpret_cast<float2*>(Us + rb * kLd + col);
        float2 ua = *pa, ub = *pb;
        ua.x -= acc[j][0];
        ua.y -= acc[j][1];
        ub.x -= acc[j][2];
        ub.y -= acc[j][3];
        *pa = ua;
        *pb = ub;
      }
    } else {           // Y scaled by e^{lg_t}
      const float ea = eg_s[ra], eb = eg_s[rb];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        acc[j][0] *= ea;
        acc[j][1] *= ea;
        acc[j][2] *= eb;
        acc[j][3] *= eb;
      }
    }
    cp_async_wait<0>();
    __syncthreads();  // U complete; nobody reads W any more; P and K have landed

    // ---- (c) O = Y e^{lg} + P U on the Y warps; P[t][j] = 0 for j > t, so row block mt needs j < 16 mt + 16 ----
    if (which == 1) {
      const float* Pm = Ps + (16 * mt + g) * kLdP + t4;
      const float* Um = Us + t4 * kLd + 8 * nt0 + g;
      for (int ks = 0; ks < 2 * mt + 2; ++ks) {
        const Tf32Pair a[4] = {split_tf32(Pm[8 * ks]), split_tf32(Pm[8 * kLdP + 8 * ks]), split_tf32(Pm[8 * ks + 4]),
                               split_tf32(Pm[8 * kLdP + 8 * ks + 4])};
#pragma unroll
        for (int j = 0; j < NT; ++j)
          mma3_tf32(acc[j], a, split_tf32(Um[(8 * ks) * kLd + 8 * j]), split_tf32(Um[(8 * ks + 4) * kLd + 8 * j]));
      }
      if constexpr (VSPLIT == 1) {  // the chunk's outputs go through the W buffer: the norm runs over all 128 v of a token
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int col = 8 * (nt0 + j) + 2 * t4;
          *reinterpret_cast<float2*>(Ws + ra * kLd + col) = make_float2(acc[j][0], acc[j][1]);
          *reinterpret_cast<float2*>(Ws + rb * kLd + col) = make_float2(acc[j][2], acc[j][3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int col = vbase + 8 * (nt0 + j) + 2 * t4;
          if (ra < nc)
            *reinterpret_cast<float2*>(o_scratch + ((size_t)(m0 + ra) * nv + vh) * kDv + col) = make_float2(acc[j][0], acc[j][1]);
          if (rb < nc)
            *reinterpret_cast<float2*>(o_scratch + ((size_t)(m0 + rb) * nv + vh) * kDv + col) = make_float2(acc[j][2], acc[j][3]);
        }
      }
    }

    // ---- (d) S = e^{lg_C} S0 + (U diag(e^{lg_C - lg}))^T K: rows v = 16 dm + g (+ 8), columns k = 8 (dn0 + j) + 2 t4 ----
    {
      float sacc[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[j][e] = 0.0f;
      const float* Um = Us + t4 * kLd + 16 * dm + g;
      const float* Km = Kd + t4 * kLd + 8 * dn0 + g;
#pragma unroll 2
      for (int ks = 0; ks < 8; ++ks) {
        const float d0 = kd_s[8 * ks + t4], d1 = kd_s[8 * ks + t4 + 4];
        const Tf32Pair a[4] = {split_tf32(Um[(8 * ks) * kLd] * d0), split_tf32(Um[(8 * ks) * kLd + 8] * d0),
                               split_tf32(Um[(8 * ks + 4) * kLd] * d1), split_tf32(Um[(8 * ks + 4) * kLd + 8] * d1)};
#pragma unroll
        for (int j = 0; j < NT; ++j)
          mma3_tf32(sacc[j], a, split_tf32(Km[(8 * ks) * kLd + 8 * j]), split_tf32(Km[(8 * ks + 4) * kLd + 8 * j]));
      }
      const float gC = eg_s[kCh - 1];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int col = 8 * (dn0 + j) + 2 * t4;
        float2* pa = reinterpret_cast<float2*>(Ss + (16 * dm + g) * kLd + col);
        float2* pb = reinterpret_cast<float2*>(Ss + (16 * dm + g + 8) * kLd + col);
        float2 xa = *pa, xb = *pb;
        xa.x = gC * xa.x + sacc[j][0];
        xa.y = gC * xa.y + sacc[j][1];
        xb.x = gC * xb.x + sacc[j][2];
        xb.y = gC * xb.y + sacc[j][3];
        *pa = xa;
        *pb = xb;
      }
    }
    if constexpr (VSPLIT == 1) {
      __syncthreads();  // the chunk's outputs are in the W buffer
      // gated RMSNorm over the 128 outputs of each token: a warp takes four tokens, a lane four v
      for (int tt = 0; tt < 4; ++tt) {
        const int t = 4 * warp + tt;
        if (t >= nc) break;
        const float4 ov = *reinterpret_cast<const float4*>(Ws + t * kLd + 4 * lane);
        const float ss = warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w);
        const float r = 1.0f / sqrtf(ss / float(kDv) + eps);
        const size_t m = (size_t)(m0 + t);
        const uint2 zraw = *reinterpret_cast<const uint2*>(z + m * ld_z + (size_t)vh * kDv + 4 * lane);
        const __nv_bfloat162* zp = reinterpret_cast<const __nv_bfloat162*>(&zraw);
        const float4 wv = *reinterpret_cast<const float4*>(norm_w + 4 * lane);
        __nv_bfloat162 res[2];
        res[0] = __floats2bfloat162_rn(ov.x * r * wv.x * silu_f(__low2float(zp[0])), ov.y * r * wv.y * silu_f(__high2float(zp[0])));
        res[1] = __floats2bfloat162_rn(ov.z * r * wv.z * silu_f(__low2float(zp[1])), ov.w * r * wv.w * silu_f(__high2float(zp[1])));
        *reinterpret_cast<uint2*>(out + m * nv * kDv + (size_t)vh * kDv + 4 * lane) = *reinterpret_cast<uint2*>(res);
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < NV * 32; i += kChunkThreads)
    *reinterpret_cast<float4*>(S + (size_t)i * 4) = *reinterpret_cast<const float4*>(Ss + (i >> 5) * kLd + 4 * (i & 31));
}

// Gated RMSNorm of the split scan's outputs: one CTA per (token, v head), 128 threads.
__global__ void __launch_bounds__(kDv) gdn_norm_gate_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                                            int ld_z, const float* __restrict__ norm_w, float eps,
                                                            __nv_bfloat16* __restrict__ out, int nv) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float red[4];
  const int m = blockIdx.x, vh = blockIdx.y, d = threadIdx.x;
  const float v = o[((size_t)m * nv + vh) * kDv + d];
  const float ss = warp_sum(v * v);
  if ((d & 31) == 0) red[d >> 5] = ss;
  __syncthreads();
  const float r = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / float(kDv) + eps);
  const float zz = __bfloat162float(z[(size_t)m * ld_z + (size_t)vh * kDv + d]);
  out[((size_t)m * nv + vh) * kDv + d] = __float2bfloat16_rn(v * r * norm_w[d] * silu_f(zz));
}

}  // namespace

int g_chunk_scan_tensor_cores = 1;

unsigned int gdn_error(bool clear) { return read_tu_error(clear); }
unsigned int* gdn_error_address() { return tu_error_address(); }

}  // namespace q38

using namespace q38;

extern "C" int q38_gdn_ab(const q38_bf16* xbf, int m, int hidden, const q38_bf16* w_ab, int rows,
                          const float* partials_in, float eps, float* ab_out, void* stream) {
  if (m == 0) return Q38_OK;
  Q38_REQUIRE(xbf && w_ab && ab_out, "gdn_ab: null argument");
  Q38_REQUIRE(m > 0 && hidden > 0 && hidden % 128 == 0 && rows > 0, "gdn_ab: m %d hidden %d rows %d", m, hidden, rows);
  const dim3 grid((rows + kAbRows - 1) / kAbRows, (m + kAbTokens - 1) / kAbTokens);
  (void)launch_kernel(gdn_ab_kernel, dim3(grid), dim3(256), 0, as_stream(stream), reinterpret_cast<const __nv_bfloat16*>(xbf), m, hidden,
                                                     reinterpret_cast<const __nv_bfloat16*>(w_ab), rows, partials_in, eps,
                                                     ab_out);
  Q38_LAUNCH_OK("gdn_ab_kernel");
  return Q38_OK;
}

extern "C" int q38_gdn_conv(const q38_gdn_conv_params* p, const q38_gdn_dims* d, const q38_batch_desc* batch,
                            const q38_gdn_state_desc* st, void* stream) {
  Q38_REQUIRE(p && d && batch && st, "gdn_conv: null argument");
  if (batch->num_tokens == 0) return Q38_OK;
  Q38_REQUIRE(d->conv_dim == (2 * d->num_k_heads + d->num_v_heads) * 128, "gdn_conv: conv_dim %d", d->conv_dim);
  Q38_REQUIRE(p->proj && p->conv_w && p->qkv && st->conv, "gdn_conv: null pointer");
  const cudaStream_t s = as_stream(stream);
  const __nv_bfloat16* proj = reinterpret_cast<const __nv_bfloat16*>(p->proj);
  __nv_bfloat16* cs = reinterpret_cast<__nv_bfloat16*>(st->conv);
  // decode batches (one token per sequence) roll the conv state inside the conv kernel; longer runs need the second
  // kernel, because the first three tokens of a run all read the old taps
  const int roll = batch->max_tokens_per_seq == 1 ? 1 : 0;
  // decode-sized steps: one token per CTA (latency); prefill-sized steps: eight, to keep the CTA count in the thousands
  const int per_cta = batch->num_tokens >= 256 ? 8 : 1;
  if (per_cta == kConvBlock && !roll) {
    (void)launch_kernel(gdn_conv_block_kernel, dim3(d->conv_dim / 128, (batch->num_tokens + kConvBlock - 1) / kConvBlock),
                        dim3(128), 0, s, proj, d->ld_proj, p->conv_w, p->qkv, d->conv_dim, d->num_k_heads * 128,
                        p->gdn_layer, st->num_gdn_layers, static_cast<const __nv_bfloat16*>(cs), batch->seq_start,
                        batch->seq_slot, batch->tok_seq, batch->num_tokens);
    Q38_LAUNCH_OK("gdn_conv_block_kernel");
  } else {
    (void)launch_kernel(gdn_conv_kernel, dim3(d->conv_dim / 128, (batch->num_tokens + per_cta - 1) / per_cta),
                        dim3(128), 0, s, proj, d->ld_proj, p->conv_w, p->qkv, d->conv_dim, d->num_k_heads * 128,
                        p->gdn_layer, st->num_gdn_layers, cs, batch->seq_start, batch->seq_slot, batch->tok_seq, roll,
                        batch->num_tokens, per_cta, (roll && batch->num_tokens == batch->num_seqs) ? 1 : 0);
    Q38_LAUNCH_OK("gdn_conv_kernel");
  }
  if (roll) return Q38_OK;
  (void)launch_kernel(gdn_conv_state_kernel, dim3(d->conv_dim / 128, batch->num_seqs), dim3(128), 0, s, 
      proj, d->ld_proj, d->conv_dim, p->gdn_layer, st->num_gdn_layers, cs, batch->seq_start, batch->seq_slot);
  Q38_LAUNCH_OK("gdn_conv_state_kernel");
  return Q38_OK;
}

extern "C" int q38_gdn_recurrence(const q38_gdn_recurrence_params* p, const q38_gdn_dims* d,
                                  const q38_batch_desc* batch, const q38_gdn_state_desc* st, void* stream) {
  Q38_REQUIRE(p && d && batch && st, "gdn_recurrence: null argument");
  if (batch->num_tokens == 0) return Q38_OK;
  Q38_REQUIRE(d->num_k_heads > 0 && d->num_v_heads % d->num_k_heads == 0, "gdn_recurrence: head ratio");
  Q38_REQUIRE(p->qkv && p->ab && p->A && p->dt_bias && p->z && p->norm_w && p->out && st->recurrent,
              "gdn_recurrence: null pointer");
  if (batch->max_tokens_per_seq == 1) {
    static const cudaError_t attr = cudaFuncSetAttribute(gdn_recurrence_decode_kernel,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes);
    Q38_CUDA_OK(attr);
    Q38_REQUIRE(d->conv_dim % 4 == 0 && p->ld_z % 8 == 0 && reinterpret_cast<uintptr_t>(p->qkv) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(p->z) % 16 == 0 && reinterpret_cast<uintptr_t>(st->recurrent) % 16 == 0,
                "gdn_recurrence: rows of qkv, z and the state must be 16-byte aligned");
    const int items = batch->num_seqs * d->num_v_heads;
    (void)launch_kernel(gdn_recurrence_decode_kernel, dim3(std::min(num_sms(), items)), dim3(kDecThreads), kDecSmemBytes, as_stream(stream), 
        p->qkv, d->conv_dim, p->ab, p->A, p->dt_bias, reinterpret_cast<const __nv_bfloat16*>(p->z), p->ld_z, p->norm_w,
        p->eps, reinterpret_cast<__nv_bfloat16*>(p->out), p->gdn_layer, st->num_gdn_layers, d->num_k_heads,
        d->num_v_heads, st->recurrent, batch->seq_start, batch->seq_slot, batch->num_seqs);
    Q38_LAUNCH_OK("gdn_recurrence_decode_kernel");
    return Q38_OK;
  }
  (void)launch_kernel(gdn_recurrence_kernel, dim3(d->num_v_heads, batch->num_seqs), dim3(kRecWarps * 32), 0, as_stream(stream), 
      p->qkv, d->conv_dim, p->ab, p->A, p->dt_bias, reinterpret_cast<const __nv_bfloat16*>(p->z), p->ld_z, p->norm_w,
      p->eps, reinterpret_cast<__nv_bfloat16*>(p->out), p->gdn_layer, st->num_gdn_layers, d->num_k_heads,
      d->num_v_heads, st->recurrent, batch->seq_start, batch->seq_slot);
  Q38_LAUNCH_OK("gdn_recurrence_kernel");
  return Q38_OK;
}

extern "C" void q38_gdn_set_chunk_scan_tensor_cores(int on) { q38::g_chunk_scan_tensor_cores = on != 0; }

extern "C" size_t q38_gdn_chunk_scratch_floats(int max_tokens, int max_seqs, int num_v_heads) {
  // per-chunk U0 / W / P / lg for every chunk slot, then one [tokens][v heads * 128] fp32 row block for the split scan
  return (size_t)(max_tokens / kCh + max_seqs) * (size_t)num_v_heads * kChunkFloats +
         (size_t)max_tokens * (size_t)num_v_heads * kDv;
}

extern "C" int q38_gdn_recurrence_chunked(const q38_gdn_recurrence_params* p, const q38_gdn_dims* d,
                                          const q38_batch_desc* batch, const q38_gdn_state_desc* st, float* scratch,
                                          size_t scratch_floats, void* stream) {
  Q38_REQUIRE(p && d && batch && st, "gdn_recurrence_chunked: null argument");
  if (batch->num_tokens == 0) return Q38_OK;
  Q38_REQUIRE(d->num_k_heads > 0 && d->num_v_heads % d->num_k_heads == 0, "gdn_recurrence_chunked: head ratio");
  Q38_REQUIRE(p->qkv && p->ab && p->A && p->dt_bias && p->z && p->norm_w && p->out && st->recurrent && scratch,
              "gdn_recurrence_chunked: null pointer");
  Q38_REQUIRE(d->conv_dim % 4 == 0 && reinterpret_cast<uintptr_t>(p->qkv) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(scratch) % 16 == 0 && reinterpret_cast<uintptr_t>(st->recurrent) % 16 == 0,
              "gdn_recurrence_chunked: qkv rows, scratch and state must be 16-byte aligned");
  Q38_REQUIRE(batch->max_tokens_per_seq >= 1, "gdn_recurrence_chunked: max_tokens_per_seq %d", batch->max_tokens_per_seq);
  const size_t need = q38_gdn_chunk_scratch_floats(batch->num_tokens, batch->num_seqs, d->num_v_heads);
  Q38_REQUIRE(scratch_floats >= need, "gdn_recurrence_chunked: scratch of %zu floats, %zu needed", scratch_floats, need);
  static const cudaError_t attr1 =
      cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmemBytes);
  static const cudaError_t attr2 =
      cudaFuncSetAttribute(gdn_chunk_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemBytes);
  static const cudaError_t attr3 =
      cudaFuncSetAttribute(gdn_chunk_scan_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemBytes);
  static const cudaError_t attr4 =
      cudaFuncSetAttribute(gdn_chunk_scan_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemBytes);
  static const cudaError_t attr5 =
      cudaFuncSetAttribute(gdn_chunk_scan_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemBytes);
  Q38_CUDA_OK(attr1);
  Q38_CUDA_OK(attr2);
  Q38_CUDA_OK(attr3);
  Q38_CUDA_OK(attr4);
  Q38_CUDA_OK(attr5);
  const bool tc = g_chunk_scan_tensor_cores != 0;
  const cudaStream_t s = as_stream(stream);
  const int max_chunks = (batch->max_tokens_per_seq + kCh - 1) / kCh;
  (void)launch_kernel(gdn_chunk_prep_kernel, dim3(max_chunks, d->num_v_heads, batch->num_seqs), dim3(kChunkThreads), kPrepSmemBytes, s, 
      p->qkv, d->conv_dim, p->ab, p->A, p->dt_bias, d->num_k_heads, d->num_v_heads, batch->seq_start, scratch);
  Q38_LAUNCH_OK("gdn_chunk_prep_kernel");
  const __nv_bfloat16* zp = reinterpret_cast<const __nv_bfloat16*>(p->z);
  __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p->out);
  float* o_scratch = scratch + (size_t)(batch->num_tokens / kCh + batch->num_seqs) * (size_t)d->num_v_heads * kChunkFloats;
  // the sequential part has one CTA per (v head, sequence); with few of them, two CTAs share a head's state rows
  const bool split = 2 * d->num_v_heads * batch->num_seqs <= num_sms();
  if (split) {
    (void)launch_kernel(tc ? gdn_chunk_scan_mma_kernel<2> : gdn_chunk_scan_kernel<2>, dim3(2 * d->num_v_heads, batch->num_seqs), dim3(kChunkThreads),
                        kScanSmemBytes, s, p->qkv, d->conv_dim, zp, p->ld_z, p->norm_w, p->eps, outp, p->gdn_layer,
                        st->num_gdn_layers, d->num_k_heads, d->num_v_heads, st->recurrent, batch->seq_start,
                        batch->seq_slot, scratch, o_scratch);
    Q38_LAUNCH_OK("gdn_chunk_scan_kernel");
    (void)launch_kernel(gdn_norm_gate_kernel, dim3(batch->num_tokens, d->num_v_heads), dim3(kDv), 0, s, o_scratch, zp,
                        p->ld_z, p->norm_w, p->eps, outp, d->num_v_heads);
    Q38_LAUNCH_OK("gdn_norm_gate_kernel");
  } else {
    (void)launch_kernel(tc ? gdn_chunk_scan_mma_kernel<1> : gdn_chunk_scan_kernel<1>, dim3(d->num_v_heads, batch->num_seqs), dim3(kChunkThreads),
                        kScanSmemBytes, s, p->qkv, d->conv_dim, zp, p->ld_z, p->norm_w, p->eps, outp, p->gdn_layer,
                        st->num_gdn_layers, d->num_k_heads, d->num_v_heads, st->recurrent, batch->seq_start,
                        batch->seq_slot, scratch, o_scratch);
    Q38_LAUNCH_OK("gdn_chunk_scan_kernel");
  }
  return Q38_OK;
}
