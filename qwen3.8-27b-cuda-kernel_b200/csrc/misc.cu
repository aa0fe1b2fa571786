// Embedding gather, ragged-batch packing, sampling and scoring kernels of the step.
#include "common.cuh"
#include "host_util.h"

namespace q38 {
namespace {

// ---------------------------------------------------------------------------------------------------
// embed: residual[m] = table[tokens[m]] widened to fp32, bf16 copy, sum of squares per 128 columns.
// Replaces kernels::embed (reference src/kernels/kernels.h:131-134, src/kernels/embed.cu:13-43).
// One CTA per token; a warp owns whole 128-column blocks (4 columns per lane) so each partial is one
// warp reduction. The table may live in mapped pinned host memory (plain loads work for both).
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_kernel(const __nv_bfloat16* __restrict__ table,
                                                    const int32_t* __restrict__ tokens, int hidden,
                                                    float* __restrict__ residual, __nv_bfloat16* __restrict__ xbf,
                                                    float* __restrict__ partials) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* row = table + (size_t)tokens[m] * hidden;
  const int blocks = hidden / 128;
  for (int b = warp; b < blocks; b += blockDim.x >> 5) {
    const int col = b * 128 + 4 * lane;
    const uint2 raw = *reinterpret_cast<const uint2*>(row + col);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float4 v = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
    *reinterpret_cast<float4*>(residual + (size_t)m * hidden + col) = v;
    *reinterpret_cast<uint2*>(xbf + (size_t)m * hidden + col) = raw;
    const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) partials[(size_t)m * blocks + b] = ss;
  }
}

// ---------------------------------------------------------------------------------------------------
// residual_update: the Residual GEMM epilogue as an op of its own, for tensor-parallel runs in which the
// row-parallel projection's partial products are summed over the ranks before they may enter the residual:
// residual += delta; xbf = bf16(residual); partials[m][col / 128] = sum of residual^2 over the 128 columns.
// One warp per (token, 128-column block), as embed_kernel.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) residual_update_kernel(const float* __restrict__ delta, int hidden,
                                                              float* __restrict__ residual,
                                                              __nv_bfloat16* __restrict__ xbf,
                                                              float* __restrict__ partials) {
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blocks = hidden / 128;
  for (int b = warp; b < blocks; b += blockDim.x >> 5) {
    const size_t at = (size_t)m * hidden + b * 128 + 4 * lane;
    const float4 d = *reinterpret_cast<const float4*>(delta + at);
    float4 r = *reinterpret_cast<const float4*>(residual + at);
    r.x += d.x;
    r.y += d.y;
    r.z += d.z;
    r.w += d.w;
    *reinterpret_cast<float4*>(residual + at) = r;
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(r.x, r.y), p1 = __floats2bfloat162_rn(r.z, r.w);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&p0);
    packed.y = *reinterpret_cast<const uint32_t*>(&p1);
    *reinterpret_cast<uint2*>(xbf + at) = packed;
    const float ss = warp_sum(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w);
    if (lane == 0) partials[(size_t)m * blocks + b] = ss;
  }
}

// ---------------------------------------------------------------------------------------------------
// pack_ragged: per-sequence (count, pos0) -> seq_start (exclusive scan), tok_pos, tok_seq.
// One CTA; the scan is a shared-memory Hillis-Steele over up to 1024 sequences per pass.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) pack_ragged_kernel(const int* __restrict__ seq_count,
                                                           const int* __restrict__ seq_pos0, int num_seqs,
                                                           int num_tokens, int* __restrict__ seq_start,
                                                           int* __restrict__ tok_pos, int* __restrict__ tok_seq) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  __shared__ int scan[1024];
  __shared__ int carry;
  const int tid = threadIdx.x;
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < num_seqs; base += 1024) {
    const int b = base + tid;
    const int cnt = b < num_seqs ? seq_count[b] : 0;
    scan[tid] = cnt;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int add = tid >= o ? scan[tid - o] : 0;
      __syncthreads();
      scan[tid] += add;
      __syncthreads();
    }
    const int start = carry + scan[tid] - cnt;
    if (b < num_seqs) seq_start[b] = start;
    __syncthreads();
    if (tid == 1023) carry += scan[1023];
    __syncthreads();
  }
  if (tid == 0) seq_start[num_seqs] = carry;
  __syncthreads();
  // expansion: one warp per sequence, lanes stride over its tokens
  const int lane = tid & 31, warp = tid >> 5;
  for (int b = warp; b < num_seqs; b += 32) {
    const int s = seq_start[b], n = seq_count[b], p0 = seq_pos0[b];
    for (int i = lane; i < n; i += 32) {
      if (s + i < num_tokens) {
        tok_pos[s + i] = p0 + i;
        tok_seq[s + i] = b;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// sampling (reference src/kernels/kernels.h:233-256, src/kernels/sampling.cu:137-310): one CTA per
// row. Definition reproduced here: repetition / presence penalties applied once per distinct token of
// the slot's history; temperature <= 0 -> argmax with the lowest id among ties (log-prob reported as
// 0); otherwise top-k keeps every logit >= the k-th largest, min-p keeps l >= max + T log(min_p),
// top-p keeps the smallest set of largest logits whose mass reaches top_p of the kept mass, and the
// token is drawn by inverse CDF in index order. All masses are integers in 2^-40 fixed point, so the
// draw is a pure function of (logits, params, seed, step).
//
// Where this departs from the reference kernel: the reference takes exp((l - max) / T) from the special-function
// unit (__expf) and the min-p bound from logf, whose bit patterns belong to one GPU generation and to no CPU. Here
// both come from fixed_mass(), a sequence of IEEE single / double operations with explicit roundings (no contraction,
// no library call), so a host restatement of this file gives the same integer masses, the same thresholds and
// therefore the same token for every (logits, params, seed, step). The min-p bound is the smallest logit whose mass
// reaches min_p * 2^40, found by bisection over the ordered float keys.
// ---------------------------------------------------------------------------------------------------
constexpr int kSampleThreads = 1024;

struct SampleShared {
  uint32_t seen[(256 * 1024) / 32];
  unsigned long long hist[256];
  unsigned long long warp_u64[32];
  float warp_f[32];
  int warp_i[32];
  uint32_t pick_prefix;
  unsigned long long pick_above;
};

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// 2^40 * exp((l - max) * inv_t), truncated, in operations that round the same way on every IEEE machine:
// x = fl32(fl32(l - max) * inv_t); y = fl64(x * log2 e); n = floor(y + 1/2); f = y - n (exact); 2^f by a degree-13
// Taylor polynomial in Horner form with fused multiply-adds; the scaling by 2^(n + 40) is exact.
__device__ __forceinline__ unsigned long long fixed_mass(float l, float max_logit, float inv_t) {
  const float x = __fmul_rn(__fsub_rn(l, max_logit), inv_t);
  const double y = __dmul_rn(double(x), 1.4426950408889634);
  if (!(y > -64.0)) return 0ull;  // below 2^-24 of one fixed-point unit (also NaN and -inf)
  if (y > 0.0) return 1ull << 40; // l above the maximum cannot happen; keeps the shift below in range
  const double n = floor(__dadd_rn(y, 0.5));
  const double f = __dsub_rn(y, n);
  double p = 1.3691488853904128e-12;
  p = fma(p, f, 2.5678435993488206e-11);
  p = fma(p, f, 4.4455382718708116e-10);
  p = fma(p, f, 7.054911620801123e-09);
  p = fma(p, f, 1.01780860092397e-07);
  p = fma(p, f, 1.321548679014431e-06);
  p = fma(p, f, 1.5252733804059841e-05);
  p = fma(p, f, 0.0001540353039338161);
  p = fma(p, f, 0.0013333558146428443);
  p = fma(p, f, 0.009618129107628477);
  p = fma(p, f, 0.05550410866482158);
  p = fma(p, f, 0.24022650695910072);
  p = fma(p, f, 0.6931471805599453);
  p = fma(p, f, 1.0);
  const long long e = (long long)n + 40;  // -24 .. 40
  const double scale = __longlong_as_double((1023ll + e) << 52);
  return (unsigned long long)__dmul_rn(p, scale);
}

__device__ __forceinline__ float key_to_float(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Smallest ordered key whose logit keeps a mass of at least min_p * 2^40 (bisection between -FLT_MAX and the maximum).
__device__ uint32_t min_p_key(float max_logit, float inv_t, float min_p) {
  const unsigned long long cut = (unsigned long long)__dmul_rn(double(min_p), 1099511627776.0);
  uint32_t lo = 0x00800000u;  // key of -FLT_MAX
  uint32_t hi = (__float_as_uint(max_logit) & 0x80000000u) ? ~__float_as_uint(max_logit)
                                                           : (__float_as_uint(max_logit) | 0x80000000u);
  if (hi < lo) return hi;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (fixed_mass(key_to_float(mid), max_logit, inv_t) >= cut) hi = mid;
    else lo = mid + 1u;
  }
  return hi;
}

__device__ unsigned long long cta_sum_u64(unsigned long long v, SampleShared& sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sm.warp_u64[warp] = v;
  __syncthreads();
  unsigned long long total = 0;
  for (int w = 0; w < kSampleThreads / 32; ++w) total += sm.warp_u64[w];
  __syncthreads();
  return total;
}

// Radix select over the ordered keys of the candidates: finds the largest key K with
// weight(keys >= K) >= target, 8 bits per pass. `weigh(l)` is 1 for top-k, the fixed-point mass for top-p.
template <typename W>
__device__ uint32_t radix_threshold(const float* logits, int V, uint32_t floor_key, unsigned long long target,
                                    SampleShared& sm, W weigh) {
  uint32_t prefix = 0u, mask = 0u;
  unsigned long long above = 0ull;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kSampleThreads) sm.hist[i] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
      const float l = logits[i];
      const uint32_t key = order_key(l);
      if (key >= floor_key && (key & mask) == prefix) atomicAdd(&sm.hist[(key >> shift) & 255u], weigh(l));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long cum = above;
      int d = 255;
      for (; d > 0; --d) {
        if (cum + sm.hist[d] >= target) break;
        cum += sm.hist[d];
      }
      sm.pick_prefix = prefix | (uint32_t(d) << shift);
      sm.pick_above = cum;
    }
    __syncthreads();
    prefix = sm.pick_prefix;
    above = sm.pick_above;
    mask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(kSampleThreads, 1) sample_kernel(q38_sampling_args a) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  extern __shared__ __align__(16) uint8_t sample_smem[];
  SampleShared& sm = *reinterpret_cast<SampleShared*>(sample_smem);
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const q38_sampling_params_dev prm = a.params[b];
  float* logits = a.logits + (size_t)b * a.ld;
  const int V = a.vocab;
  const int slot = a.row_slot ? a.row_slot[b] : b;

  auto commit = [&](int tok, float logprob) {
    a.tokens_out[b] = tok;
    if (a.logprob_out) a.logprob_out[b] = logprob;
    if (a.history) {
      const int len = a.history_len[slot];
      a.history[(size_t)slot * a.history_cap + (len % a.history_cap)] = tok;
      a.history_len[slot] = len + 1;
    }
  };

  if ((prm.presence_penalty != 0.0f || prm.repetition_penalty != 1.0f) && a.history) {
    for (int i = tid; i < (V + 31) / 32; i += kSampleThreads) sm.seen[i] = 0u;
    __syncthreads();
    const int n = min(a.history_len[slot], a.history_cap);
    const int32_t* hist = a.history + (size_t)slot * a.history_cap;
    for (int i = tid; i < n; i += kSampleThreads) {
      const int t = hist[i];
      if (t < 0 || t >= V) continue;
      const uint32_t bit = 1u << (t & 31);
      if (atomicOr(&sm.seen[t >> 5], bit) & bit) continue;
      float l = logits[t];
      if (prm.repetition_penalty != 1.0f)
        l = l > 0.0f ? __fdiv_rn(l, prm.repetition_penalty) : __fmul_rn(l, prm.repetition_penalty);
      logits[t] = __fsub_rn(l, prm.presence_penalty);  // explicit roundings: no multiply-subtract contraction
    }
    __syncthreads();
  }

  // maximum with the lowest index among ties
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float l = logits[i];
    if (l > best) {
      best = l;
      best_i = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    sm.warp_f[warp] = best;
    sm.warp_i[warp] = best_i;
  }
  __syncthreads();
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    const float ov = sm.warp_f[w];
    const int oi = sm.warp_i[w];
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  __syncthreads();
  if (prm.temperature <= 0.0f) {
    if (tid == 0) commit(best_i, 0.0f);
    return;
  }
  const float M = best;
  const float inv_t = __fdiv_rn(1.0f, prm.temperature);
  auto mass = [&](float l) -> unsigned long long { return fixed_mass(l, M, inv_t); };

  uint32_t thresh = 0u;
  if (prm.top_k > 0 && prm.top_k < V)
    thresh = radix_threshold(logits, V, 0u, (unsigned long long)prm.top_k, sm, [](float) { return 1ull; });
  if (prm.min_p > 0.0f) thresh = max(thresh, min_p_key(M, inv_t, prm.min_p));
  if (prm.top_p < 1.0f) {
    unsigned long long local = 0ull;
    for (int i = tid; i < V; i += kSampleThreads) {
      const float l = logits[i];
      if (order_key(l) >= thresh) local += mass(l);
    }
    const unsigned long long kept = cta_sum_u64(local, sm);
    const unsigned long long target = (unsigned long long)__dmul_rn(double(prm.top_p), double(kept));
    thresh = max(thresh, radix_threshold(logits, V, thresh, target > 0 ? target : 1ull, sm, mass));
  }

  // inverse CDF in index order: thread t owns the contiguous ids [t * chunk, (t + 1) * chunk)
  const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
  const int i0 = tid * chunk, i1 = min(V, i0 + chunk);
  unsigned long long own = 0ull, all = 0ull;
  for (int i = i0; i < i1; ++i) {
    const float l = logits[i];
    const unsigned long long w = mass(l);
    all += w;
    if (order_key(l) >= thresh) own += w;
  }
  unsigned long long incl = own;
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) sm.warp_u64[warp] = incl;
  __syncthreads();
  unsigned long long before = incl - own, total = 0ull;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    const unsigned long long s = sm.warp_u64[w];
    if (w < warp) before += s;
    total += s;
  }
  __syncthreads();
  const unsigned long long all_sum = cta_sum_u64(all, sm);

  const int step = a.step ? a.step[b] : 0;
  const uint64_t r = mix64(prm.seed ^ (0xD1B54A32D192ED03ull * uint64_t(step + 1)));
  const double u01 = __dmul_rn(double(r >> 11), 1.0 / 9007199254740992.0);
  unsigned long long u = (unsigned long long)__dmul_rn(u01, double(total));
  if (u >= total) u = total - 1ull;  // double(total) may round up beyond 2^53: the draw stays inside the kept mass
  if (own > 0 && u >= before && u < before + own) {
    unsigned long long cum = before;
    int tok = -1, last = -1;
    for (int i = i0; i < i1; ++i) {
      const float l = logits[i];
      if (order_key(l) < thresh) continue;
      last = i;
      cum += mass(l);
      if (u < cum) {
        tok = i;
        break;
      }
    }
    if (tok < 0) tok = last;
    const double p = double(mass(logits[tok])) / double(all_sum > 0 ? all_sum : 1ull);
    commit(tok, float(log(p > 0.0 ? p : 1e-300)));
  }
}

// out[r] = log softmax(logits[r])[targets[r]], sums in double
// (reference src/kernels/kernels.h:258-260, src/kernels/sampling.cu:312-339).
__global__ void __launch_bounds__(256) target_logprob_kernel(const float* __restrict__ logits, int ld, int vocab,
                                                             const int32_t* __restrict__ targets,
                                                             float* __restrict__ out) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  __shared__ float red_f[8];
  __shared__ double red_d[8];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += 256) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  if (lane == 0) red_f[warp] = mx;
  __syncthreads();
  mx = red_f[0];
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
  double sum = 0.0;
  for (int i = tid; i < vocab; i += 256) sum += exp(double(row[i] - mx));
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red_d[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int w = 0; w < 8; ++w) total += red_d[w];
    const int t = targets[r];
    out[r] = (t >= 0 && t < vocab) ? float(double(row[t] - mx) - log(total)) : 0.0f;
  }
}

}  // namespace

unsigned int misc_error(bool clear) { return read_tu_error(clear); }
unsigned int* misc_error_address() { return tu_error_address(); }

}  // namespace q38

namespace q38 {
namespace {
// Rows `rows[i]` of the step's normalised-input arrays (bf16 hidden row + its norm partial sums) packed into
// rows i = 0..n-1: the LM-head input of the sequences that sample in a ragged step.
__global__ void __launch_bounds__(256) gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ partials,
                                                          const int* __restrict__ rows, int hidden, int blocks,
                                                          __nv_bfloat16* __restrict__ x_out,
                                                          float* __restrict__ partials_out) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x, src = rows[i];
  const uint4* from = reinterpret_cast<const uint4*>(x + (size_t)src * hidden);
  uint4* to = reinterpret_cast<uint4*>(x_out + (size_t)i * hidden);
  for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) to[c] = from[c];
  for (int c = threadIdx.x; c < blocks; c += blockDim.x) partials_out[(size_t)i * blocks + c] = partials[(size_t)src * blocks + c];
}
}  // namespace
}  // namespace q38

using namespace q38;

extern "C" int q38_gather_rows(const q38_bf16* x, const float* partials, const int* rows, int n, int hidden,
                               q38_bf16* x_out, float* partials_out, void* stream) {
  if (n == 0) return Q38_OK;
  Q38_REQUIRE(x && partials && rows && x_out && partials_out, "gather_rows: null argument");
  Q38_REQUIRE(n > 0 && hidden > 0 && hidden % 128 == 0, "gather_rows: n %d hidden %d", n, hidden);
  (void)launch_kernel(gather_rows_kernel, dim3(n), dim3(256), 0, as_stream(stream),
                      reinterpret_cast<const __nv_bfloat16*>(x), partials, rows, hidden, hidden / 128,
                      reinterpret_cast<__nv_bfloat16*>(x_out), partials_out);
  Q38_LAUNCH_OK("gather_rows_kernel");
  return Q38_OK;
}

extern "C" int q38_embed(const q38_bf16* table, const int32_t* tokens, int m, int hidden, float* residual,
                         q38_bf16* xbf, float* partials, void* stream) {
  if (m == 0) return Q38_OK;
  Q38_REQUIRE(table && tokens && residual && xbf && partials, "embed: null argument");
  Q38_REQUIRE(m > 0 && hidden > 0 && hidden % 128 == 0, "embed: m %d hidden %d", m, hidden);
  (void)launch_kernel(embed_kernel, dim3(m), dim3(256), 0, as_stream(stream), reinterpret_cast<const __nv_bfloat16*>(table), tokens, hidden,
                                                 residual, reinterpret_cast<__nv_bfloat16*>(xbf), partials);
  Q38_LAUNCH_OK("embed_kernel");
  return Q38_OK;
}

extern "C" int q38_residual_update(const float* delta, int m, int hidden, float* residual, q38_bf16* xbf,
                                   float* partials, void* stream) {
  if (m == 0) return Q38_OK;
  Q38_REQUIRE(delta && residual && xbf && partials, "residual_update: null argument");
  Q38_REQUIRE(m > 0 && hidden > 0 && hidden % 128 == 0, "residual_update: m %d hidden %d", m, hidden);
  (void)launch_kernel(residual_update_kernel, dim3(m), dim3(256), 0, as_stream(stream), delta, hidden, residual,
                      reinterpret_cast<__nv_bfloat16*>(xbf), partials);
  Q38_LAUNCH_OK("residual_update_kernel");
  return Q38_OK;
}

extern "C" int q38_pack_ragged(const int* seq_count, const int* seq_pos0, int num_seqs, int num_tokens,
                               int* seq_start, int* tok_pos, int* tok_seq, void* stream) {
  if (num_seqs == 0) return Q38_OK;
  Q38_REQUIRE(seq_count && seq_pos0 && seq_start && tok_pos && tok_seq, "pack_ragged: null argument");
  Q38_REQUIRE(num_seqs > 0 && num_tokens >= 0, "pack_ragged: sizes");
  (void)launch_kernel(pack_ragged_kernel, dim3(1), dim3(1024), 0, as_stream(stream), seq_count, seq_pos0, num_seqs, num_tokens, seq_start,
                                                        tok_pos, tok_seq);
  Q38_LAUNCH_OK("pack_ragged_kernel");
  return Q38_OK;
}

extern "C" int q38_sample(const q38_sampling_args* a, int batch, void* stream) {
  Q38_REQUIRE(a, "sample: null argument");
  Q38_REQUIRE(a->vocab > 0 && a->vocab <= 256 * 1024, "sample: vocab size %d", a->vocab);
  if (batch == 0) return Q38_OK;
  Q38_REQUIRE(a->logits && a->params && a->tokens_out, "sample: null pointer");
  static const cudaError_t attr =
      cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(SampleShared)));
  Q38_CUDA_OK(attr);
  (void)launch_kernel(sample_kernel, dim3(batch), dim3(kSampleThreads), sizeof(SampleShared), as_stream(stream), *a);
  Q38_LAUNCH_OK("sample_kernel");
  return Q38_OK;
}

extern "C" int q38_target_logprobs(const float* logits, int ld, int vocab, const int32_t* targets, int rows,
                                   float* out, void* stream) {
  if (rows == 0) return Q38_OK;
  Q38_REQUIRE(logits && targets && out && vocab > 0, "target_logprobs: arguments");
  (void)launch_kernel(target_logprob_kernel, dim3(rows), dim3(256), 0, as_stream(stream), logits, ld, vocab, targets, out);
  Q38_LAUNCH_OK("target_logprob_kernel");
  return Q38_OK;
}
