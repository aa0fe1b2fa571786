// TEST INFRASTRUCTURE — the CPU oracle. Never linked into, imported by or called from the product
// path; only the tests, the smoke check and the benchmark's CPU-baseline leg may use it.
//
// A plain C++ restatement (own code, C ABI, raw float arrays) of the reference CPU model of
// xetlan/qwen3.8-27b-cuda-kernel in "engine mode": every operation of the ragged step with the
// rounding points of the CUDA engine (bf16 activations, fp16 queries, int8 KV with fp16 scales).
// Each function names the reference file:line it follows. Accumulation order and widths (double
// dot products, fp32 state) are the reference's, so that on identical inputs the results are
// bit-identical with the reference build in oracle/_ref (tests/test_oracle_pins.py checks this).
//
// Parity status: PINNED — against oracle/_ref (the unmodified reference sources compiled here) and
// against the golden vectors in tests/golden/ produced from the reference's own code.
#include <algorithm>
#include <bit>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// Static row partition over host threads (results do not depend on the thread count: every output
// element is produced by exactly one thread with a fixed summation order).
template <typename F>
void parallel_rows(int64_t n, F&& body) {
  static const unsigned hw = [] {
    const char* e = std::getenv("Q38_ORACLE_THREADS");
    const unsigned want = e ? unsigned(std::atoi(e)) : std::thread::hardware_concurrency();
    return std::max(1u, std::min(want, 64u));
  }();
  const int64_t workers = std::min<int64_t>(hw, n);
  if (workers <= 1) {
    for (int64_t i = 0; i < n; ++i) body(i);
    return;
  }
  std::vector<std::thread> pool;
  for (int64_t w = 0; w < workers; ++w)
    pool.emplace_back([=, &body] {
      for (int64_t i = n * w / workers; i < n * (w + 1) / workers; ++i) body(i);
    });
  for (auto& t : pool) t.join();
}

// ---- 16-bit float rounding (include/qwen38/common.h:38-83) ---------------------------------------
inline float bf16_bits_to_f32(uint16_t b) { return std::bit_cast<float>(uint32_t(b) << 16); }

inline uint16_t f32_to_bf16_bits(float f) {
  const uint32_t u = std::bit_cast<uint32_t>(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40u);
  return uint16_t((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

inline float rbf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

inline float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 31u, m = h & 1023u;
  if (e == 0) {
    if (!m) return std::bit_cast<float>(sign);
    const float v = std::ldexp(float(m), -24);
    return sign ? -v : v;
  }
  if (e == 31) return std::bit_cast<float>(sign | 0x7f800000u | (m << 13));
  return std::bit_cast<float>(sign | ((e + 112u) << 23) | (m << 13));
}

inline uint16_t f32_to_f16_bits(float f) {
  const uint32_t u = std::bit_cast<uint32_t>(f);
  const uint32_t sign = (u >> 16) & 0x8000u, mag = u & 0x7fffffffu;
  if (mag > 0x7f800000u) return uint16_t(sign | 0x7e00u);
  if (mag >= 0x477ff000u) return uint16_t(sign | 0x7c00u);
  if (mag < 0x38800000u) {
    const float scaled = std::bit_cast<float>(mag) * 16777216.0f;
    return uint16_t(sign | uint32_t(std::nearbyint(scaled)));
  }
  const uint32_t v = (mag + 0xfffu + ((mag >> 13) & 1u)) >> 13;
  return uint16_t(sign | (v - (112u << 10)));
}

inline float rf16(float f) { return f16_bits_to_f32(f32_to_f16_bits(f)); }

inline float silu_f(float x) { return x / (1.0f + std::exp(-x)); }             // src/ref/ops.h:21
inline float sigmoid_f(float x) { return 1.0f / (1.0f + std::exp(-x)); }       // src/ref/ops.h:22
inline float softplus_f(float x) { return x > 20.0f ? x : std::log1p(std::exp(x)); }  // src/ref/ops.h:23

inline uint32_t rd32(const uint8_t* p) {
  uint32_t v;
  std::memcpy(&v, p, 4);
  return v;
}

// Where element (n, k) of a BQ matrix lives (docs/FORMAT.md 2.2; src/bq_host.cpp:37-57).
struct Where {
  int64_t slab;
  int lane, pair, elem;
};

inline Where where_is(int64_t n, int64_t k, int64_t K) {
  const int nl = int(n & 63), kl = int(k & 15);
  Where w;
  w.slab = (n >> 6) * (K >> 4) + (k >> 4);
  w.lane = 4 * (nl & 7) + ((kl & 7) >> 1);
  w.pair = 2 * (nl >> 3) + (kl >> 3);
  w.elem = kl & 1;
  return w;
}

inline unsigned nibble(const uint8_t* plane, const Where& w) {
  const uint32_t word = rd32(plane + w.slab * 512 + w.lane * 16 + 4 * (w.pair >> 2));
  return (word >> ((w.elem ? 16 : 0) + 4 * (w.pair & 3))) & 15u;
}

inline int code_at(const uint8_t* lo, const uint8_t* hi, int bits, int64_t n, int64_t k, int64_t K) {
  const Where w = where_is(n, k, K);
  unsigned u = nibble(lo, w);
  if (bits == 5) {
    u |= ((rd32(hi + w.slab * 128 + w.lane * 4) >> ((w.elem ? 16 : 0) + w.pair)) & 1u) << 4;
  } else if (bits == 6) {
    const uint32_t word = rd32(hi + w.slab * 256 + w.lane * 8 + 4 * (w.pair >> 3));
    u |= ((word >> ((w.elem ? 16 : 0) + 2 * (w.pair & 7))) & 3u) << 4;
  } else if (bits == 8) {
    u |= nibble(hi, w) << 4;
  }
  return int(u) - (1 << (bits - 1));
}

inline uint16_t scale_bits_at(const uint16_t* scales, int64_t n, int64_t g, int64_t K) {
  const int nl = int(n & 63);
  return scales[((n >> 6) * (K >> 6) + g) * 64 + (nl & 7) * 8 + (nl >> 3)];
}

}  // namespace

extern "C" {

float orc_round_bf16(float x) { return rbf16(x); }
float orc_round_f16(float x) { return rf16(x); }

// Signed codes and scale bits of a BQ tensor (src/bq_host.cpp:59-82).
void orc_bq_codes(const uint8_t* lo, const uint8_t* hi, const uint16_t* scales, int bits, int64_t n, int64_t k,
                  int32_t* codes, uint16_t* scale_bits) {
  parallel_rows(n, [&](int64_t r) {
    for (int64_t c = 0; c < k; ++c) codes[r * k + c] = code_at(lo, hi, bits, r, c, k);
    for (int64_t g = 0; g < k / 64; ++g) scale_bits[r * (k / 64) + g] = scale_bits_at(scales, r, g, k);
  });
}

// W[n][k] = bf16(float(code) * float(scale)) (docs/FORMAT.md 2.1; src/bq_host.cpp:84-97).
void orc_bq_dequant(const uint8_t* lo, const uint8_t* hi, const uint16_t* scales, int bits, int64_t n, int64_t k,
                    float* out) {
  parallel_rows(n, [&](int64_t r) {
    for (int64_t c = 0; c < k; ++c)
      out[r * k + c] =
          rbf16(float(code_at(lo, hi, bits, r, c, k)) * bf16_bits_to_f32(scale_bits_at(scales, r, c >> 6, k)));
  });
}

// src/ref/ops.cpp:10-14
float orc_norm_row_scale(const float* partials, int blocks, int hidden, float eps) {
  float sum = 0.0f;
  for (int b = 0; b < blocks; ++b) sum += partials[b];
  return 1.0f / std::sqrt(sum / float(hidden) + eps);
}

// src/ref/ops.cpp:16-22
void orc_norm_partials(const float* row, int hidden, float* partials) {
  for (int b = 0; b < hidden / 128; ++b) {
    double s = 0;
    for (int i = 0; i < 128; ++i) s += double(row[b * 128 + i]) * row[b * 128 + i];
    partials[b] = float(s);
  }
}

// C[m][n] = sum_k A[m][k] W[n][k], double accumulation in k order (src/ref/ops.cpp:24-34).
void orc_matmul_nt(const float* a, int m, int k, const float* w, int n, float* c) {
  parallel_rows(n, [&](int64_t j) {
    const float* wr = w + j * int64_t(k);
    for (int i = 0; i < m; ++i) {
      const float* ar = a + int64_t(i) * k;
      double acc = 0;
      for (int t = 0; t < k; ++t) acc += double(ar[t]) * wr[t];
      c[int64_t(i) * n + j] = float(acc);
    }
  });
}

// One quantized projection with a fused epilogue (src/ref/ops.cpp:36-69).
// epilogue: 0 StoreBF16, 1 SwiGLU, 2 Residual, 3 StoreF32.
void orc_qgemm(const float* a, int m, const float* w, int n, int k, const float* row_scale, int epilogue, float* out,
               int ldo, float* residual, float* xbf, float* partials, int exact) {
  std::vector<float> c(size_t(m) * n);
  orc_matmul_nt(a, m, k, w, n, c.data());
  for (int i = 0; i < m; ++i) {
    const float rs = row_scale ? row_scale[i] : 1.0f;
    const float* cr = c.data() + size_t(i) * n;
    if (epilogue == 0) {
      for (int j = 0; j < n; ++j) out[size_t(i) * ldo + j] = exact ? cr[j] * rs : rbf16(cr[j] * rs);
    } else if (epilogue == 3) {
      for (int j = 0; j < n; ++j) out[size_t(i) * ldo + j] = cr[j] * rs;
    } else if (epilogue == 1) {
      for (int j = 0; j < n / 2; ++j) {
        const float g = cr[2 * j] * rs, u = cr[2 * j + 1] * rs;
        const float v = silu_f(g) * u;
        out[size_t(i) * ldo + j] = exact ? v : rbf16(v);
      }
    } else {
      float* res = residual + size_t(i) * n;
      float* xb = xbf + size_t(i) * n;
      for (int j = 0; j < n; ++j) {
        res[j] += cr[j];
        xb[j] = exact ? res[j] : rbf16(res[j]);
      }
      orc_norm_partials(res, n, partials + size_t(i) * (n / 128));
    }
  }
}

// Symmetric int8 quantize-dequantize per 64 values with an fp16 scale (src/ref/ops.cpp:79-90).
void orc_int8_group_roundtrip(float* x, int n) {
  for (int g0 = 0; g0 < n; g0 += 64) {
    float amax = 0.0f;
    for (int i = 0; i < 64; ++i) amax = std::max(amax, std::fabs(x[g0 + i]));
    const float scale = rf16(amax / 127.0f);
    for (int i = 0; i < 64; ++i) {
      float q = 0.0f;
      if (scale > 0.0f) q = std::clamp(std::nearbyint(x[g0 + i] / scale), -127.0f, 127.0f);
      x[g0 + i] = q * scale;
    }
  }
}

// The same quantisation, returning the stored bytes: q int8 [n], scale fp16 bits [n / 64].
void orc_int8_group_quantize(const float* x, int n, int8_t* q, uint16_t* scale_bits) {
  for (int g0 = 0; g0 < n; g0 += 64) {
    float amax = 0.0f;
    for (int i = 0; i < 64; ++i) amax = std::max(amax, std::fabs(x[g0 + i]));
    const uint16_t sb = f32_to_f16_bits(amax / 127.0f);
    const float scale = f16_bits_to_f32(sb);
    scale_bits[g0 / 64] = sb;
    for (int i = 0; i < 64; ++i) {
      float v = 0.0f;
      if (scale > 0.0f) v = std::clamp(std::nearbyint(x[g0 + i] / scale), -127.0f, 127.0f);
      q[g0 + i] = int8_t(v);
    }
  }
}

namespace {

// src/ref/ops.cpp:94-99
void offset_rmsnorm(const float* x, int n, const float* w, float eps, float* y) {
  double ss = 0;
  for (int i = 0; i < n; ++i) ss += double(x[i]) * x[i];
  const float r = 1.0f / std::sqrt(float(ss / n) + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * r * w[i];
}

// src/ref/ops.cpp:101-111: pairs (i, i + rotary/2), fp32 angle = float(pos) * inv_freq
void rope_partial(float* y, int rotary_dim, int pos, double theta) {
  const int half = rotary_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float inv = 1.0f / std::pow(float(theta), float(2 * i) / float(rotary_dim));
    const float angle = float(pos) * inv;
    const float c = std::cos(angle), s = std::sin(angle);
    const float x1 = y[i], x2 = y[i + half];
    y[i] = x1 * c - x2 * s;
    y[i + half] = x2 * c + x1 * s;
  }
}

// src/ref/ops.cpp:113-121
void store_kv_row(float* dst, const float* src, int n, int kv_dtype, bool exact) {
  std::copy(src, src + n, dst);
  if (exact || kv_dtype == 0) return;
  if (kv_dtype == 1) {
    for (int i = 0; i < n; ++i) dst[i] = rbf16(dst[i]);
  } else {
    orc_int8_group_roundtrip(dst, n);
  }
}

}  // namespace

// The 32 inverse RoPE frequencies exactly as the reference evaluates them (src/ref/ops.cpp:104).
void orc_rope_inv_freq(double theta, int rotary_dim, float* out) {
  for (int i = 0; i < rotary_dim / 2; ++i)
    out[i] = 1.0f / std::pow(float(theta), float(2 * i) / float(rotary_dim));
}

// q/k offset-RMSNorm, partial RoPE, KV append for one token (src/ref/ops.cpp:123-142).
// k_store / v_store: [kv_heads][capacity][256] dequantised cache of one sequence and layer.
// kv_dtype: 0 f32, 1 bf16, 2 int8.
void orc_qk_norm_rope_append(int nq, int nkv, float eps, double theta, const float* proj_row, int pos,
                             const float* q_norm, const float* k_norm, float* q_out, float* k_store, float* v_store,
                             int capacity, int kv_dtype, int exact) {
  const int hd = 256, rot = 64;
  float y[256];
  for (int h = 0; h < nq; ++h) {
    offset_rmsnorm(proj_row + size_t(h) * hd, hd, q_norm, eps, y);
    rope_partial(y, rot, pos, theta);
    for (int d = 0; d < hd; ++d) q_out[size_t(h) * hd + d] = exact ? y[d] : rf16(y[d]);
  }
  const float* kbase = proj_row + size_t(2) * nq * hd;
  const float* vbase = kbase + size_t(nkv) * hd;
  for (int h = 0; h < nkv; ++h) {
    offset_rmsnorm(kbase + size_t(h) * hd, hd, k_norm, eps, y);
    rope_partial(y, rot, pos, theta);
    store_kv_row(k_store + (size_t(h) * capacity + pos) * hd, y, hd, kv_dtype, exact != 0);
    store_kv_row(v_store + (size_t(h) * capacity + pos) * hd, vbase + size_t(h) * hd, hd, kv_dtype, exact != 0);
  }
}

// Causal GQA attention of one query token over positions [0, pos], then the sigmoid output gate
// (src/ref/ops.cpp:144-171).
void orc_attention_token(int nq, int nkv, const float* q, const float* gate, int pos, const float* k_store,
                         const float* v_store, int capacity, float* out, int exact) {
  const int hd = 256, group = nq / nkv;
  const double scale = 1.0 / std::sqrt(double(hd));
  parallel_rows(nq, [&](int64_t h) {
    std::vector<double> s(size_t(pos) + 1);
    const int kvh = int(h) / group;
    double mx = -1e300;
    for (int j = 0; j <= pos; ++j) {
      const float* kr = k_store + (size_t(kvh) * capacity + j) * hd;
      double dot = 0;
      for (int d = 0; d < hd; ++d) dot += double(q[size_t(h) * hd + d]) * kr[d];
      s[j] = dot * scale;
      mx = std::max(mx, s[j]);
    }
    double l = 0;
    for (int j = 0; j <= pos; ++j) {
      s[j] = std::exp(s[j] - mx);
      l += s[j];
    }
    std::vector<double> o(hd, 0.0);
    for (int j = 0; j <= pos; ++j) {
      const float* vr = v_store + (size_t(kvh) * capacity + j) * hd;
      const double p = s[j];
      for (int d = 0; d < hd; ++d) o[d] += p * vr[d];
    }
    for (int d = 0; d < hd; ++d) {
      const float val = float(o[d] / l) * sigmoid_f(gate[size_t(h) * hd + d]);
      out[size_t(h) * hd + d] = exact ? val : rbf16(val);
    }
  });
}

// Full Gated DeltaNet mixer for one token: causal conv + SiLU, q/k L2 norm, gates, 128x128
// recurrence, gated RMSNorm (src/ref/ops.cpp:173-242). state_s [lv][128 dv][128 dk],
// state_conv [3][conv_dim] oldest first; both updated in place.
void orc_gdn_token(int lk, int lv, float eps, const float* proj_row, const float* ab_row, const float* conv_w,
                   const float* A, const float* dt_bias, const float* norm_w, float* state_s, float* state_conv,
                   float* out, int exact) {
  const int dk = 128, dv = 128, taps = 4;
  const int conv_dim = 2 * lk * dk + lv * dv;
  const int ratio = lv / lk;
  std::vector<float> act(conv_dim);
  for (int c = 0; c < conv_dim; ++c) {
    float acc = 0.0f;
    for (int j = 0; j < taps - 1; ++j) acc += conv_w[size_t(c) * taps + j] * state_conv[size_t(j) * conv_dim + c];
    acc += conv_w[size_t(c) * taps + taps - 1] * proj_row[c];
    act[c] = silu_f(acc);
  }
  std::memmove(state_conv, state_conv + conv_dim, size_t(taps - 2) * conv_dim * sizeof(float));
  std::memcpy(state_conv + size_t(taps - 2) * conv_dim, proj_row, size_t(conv_dim) * sizeof(float));

  float* qall = act.data();
  float* kall = act.data() + size_t(lk) * dk;
  const float* vall = act.data() + size_t(2) * lk * dk;
  const float* z = proj_row + conv_dim;
  const float qscale = 1.0f / std::sqrt(float(dk));
  for (int h = 0; h < lk; ++h) {
    float* vecs[2] = {qall + size_t(h) * dk, kall + size_t(h) * dk};
    for (float* vec : vecs) {
      double ss = 0;
      for (int d = 0; d < dk; ++d) ss += double(vec[d]) * vec[d];
      const float r = 1.0f / std::sqrt(float(ss) + 1e-6f);
      for (int d = 0; d < dk; ++d) vec[d] *= r;
    }
    for (int d = 0; d < dk; ++d) qall[size_t(h) * dk + d] *= qscale;
  }

  for (int j = 0; j < lv; ++j) {
    const float* q = qall + size_t(j / ratio) * dk;
    const float* k = kall + size_t(j / ratio) * dk;
    const float* v = vall + size_t(j) * dv;
    const float beta = sigmoid_f(ab_row[j]);
    const float decay = std::exp(A[j] * softplus_f(ab_row[lv + j] + dt_bias[j]));
    float* S = state_s + size_t(j) * dv * dk;
    float o[128];
    for (int a = 0; a < dv; ++a) {
      float* row = S + size_t(a) * dk;
      float kv_mem = 0.0f;
      for (int b = 0; b < dk; ++b) {
        row[b] *= decay;
        kv_mem += row[b] * k[b];
      }
      const float delta = beta * (v[a] - kv_mem);
      float acc = 0.0f;
      for (int b = 0; b < dk; ++b) {
        row[b] += delta * k[b];
        acc += row[b] * q[b];
      }
      o[a] = acc;
    }
    double ss = 0;
    for (int a = 0; a < dv; ++a) ss += double(o[a]) * o[a];
    const float r = 1.0f / std::sqrt(float(ss / dv) + eps);
    for (int a = 0; a < dv; ++a) {
      const float val = o[a] * r * norm_w[a] * silu_f(z[size_t(j) * dv + a]);
      out[size_t(j) * dv + a] = exact ? val : rbf16(val);
    }
  }
}

// Greedy choice: the lowest id among the maxima (src/apps/ref_main.cpp:77).
int orc_greedy(const float* logits, int vocab) {
  int best = 0;
  for (int i = 1; i < vocab; ++i)
    if (logits[i] > logits[best]) best = i;
  return best;
}

// log softmax(logits)[target] in double (restates the scoring rule of src/kernels/sampling.cu:312-339).
float orc_target_logprob(const float* logits, int vocab, int target) {
  double mx = -1e300;
  for (int i = 0; i < vocab; ++i) mx = std::max(mx, double(logits[i]));
  double z = 0;
  for (int i = 0; i < vocab; ++i) z += std::exp(double(logits[i]) - mx);
  return float(double(logits[target]) - mx - std::log(z));
}

// ---------------------------------------------------------------------------------------------------
// Stochastic sampler (restates the engine's sampling kernel, which follows the definition of the reference's
// src/kernels/sampling.cu:137-310: penalties once per distinct history token, top-k / min-p / top-p cuts on the
// ordered logit keys, 2^-40 fixed-point masses, splitmix64 inverse-CDF draw in index order). The reference has no CPU
// sampler; this restatement and the kernel share one arithmetic definition made of IEEE operations only (explicit
// single / double roundings, fused multiply-adds, no library exp or log), so the two must agree bit for bit.
// ---------------------------------------------------------------------------------------------------
namespace {

inline uint32_t order_key(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
inline float key_to_float(uint32_t key) {
  const uint32_t u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
  float x;
  std::memcpy(&x, &u, 4);
  return x;
}

#if defined(__x86_64__)
__attribute__((target("fma"))) double poly_fma_hw(double f) {
  double p = 1.3691488853904128e-12;
  const double c[] = {2.5678435993488206e-11, 4.4455382718708116e-10, 7.054911620801123e-09, 1.01780860092397e-07,
                      1.321548679014431e-06,  1.5252733804059841e-05, 0.0001540353039338161, 0.0013333558146428443,
                      0.009618129107628477,   0.05550410866482158,    0.24022650695910072,   0.6931471805599453,
                      1.0};
  for (double ck : c) p = __builtin_fma(p, f, ck);
  return p;
}
#endif
double poly_fma_sw(double f) {
  double p = 1.3691488853904128e-12;
  const double c[] = {2.5678435993488206e-11, 4.4455382718708116e-10, 7.054911620801123e-09, 1.01780860092397e-07,
                      1.321548679014431e-06,  1.5252733804059841e-05, 0.0001540353039338161, 0.0013333558146428443,
                      0.009618129107628477,   0.05550410866482158,    0.24022650695910072,   0.6931471805599453,
                      1.0};
  for (double ck : c) p = std::fma(p, f, ck);  // correctly rounded in software where the CPU has no FMA unit
  return p;
}
double exp2_fraction(double f) {
#if defined(__x86_64__)
  static const bool hw = __builtin_cpu_supports("fma");
  if (hw) return poly_fma_hw(f);
#endif
  return poly_fma_sw(f);
}

// 2^40 * exp((l - max) * inv_t), truncated: the operation sequence of the kernel's fixed_mass().
uint64_t fixed_mass(float l, float max_logit, float inv_t) {
  volatile float d = l - max_logit;  // volatile: each step rounds to its declared width
  volatile float x = d * inv_t;
  volatile double y = double(x) * 1.4426950408889634;
  if (!(y > -64.0)) return 0;
  if (y > 0.0) return uint64_t(1) << 40;
  volatile double yh = y + 0.5;
  const double n = std::floor(yh);
  volatile double f = y - n;
  const double p = exp2_fraction(f);
  const int64_t e = int64_t(n) + 40;
  const uint64_t bits = uint64_t(1023 + e) << 52;
  double scale;
  std::memcpy(&scale, &bits, 8);
  volatile double scaled = p * scale;
  return uint64_t(scaled);
}

uint32_t min_p_key(float max_logit, float inv_t, float min_p) {
  volatile double c = double(min_p) * 1099511627776.0;
  const uint64_t cut = uint64_t(c);
  uint32_t lo = 0x00800000u, hi = order_key(max_logit);
  if (hi < lo) return hi;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (fixed_mass(key_to_float(mid), max_logit, inv_t) >= cut) hi = mid;
    else lo = mid + 1;
  }
  return hi;
}

inline uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

}  // namespace

// Penalties in place: every distinct token among the first min(len, cap) history entries is penalised once.
void orc_sample_penalties(float* logits, int vocab, const int32_t* history, int len, int cap, float presence,
                          float repetition) {
  if (presence == 0.0f && repetition == 1.0f) return;
  std::vector<bool> seen(size_t(vocab), false);
  const int n = std::min(len, cap);
  for (int i = 0; i < n; ++i) {
    const int t = history[i];
    if (t < 0 || t >= vocab || seen[size_t(t)]) continue;
    seen[size_t(t)] = true;
    volatile float l = logits[t];
    if (repetition != 1.0f) l = l > 0.0f ? l / repetition : l * repetition;
    volatile float r = l - presence;
    logits[t] = r;
  }
}

// `count` draws from one (already penalised) logits row with one parameter set and per-draw (seed, step).
// tokens_out / logprob_out as the kernel reports them; temperature <= 0 gives the lowest-id argmax and logprob 0.
void orc_sample_draws(const float* logits, int vocab, float temperature, int top_k, float top_p, float min_p,
                      const uint64_t* seeds, const int32_t* steps, int count, int32_t* tokens_out, float* logprob_out) {
  int best = 0;
  for (int i = 1; i < vocab; ++i)
    if (logits[i] > logits[best]) best = i;
  if (temperature <= 0.0f) {
    for (int d = 0; d < count; ++d) {
      tokens_out[d] = best;
      logprob_out[d] = 0.0f;
    }
    return;
  }
  const float M = logits[best];
  volatile float inv_t_v = 1.0f / temperature;
  const float inv_t = inv_t_v;
  std::vector<uint64_t> mass(static_cast<size_t>(vocab));
  std::vector<uint32_t> key(static_cast<size_t>(vocab));
  uint64_t all_sum = 0;
  for (int i = 0; i < vocab; ++i) {
    mass[size_t(i)] = fixed_mass(logits[i], M, inv_t);
    key[size_t(i)] = order_key(logits[i]);
    all_sum += mass[size_t(i)];
  }
  uint32_t thresh = 0;
  if (top_k > 0 && top_k < vocab) {  // the k-th largest key: every logit that ties with it stays
    std::vector<uint32_t> tmp(key);
    std::nth_element(tmp.begin(), tmp.begin() + (top_k - 1), tmp.end(), std::greater<uint32_t>());
    thresh = tmp[size_t(top_k - 1)];
  }
  if (min_p > 0.0f) thresh = std::max(thresh, min_p_key(M, inv_t, min_p));
  if (top_p < 1.0f) {
    std::vector<std::pair<uint32_t, uint64_t>> cand;
    uint64_t kept = 0;
    for (int i = 0; i < vocab; ++i)
      if (key[size_t(i)] >= thresh) {
        cand.emplace_back(key[size_t(i)], mass[size_t(i)]);
        kept += mass[size_t(i)];
      }
    volatile double tv = double(top_p) * double(kept);
    uint64_t target = uint64_t(tv);
    if (target == 0) target = 1;
    std::sort(cand.begin(), cand.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
    uint64_t cum = 0;
    uint32_t cut = thresh;
    for (size_t i = 0; i < cand.size();) {  // whole groups of equal keys: the largest key whose tail mass reaches the target
      size_t j = i;
      while (j < cand.size() && cand[j].first == cand[i].first) cum += cand[j++].second;
      if (cum >= target) {
        cut = cand[i].first;
        break;
      }
      i = j;
    }
    thresh = std::max(thresh, cut);
  }
  std::vector<uint64_t> prefix(static_cast<size_t>(vocab) + 1, 0);  // kept mass before index i
  for (int i = 0; i < vocab; ++i) prefix[size_t(i) + 1] = prefix[size_t(i)] + (key[size_t(i)] >= thresh ? mass[size_t(i)] : 0);
  const uint64_t total = prefix[size_t(vocab)];
  for (int d = 0; d < count; ++d) {
    const uint64_t r = mix64(seeds[d] ^ (0xD1B54A32D192ED03ull * uint64_t(steps[d] + 1)));
    volatile double u01 = double(r >> 11) * (1.0 / 9007199254740992.0);
    volatile double ud = u01 * double(total);
    uint64_t u = uint64_t(ud);
    if (u >= total) u = total - 1;
    // first index whose inclusive kept mass exceeds u
    const size_t at = size_t(std::upper_bound(prefix.begin() + 1, prefix.end(), u) - (prefix.begin() + 1));
    tokens_out[d] = int32_t(at);
    const double p = double(mass[at]) / double(all_sum > 0 ? all_sum : 1);
    logprob_out[d] = float(std::log(p > 0.0 ? p : 1e-300));
  }
}

}  // extern "C"
