// TEST INFRASTRUCTURE — not part of the product.
//
// C-ABI shim around the UNMODIFIED reference CPU implementation (src/ref/ops.{h,cpp},
// src/bq_host.cpp, src/model_file.cpp of xetlan/qwen3.8-27b-cuda-kernel). It is compiled together
// with those reference sources, where they lie, into oracle/_ref/libq38_ref.so by oracle/Makefile
// (`make ref REF=<reference checkout>`). Nothing of the reference is copied into this repository;
// this file only forwards plain pointers to the reference's functions so that the tests can pin the
// oracle restatement (oracle/q38_oracle.cpp) against the reference itself.
#include <cstdint>
#include <cstring>
#include <vector>

#include "qwen38/bq.h"
#include "qwen38/common.h"
#include "qwen38/config.h"
#include "ref/ops.h"

using namespace qwen38;

namespace {

ModelConfig make_cfg(int nq, int nkv, int lk, int lv, float eps, double theta) {
  ModelConfig c;
  c.num_attention_heads = nq;
  c.num_key_value_heads = nkv;
  c.head_dim = 256;
  c.rotary_dim = 64;
  c.rope_theta = theta;
  c.linear_num_key_heads = lk;
  c.linear_num_value_heads = lv;
  c.linear_key_head_dim = 128;
  c.linear_value_head_dim = 128;
  c.linear_conv_kernel_dim = 4;
  c.rms_norm_eps = eps;
  return c;
}

}  // namespace

extern "C" {

// BQView::dequant_all over raw planes (src/bq_host.cpp:59-97).
void ref_bq_dequant(const uint8_t* lo, const uint8_t* hi, const uint16_t* scales, int bits, int64_t n, int64_t k,
                    float* out) {
  BQView v;
  v.bits = bits;
  v.n = n;
  v.k = k;
  v.rows = n;
  v.lo = lo;
  v.hi = hi;
  v.scales = scales;
  for (int64_t r = 0; r < n; ++r) v.dequant_row(r, out + r * k);
}

void ref_bq_codes(const uint8_t* lo, const uint8_t* hi, const uint16_t* scales, int bits, int64_t n, int64_t k,
                  int32_t* codes, uint16_t* scale_bits) {
  BQView v;
  v.bits = bits;
  v.n = n;
  v.k = k;
  v.rows = n;
  v.lo = lo;
  v.hi = hi;
  v.scales = scales;
  for (int64_t r = 0; r < n; ++r) {
    for (int64_t c = 0; c < k; ++c) codes[r * k + c] = v.code(r, c);
    for (int64_t g = 0; g < k / 64; ++g) scale_bits[r * (k / 64) + g] = v.scale_bits(r, g);
  }
}

float ref_norm_row_scale(const float* partials, int blocks, int hidden, float eps) {
  return ref::norm_row_scale(partials, blocks, hidden, eps);
}

void ref_norm_partials(const float* row, int hidden, float* partials) { ref::norm_partials(row, hidden, partials); }

// ref::qgemm (src/ref/ops.cpp:36-69). epilogue: 0 StoreBF16, 1 SwiGLU, 2 Residual, 3 StoreF32.
void ref_qgemm(const float* a, int m, const float* w_dequant, int n, int k, const float* row_scale, int epilogue,
               float* out, int ldo, float* residual, float* xbf, float* partials, int exact) {
  std::vector<float> w(w_dequant, w_dequant + size_t(n) * k);
  ref::GemmOut o{out, ldo, residual, xbf, partials};
  const ref::Epilogue ep = epilogue == 0   ? ref::Epilogue::StoreBF16
                           : epilogue == 1 ? ref::Epilogue::SwiGLU
                           : epilogue == 2 ? ref::Epilogue::Residual
                                           : ref::Epilogue::StoreF32;
  ref::qgemm(a, m, w, n, k, row_scale, ep, o, exact != 0);
}

void ref_int8_group_roundtrip(float* x, int n) { ref::int8_group_roundtrip(x, n); }

float ref_round_bf16(float x) { return round_bf16(x); }
float ref_round_f16(float x) { return round_f16(x); }

// ---- attention: a KvStore handle for one sequence and one layer --------------------------------
void* ref_kv_create(int kv_heads, int capacity) {
  auto* s = new ref::KvStore();
  s->resize(kv_heads, 256, capacity);
  return s;
}
void ref_kv_destroy(void* h) { delete static_cast<ref::KvStore*>(h); }
float* ref_kv_k(void* h) { return static_cast<ref::KvStore*>(h)->k.data(); }
float* ref_kv_v(void* h) { return static_cast<ref::KvStore*>(h)->v.data(); }

// kv_dtype: 0 f32, 1 bf16, 2 int8 (src/ref/ops.cpp:123-142)
void ref_qk_norm_rope_append(int nq, int nkv, float eps, double theta, const float* proj_row, int pos,
                             const float* q_norm, const float* k_norm, float* q_out, void* kv, int kv_dtype,
                             int exact) {
  const ModelConfig c = make_cfg(nq, nkv, 1, 1, eps, theta);
  const ref::KvDtype d = kv_dtype == 0 ? ref::KvDtype::F32 : kv_dtype == 1 ? ref::KvDtype::BF16 : ref::KvDtype::Int8;
  ref::qk_norm_rope_append(c, proj_row, pos, q_norm, k_norm, q_out, *static_cast<ref::KvStore*>(kv), d, exact != 0);
}

// src/ref/ops.cpp:144-171
void ref_attention_token(int nq, int nkv, const float* q, const float* gate, int pos, void* kv, float* out,
                         int exact) {
  const ModelConfig c = make_cfg(nq, nkv, 1, 1, 1e-6f, 1e7);
  ref::attention_token(c, q, gate, pos, *static_cast<ref::KvStore*>(kv), out, exact != 0);
}

// ---- GDN: state is caller-owned: s [lv][128][128], conv [3][conv_dim] (src/ref/ops.cpp:173-242) --
void ref_gdn_token(int lk, int lv, float eps, const float* proj_row, const float* ab_row, const float* conv_w,
                   const float* A, const float* dt_bias, const float* norm_w, float* state_s, float* state_conv,
                   float* out, int exact) {
  const ModelConfig c = make_cfg(1, 1, lk, lv, eps, 1e7);
  const int conv_dim = c.gdn_conv_dim();
  ref::GdnState st;
  st.s.assign(state_s, state_s + size_t(lv) * 128 * 128);
  st.conv.assign(state_conv, state_conv + size_t(3) * conv_dim);
  ref::gdn_token(c, proj_row, ab_row, conv_w, A, dt_bias, norm_w, st, out, exact != 0);
  std::memcpy(state_s, st.s.data(), st.s.size() * 4);
  std::memcpy(state_conv, st.conv.data(), st.conv.size() * 4);
}

}  // extern "C"
