// C++ face of the kernel library: namespace qwen38::kernels with the descriptor types and launcher
// signatures the reference engine's internal kernel API declares (reference src/kernels/kernels.h), each
// launcher forwarding to the C ABI of include/q38_kernels.h. This header is the whole binding a host that
// was written against the reference needs: include it instead of the reference's kernels.h and link
// libq38_kernels.so instead of the reference's kernel objects.
//
// Contract (unchanged): launchers are asynchronous on `stream`, allocate nothing, never synchronise and
// may be captured into a CUDA graph. A failed argument check throws qwen38::Error with the library's
// message, as the reference launchers do.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "q38_kernels.h"

namespace qwen38 {
[[noreturn]] void throw_kernel_error(const char* message);  // throws qwen38::Error
}

namespace qwen38::kernels {

namespace detail {
inline void ok(int rc) {
  if (rc != Q38_OK) throw_kernel_error(q38_last_error());
}
}  // namespace detail

struct BatchDesc {
  int num_seqs = 0, num_tokens = 0, max_tokens_per_seq = 0;
  const int* seq_start = nullptr;
  const int* seq_slot = nullptr;
  const int* seq_pos0 = nullptr;
  const int* tok_pos = nullptr;
  const int* tok_seq = nullptr;
  q38_batch_desc c() const {
    return {num_seqs, num_tokens, max_tokens_per_seq, seq_start, seq_slot, seq_pos0, tok_pos, tok_seq};
  }
};

enum class KvDtype : int { Int8 = Q38_KV_INT8, BF16 = Q38_KV_BF16 };
constexpr int kPageTokens = Q38_PAGE_TOKENS;
constexpr int kHeadDim = Q38_HEAD_DIM;

struct KvCacheDesc {
  uint8_t* pool = nullptr;
  KvDtype dtype = KvDtype::Int8;
  int kv_heads = 0, num_pages = 0;
  size_t page_bytes = 0, layer_stride = 0;
  const int* block_table = nullptr;
  int max_pages_per_seq = 0;

  size_t elem_bytes() const { return dtype == KvDtype::Int8 ? 1 : 2; }
  size_t k_offset(int head, int tok) const { return (size_t(head) * kPageTokens + tok) * kHeadDim * elem_bytes(); }
  size_t v_offset(int head, int tok) const {
    return size_t(kv_heads) * kPageTokens * kHeadDim * elem_bytes() + k_offset(head, tok);
  }
  size_t ks_offset(int head, int tok) const {
    return 2 * size_t(kv_heads) * kPageTokens * kHeadDim + (size_t(head) * kPageTokens + tok) * 8;
  }
  size_t vs_offset(int head, int tok) const { return ks_offset(head, tok) + size_t(kv_heads) * kPageTokens * 8; }
  static size_t page_bytes_for(KvDtype d, int kv_heads) { return q38_kv_page_bytes(int(d), kv_heads); }
  q38_kv_cache_desc c() const {
    return {pool, int(dtype), kv_heads, num_pages, page_bytes, layer_stride, block_table, max_pages_per_seq};
  }
};

enum class Epilogue : int {
  StoreBF16 = Q38_EPI_STORE_BF16,
  SwiGLU = Q38_EPI_SWIGLU,
  Residual = Q38_EPI_RESIDUAL,
  StoreF32 = Q38_EPI_STORE_F32,
};

struct BQWeight {
  const uint8_t* lo = nullptr;
  const uint8_t* hi = nullptr;
  const __nv_bfloat16* scales = nullptr;
  int bits = 4, n = 0, k = 0, rows = 0;
  q38_bq_weight c() const { return {lo, hi, reinterpret_cast<const q38_bf16*>(scales), bits, n, k, rows}; }
};

struct GemmEpilogue {
  Epilogue kind = Epilogue::StoreBF16;
  void* out = nullptr;
  int ldo = 0, n_store = 0;
  float* residual = nullptr;
  __nv_bfloat16* xbf = nullptr;
  float* partials_out = nullptr;
  const float* partials_in = nullptr;
  int hidden = 0;
  float eps = 1e-6f;
  q38_gemm_epilogue c() const {
    return {int(kind), out, ldo, n_store, residual, reinterpret_cast<q38_bf16*>(xbf), partials_out, partials_in,
            hidden, eps};
  }
};

struct GemmWorkspace {
  float* partials = nullptr;
  size_t partial_floats = 0;
  int* counters = nullptr;
  int num_counters = 0;
};

constexpr int kGemmConfigAuto = Q38_GEMM_CONFIG_AUTO;
inline int qgemm_num_configs() { return q38_qgemm_num_configs(); }
inline const char* qgemm_config_name(int config) { return q38_qgemm_config_name(config); }
inline int qgemm_config_tile_m(int config) { return q38_qgemm_config_tile_m(config); }

inline void qgemm(const __nv_bfloat16* a, int m, const BQWeight& w, const GemmEpilogue& ep, const GemmWorkspace& ws,
                  cudaStream_t stream, int config = kGemmConfigAuto) {
  const q38_bq_weight cw = w.c();
  const q38_gemm_epilogue ce = ep.c();
  const q38_gemm_workspace cws{ws.partials, ws.partial_floats, ws.counters, ws.num_counters};
  detail::ok(q38_qgemm(reinterpret_cast<const q38_bf16*>(a), m, &cw, &ce, &cws, stream, config));
}

using GemmTuningLookup = int (*)(int bits, int n, int k, int m);
inline void set_qgemm_tuning(GemmTuningLookup lookup) { q38_set_qgemm_tuning(lookup); }

inline void embed(const __nv_bfloat16* table, const int32_t* tokens, int m, int hidden, float* residual,
                  __nv_bfloat16* xbf, float* partials, cudaStream_t stream) {
  detail::ok(q38_embed(reinterpret_cast<const q38_bf16*>(table), tokens, m, hidden, residual,
                       reinterpret_cast<q38_bf16*>(xbf), partials, stream));
}

struct QkNormRopeParams {
  const __nv_bfloat16* proj = nullptr;
  int ld_proj = 0;
  const float* q_norm = nullptr;
  const float* k_norm = nullptr;
  float eps = 1e-6f;
  float rope_theta = 1e7f;
  int num_q_heads = 0, num_kv_heads = 0;
  __half* q_out = nullptr;
  int attn_layer = 0;
};
inline void qk_norm_rope_append(const QkNormRopeParams& p, const BatchDesc& batch, const KvCacheDesc& kv,
                                cudaStream_t stream) {
  const q38_qk_norm_rope_params cp{reinterpret_cast<const q38_bf16*>(p.proj), p.ld_proj, p.q_norm, p.k_norm, p.eps,
                                   p.rope_theta, p.num_q_heads, p.num_kv_heads, reinterpret_cast<q38_f16*>(p.q_out),
                                   p.attn_layer};
  const q38_batch_desc cb = batch.c();
  const q38_kv_cache_desc ck = kv.c();
  detail::ok(q38_qk_norm_rope_append(&cp, &cb, &ck, stream));
}

struct AttentionParams {
  const __half* q = nullptr;
  const __nv_bfloat16* gate = nullptr;
  int ld_gate = 0;
  __nv_bfloat16* out = nullptr;
  int num_q_heads = 0, num_kv_heads = 0, attn_layer = 0;
  float* split_scratch = nullptr;
  int max_splits = 0;
  int scratch_rows = 0;  // extension: rows the scratch holds (prefill may split its keys if >= the step's tokens)
  q38_attention_params c() const {
    return {reinterpret_cast<const q38_f16*>(q), reinterpret_cast<const q38_bf16*>(gate), ld_gate,
            reinterpret_cast<q38_bf16*>(out), num_q_heads, num_kv_heads, attn_layer, split_scratch, max_splits,
            scratch_rows};
  }
};
inline int attention_decode_splits(int batch_seqs, int kv_heads, int num_sms, int max_splits) {
  return q38_attention_decode_splits(batch_seqs, kv_heads, num_sms, max_splits);
}
inline void attention_decode(const AttentionParams& p, const BatchDesc& batch, const KvCacheDesc& kv,
                             cudaStream_t stream) {
  const q38_attention_params cp = p.c();
  const q38_batch_desc cb = batch.c();
  const q38_kv_cache_desc ck = kv.c();
  detail::ok(q38_attention_decode(&cp, &cb, &ck, stream));
}
inline void attention_prefill(const AttentionParams& p, const BatchDesc& batch, const KvCacheDesc& kv,
                              cudaStream_t stream) {
  const q38_attention_params cp = p.c();
  const q38_batch_desc cb = batch.c();
  const q38_kv_cache_desc ck = kv.c();
  detail::ok(q38_attention_prefill(&cp, &cb, &ck, stream));
}

struct GdnDims {
  int num_k_heads = 0, num_v_heads = 0, conv_dim = 0, ld_proj = 0;
};
struct GdnStateDesc {
  float* recurrent = nullptr;
  __nv_bfloat16* conv = nullptr;
  int num_gdn_layers = 0;
};
inline void gdn_ab(const __nv_bfloat16* xbf, int m, int hidden, const __nv_bfloat16* w_ab, int rows,
                   const float* partials_in, float eps, float* ab_out, cudaStream_t stream) {
  detail::ok(q38_gdn_ab(reinterpret_cast<const q38_bf16*>(xbf), m, hidden, reinterpret_cast<const q38_bf16*>(w_ab), rows,
                        partials_in, eps, ab_out, stream));
}
struct GdnConvParams {
  const __nv_bfloat16* proj = nullptr;
  const float* conv_w = nullptr;
  float* qkv = nullptr;
  int gdn_layer = 0;
};
inline void gdn_conv(const GdnConvParams& p, const GdnDims& d, const BatchDesc& batch, const GdnStateDesc& st,
                     cudaStream_t stream) {
  const q38_gdn_conv_params cp{reinterpret_cast<const q38_bf16*>(p.proj), p.conv_w, p.qkv, p.gdn_layer};
  const q38_gdn_dims cd{d.num_k_heads, d.num_v_heads, d.conv_dim, d.ld_proj};
  const q38_batch_desc cb = batch.c();
  const q38_gdn_state_desc cs{st.recurrent, reinterpret_cast<q38_bf16*>(st.conv), st.num_gdn_layers};
  detail::ok(q38_gdn_conv(&cp, &cd, &cb, &cs, stream));
}
struct GdnRecurrenceParams {
  const float* qkv = nullptr;
  const float* ab = nullptr;
  const float* A = nullptr;
  const float* dt_bias = nullptr;
  const __nv_bfloat16* z = nullptr;
  int ld_z = 0;
  const float* norm_w = nullptr;
  float eps = 1e-6f;
  __nv_bfloat16* out = nullptr;
  int gdn_layer = 0;
};
inline void gdn_recurrence(const GdnRecurrenceParams& p, const GdnDims& d, const BatchDesc& batch,
                           const GdnStateDesc& st, cudaStream_t stream) {
  const q38_gdn_recurrence_params cp{p.qkv, p.ab, p.A, p.dt_bias, reinterpret_cast<const q38_bf16*>(p.z), p.ld_z,
                                     p.norm_w, p.eps, reinterpret_cast<q38_bf16*>(p.out), p.gdn_layer};
  const q38_gdn_dims cd{d.num_k_heads, d.num_v_heads, d.conv_dim, d.ld_proj};
  const q38_batch_desc cb = batch.c();
  const q38_gdn_state_desc cs{st.recurrent, reinterpret_cast<q38_bf16*>(st.conv), st.num_gdn_layers};
  detail::ok(q38_gdn_recurrence(&cp, &cd, &cb, &cs, stream));
}
// Chunked (64-token) form of gdn_recurrence for prefill-sized runs; extension, no counterpart in the reference.
inline size_t gdn_chunk_scratch_floats(int max_tokens, int max_seqs, int num_v_heads) {
  return q38_gdn_chunk_scratch_floats(max_tokens, max_seqs, num_v_heads);
}
inline void gdn_recurrence_chunked(const GdnRecurrenceParams& p, const GdnDims& d, const BatchDesc& batch,
                                   const GdnStateDesc& st, float* scratch, size_t scratch_floats, cudaStream_t stream) {
  const q38_gdn_recurrence_params cp{p.qkv, p.ab, p.A, p.dt_bias, reinterpret_cast<const q38_bf16*>(p.z), p.ld_z,
                                     p.norm_w, p.eps, reinterpret_cast<q38_bf16*>(p.out), p.gdn_layer};
  const q38_gdn_dims cd{d.num_k_heads, d.num_v_heads, d.conv_dim, d.ld_proj};
  const q38_batch_desc cb = batch.c();
  const q38_gdn_state_desc cs{st.recurrent, reinterpret_cast<q38_bf16*>(st.conv), st.num_gdn_layers};
  detail::ok(q38_gdn_recurrence_chunked(&cp, &cd, &cb, &cs, scratch, scratch_floats, stream));
}

using SamplingParamsDev = q38_sampling_params_dev;
struct SamplingArgs {
  float* logits = nullptr;
  int ld = 0, vocab = 0;
  const SamplingParamsDev* params = nullptr;
  const int* row_slot = nullptr;
  int32_t* history = nullptr;
  int* history_len = nullptr;
  int history_cap = 0;
  const int* step = nullptr;
  int32_t* tokens_out = nullptr;
  float* logprob_out = nullptr;
};
inline void sample(const SamplingArgs& a, int batch, cudaStream_t stream) {
  const q38_sampling_args ca{a.logits, a.ld,          a.vocab, a.params,     a.row_slot,   a.history,
                             a.history_len, a.history_cap, a.step,  a.tokens_out, a.logprob_out};
  detail::ok(q38_sample(&ca, batch, stream));
}
inline void target_logprobs(const float* logits, int ld, int vocab, const int32_t* targets, int rows, float* out,
                            cudaStream_t stream) {
  detail::ok(q38_target_logprobs(logits, ld, vocab, targets, rows, out, stream));
}

// Extension: ragged-batch packing on the GPU (see q38_pack_ragged).
inline void pack_ragged(const int* seq_count, const int* seq_pos0, int num_seqs, int num_tokens, int* seq_start,
                        int* tok_pos, int* tok_seq, cudaStream_t stream) {
  detail::ok(q38_pack_ragged(seq_count, seq_pos0, num_seqs, num_tokens, seq_start, tok_pos, tok_seq, stream));
}

// Extension: LM-head input rows of a ragged step packed by one kernel (see q38_gather_rows).
inline void gather_rows(const __nv_bfloat16* x, const float* partials, const int* rows, int n, int hidden,
                        __nv_bfloat16* x_out, float* partials_out, cudaStream_t stream) {
  detail::ok(q38_gather_rows(reinterpret_cast<const q38_bf16*>(x), partials, rows, n, hidden,
                             reinterpret_cast<q38_bf16*>(x_out), partials_out, stream));
}

// Extension: the library's device error status as a node of the step (see q38_device_error_collect).
inline void collect_device_errors(unsigned int* dst, cudaStream_t stream) {
  detail::ok(q38_device_error_collect(dst, stream));
}

}  // namespace qwen38::kernels
