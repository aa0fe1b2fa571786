/* q38_kernels.h — C ABI of the B200 (sm_100a) kernels of the ragged continuous-batching step.
 *
 * This is the drop-in boundary: every entry point replaces one launcher of the reference's internal
 * kernel API `src/kernels/kernels.h` (namespace qwen38::kernels). Signatures use plain pointers,
 * sizes and POD structs only (no C++ or torch types), so the library can be bound from C, C++, or any
 * FFI. The contract of the reference launchers is kept (src/kernels/kernels.h:3-6):
 *   - activations are row-major, M = number of tokens of the step;
 *   - every pointer is a device pointer unless stated otherwise (the embedding table may be mapped
 *     pinned host memory);
 *   - every launcher is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 *     default stream), allocates nothing, never synchronises the host and may be captured into a CUDA
 *     graph: all data-dependent sizes are read from device memory, only `num_seqs`, `num_tokens` and
 *     `max_tokens_per_seq` are host values fixed per captured graph.
 * Errors: launchers validate arguments on the host and return Q38_OK or a negative code; the message
 * is available from q38_last_error(). Kernels never trap or assert; bounded device-side waits report
 * through q38_device_error().
 */
#ifndef Q38_KERNELS_H_
#define Q38_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q38_OK 0
#define Q38_ERR_INVALID (-1) /* argument validation failed (reference: QWEN38_CHECK -> qwen38::Error) */
#define Q38_ERR_CUDA (-2)    /* a CUDA runtime / driver call made by the launcher failed */

#define Q38_PAGE_TOKENS 64 /* src/kernels/kernels.h:38 kPageTokens */
#define Q38_HEAD_DIM 256   /* src/kernels/kernels.h:39 kHeadDim */

typedef uint16_t q38_bf16; /* raw bfloat16 bits */
typedef uint16_t q38_f16;  /* raw IEEE half bits */

/* Ragged batch of one step. Replaces kernels::BatchDesc (src/kernels/kernels.h:22-31). */
typedef struct q38_batch_desc {
  int num_seqs;           /* B (host value) */
  int num_tokens;         /* M (host value) */
  int max_tokens_per_seq; /* upper bound of a sequence's run length in this step (host value) */
  const int* seq_start;   /* [B + 1] */
  const int* seq_slot;    /* [B] state slot = block-table row */
  const int* seq_pos0;    /* [B] position of the sequence's first token of this step */
  const int* tok_pos;     /* [M] absolute position of every token */
  const int* tok_seq;     /* [M] sequence index of every token */
} q38_batch_desc;

/* Paged KV cache. Replaces kernels::KvCacheDesc (src/kernels/kernels.h:36-70); the byte layout of a
 * (layer, page) block is the reference's: K [kv_head][64][256], V same, then for int8 the fp16 scales
 * K [kv_head][64][4], V same. */
#define Q38_KV_INT8 0
#define Q38_KV_BF16 1
typedef struct q38_kv_cache_desc {
  uint8_t* pool;
  int dtype; /* Q38_KV_INT8 | Q38_KV_BF16 */
  int kv_heads;
  int num_pages;
  size_t page_bytes;
  size_t layer_stride;
  const int* block_table; /* [slots][max_pages_per_seq] */
  int max_pages_per_seq;
} q38_kv_cache_desc;
size_t q38_kv_page_bytes(int dtype, int kv_heads); /* KvCacheDesc::page_bytes_for, kernels.h:66-69 */

/* BQ weight (reference docs/FORMAT.md section 2). Replaces kernels::BQWeight (kernels.h:82-90). */
typedef struct q38_bq_weight {
  const uint8_t* lo;
  const uint8_t* hi;      /* NULL for 4-bit */
  const q38_bf16* scales;
  int bits;               /* 4, 5, 6, 8 */
  int n;                  /* padded rows, multiple of 128 */
  int k;                  /* multiple of 64 */
  int rows;               /* logical rows */
} q38_bq_weight;

/* GEMM epilogues. Replaces kernels::Epilogue / GemmEpilogue / GemmWorkspace (kernels.h:75-111). */
#define Q38_EPI_STORE_BF16 0 /* out = bf16(C * rs) */
#define Q38_EPI_SWIGLU 1     /* out[i] = bf16(silu(C[2i] * rs) * C[2i+1] * rs) */
#define Q38_EPI_RESIDUAL 2   /* residual += C; xbf = bf16(residual); partials_out = sum of squares / 128 cols */
#define Q38_EPI_STORE_F32 3  /* out = C * rs */
/* Tensor parallelism, row-parallel projections of up to 16 tokens: C is this rank's partial product. The GEMM kernel
 * itself stores each finished 128-column tile into every rank's receive buffer (plain peer stores over NVLink), raises
 * a per-tile flag there, waits - bounded - for the other ranks' flags in its own memory, sums the pieces in rank order
 * (every rank gets the same bits) and then runs the Residual epilogue on the sum. No counterpart in the reference
 * (single GPU); replaces the all-reduce a host would otherwise place between q38_qgemm and q38_residual_update. */
#define Q38_EPI_ALLREDUCE_RESIDUAL 4
#define Q38_MAX_PEERS 8
#define Q38_ALLREDUCE_ROWS 16
typedef struct q38_peer_allreduce {
  int world, rank;
  /* rank r's receive buffer as mapped into this process, [2][world][Q38_ALLREDUCE_ROWS][n] floats (two buffers used in
   * turn), and its flags, [n / 128][world] words; entry `rank` is this rank's own memory. All zero before first use. */
  float* recv[Q38_MAX_PEERS];
  unsigned int* flags[Q38_MAX_PEERS];
  unsigned int* seq;       /* this rank's call counters, [n / 128] words, zero before first use */
  unsigned int poll_limit; /* polls of a flag before the wait gives up and sets q38_device_error(); 0 = 2^22 */
} q38_peer_allreduce;
typedef struct q38_gemm_epilogue {
  int kind;
  void* out;
  int ldo;
  int n_store;
  float* residual;
  q38_bf16* xbf;
  float* partials_out;
  const float* partials_in; /* rs = rsqrt(sum(partials_in[row]) / hidden + eps); NULL = 1 */
  int hidden;
  float eps;
  const q38_peer_allreduce* allreduce; /* Q38_EPI_ALLREDUCE_RESIDUAL only; NULL otherwise */
} q38_gemm_epilogue;

typedef struct q38_gemm_workspace {
  float* partials;       /* stream-K partial tiles */
  size_t partial_floats;
  int* counters;         /* per-tile arrival counters: zeroed once by the caller, self-resetting */
  int num_counters;
} q38_gemm_workspace;

/* kernels.h:113-125 */
#define Q38_GEMM_CONFIG_AUTO (-1)
int q38_qgemm_num_configs(void);
const char* q38_qgemm_config_name(int config);
int q38_qgemm_config_tile_m(int config);
/* The configuration q38_qgemm picks for Q38_GEMM_CONFIG_AUTO: the installed tuning lookup's answer if it has one,
 * else the built-in rule (pure host logic, no device access; no counterpart in the reference, whose launcher keeps
 * the choice to itself - tools use it to report what "auto" meant). */
int q38_qgemm_auto_config(int bits, int n, int k, int m);
/* C[M][N] = A[M][K] * W^T; A bf16 row-major with leading dimension K. (kernels::qgemm, kernels.h:120-121) */
int q38_qgemm(const q38_bf16* a, int m, const q38_bq_weight* w, const q38_gemm_epilogue* ep,
              const q38_gemm_workspace* ws, void* stream, int config);
/* The same GEMM for callers that cannot allocate device memory (no counterpart in the reference, whose launcher
 * always receives a caller-owned GemmWorkspace). The stream-K workspace is a fixed array inside the library
 * (about 3.2 MB of device memory per GPU that loads it). Limits: 1 <= m <= 16, n <= 524288, at most 192 SMs;
 * anything larger is rejected with Q38_ERR_INVALID. The first call on a device looks the array's address up
 * (cudaGetSymbolAddress) and should therefore be made before any stream capture starts. Every call on a device
 * uses the same array: calls that may overlap on the GPU must be serialised by the caller. Allocates nothing. */
int q38_qgemm_static(const q38_bf16* a, int m, const q38_bq_weight* w, const q38_gemm_epilogue* ep, void* stream);
typedef int (*q38_gemm_tuning_lookup)(int bits, int n, int k, int m);
void q38_set_qgemm_tuning(q38_gemm_tuning_lookup lookup); /* kernels::set_qgemm_tuning, kernels.h:124-125 */

/* Dequantised weights W[n][k] as bf16 (row-major, padded rows included): the values the GEMM feeds to
 * the tensor cores. Test / inspection helper of the in-register decoder (the reference checks the same
 * logic on the host, tests/host/test_bq_layout.cpp). */
int q38_bq_dequant(const q38_bq_weight* w, q38_bf16* out, void* stream);

/* kernels::embed, kernels.h:131-134 */
int q38_embed(const q38_bf16* table, const int32_t* tokens, int m, int hidden, float* residual, q38_bf16* xbf,
              float* partials, void* stream);

/* The Residual GEMM epilogue as an op of its own: residual += delta, xbf = bf16(residual), partials[m][col / 128] =
 * sum of squares. For tensor-parallel runs, where the row-parallel projections store fp32 partial products
 * (Q38_EPI_STORE_F32) that are summed over the ranks first. No counterpart in the reference (single GPU). */
int q38_residual_update(const float* delta, int m, int hidden, float* residual, q38_bf16* xbf, float* partials,
                        void* stream);

/* Device memory that other processes of the node can map (buffers and flags of Q38_EPI_ALLREDUCE_RESIDUAL): allocation
 * (zero-filled), the 64-byte handle a peer process opens, opening and closing a peer's handle. The handles travel
 * through whatever the host uses between its ranks. One process per GPU; peer access is enabled on opening. */
int q38_peer_alloc(size_t bytes, void** ptr);
int q38_peer_free(void* ptr);
int q38_peer_export(void* ptr, unsigned char handle[64]);
int q38_peer_open(const unsigned char handle[64], void** ptr);
int q38_peer_close(void* ptr);

/* Packs rows rows[0..n) of the step's LM-head inputs (bf16 hidden rows x [M][hidden] and their norm partial sums
 * [M][hidden / 128]) into rows 0..n-1 of x_out / partials_out: the last-token rows of the sequences that sample in a
 * ragged step. Replaces the per-row device copies of the reference's prefill path (src/model_runner.cpp:471-489 reads
 * one row; a ragged step has up to one per sequence). `rows` is a device array. */
int q38_gather_rows(const q38_bf16* x, const float* partials, const int* rows, int n, int hidden, q38_bf16* x_out,
                    float* partials_out, void* stream);

/* kernels::QkNormRopeParams + qk_norm_rope_append, kernels.h:140-155 */
typedef struct q38_qk_norm_rope_params {
  const q38_bf16* proj; /* [M][ld_proj]: [q | gate | k | v] */
  int ld_proj;
  const float* q_norm;  /* [256], already 1 + w */
  const float* k_norm;
  float eps;
  float rope_theta;
  int num_q_heads;
  int num_kv_heads;
  q38_f16* q_out;       /* [M][nq][256] */
  int attn_layer;
} q38_qk_norm_rope_params;
int q38_qk_norm_rope_append(const q38_qk_norm_rope_params* p, const q38_batch_desc* batch,
                            const q38_kv_cache_desc* kv, void* stream);

/* kernels::AttentionParams, attention_decode_splits, attention_decode, attention_prefill, kernels.h:157-179 */
typedef struct q38_attention_params {
  const q38_f16* q;      /* [M][nq][256] */
  const q38_bf16* gate;  /* proj + nq*256, row stride ld_gate */
  int ld_gate;
  q38_bf16* out;         /* [M][nq*256] */
  int num_q_heads;
  int num_kv_heads;
  int attn_layer;
  float* split_scratch;  /* [B][nq][max_splits][256 + 2] floats */
  int max_splits;
  /* Extension (not in the reference's struct): rows B the scratch was sized for. Decode needs one row per sequence
   * and ignores the field. Prefill cuts the keys of its query tiles over several CTAs only when there are few tiles
   * for the GPU (one long request, a tensor-parallel rank with one kv head) and only if the scratch holds one row
   * per prompt token of the step: scratch_rows >= num_tokens. 0 = sized for the decode batch only (never split). */
  int scratch_rows;
} q38_attention_params;
int q38_attention_decode_splits(int batch_seqs, int kv_heads, int num_sms, int max_splits);
int q38_attention_decode(const q38_attention_params* p, const q38_batch_desc* batch, const q38_kv_cache_desc* kv,
                         void* stream);
int q38_attention_prefill(const q38_attention_params* p, const q38_batch_desc* batch, const q38_kv_cache_desc* kv,
                          void* stream);

/* kernels::GdnDims / GdnStateDesc, kernels.h:184-195 */
typedef struct q38_gdn_dims {
  int num_k_heads;
  int num_v_heads;
  int conv_dim; /* 2 * nk * 128 + nv * 128 */
  int ld_proj;
} q38_gdn_dims;
typedef struct q38_gdn_state_desc {
  float* recurrent;  /* [slots][gdn_layers][nv][128 dv][128 dk] */
  q38_bf16* conv;    /* [slots][gdn_layers][3][conv_dim] */
  int num_gdn_layers;
} q38_gdn_state_desc;

/* kernels::gdn_ab, kernels.h:197-199 */
int q38_gdn_ab(const q38_bf16* xbf, int m, int hidden, const q38_bf16* w_ab, int rows, const float* partials_in,
               float eps, float* ab_out, void* stream);

/* kernels::GdnConvParams + gdn_conv, kernels.h:201-210 */
typedef struct q38_gdn_conv_params {
  const q38_bf16* proj;
  const float* conv_w; /* [conv_dim][4] */
  float* qkv;          /* [M][conv_dim] */
  int gdn_layer;
} q38_gdn_conv_params;
int q38_gdn_conv(const q38_gdn_conv_params* p, const q38_gdn_dims* d, const q38_batch_desc* batch,
                 const q38_gdn_state_desc* st, void* stream);

/* kernels::GdnRecurrenceParams + gdn_recurrence, kernels.h:212-228 */
typedef struct q38_gdn_recurrence_params {
  const float* qkv;
  const float* ab;
  const float* A;
  const float* dt_bias;
  const q38_bf16* z;
  int ld_z;
  const float* norm_w;
  float eps;
  q38_bf16* out;
  int gdn_layer;
} q38_gdn_recurrence_params;
int q38_gdn_recurrence(const q38_gdn_recurrence_params* p, const q38_gdn_dims* d, const q38_batch_desc* batch,
                       const q38_gdn_state_desc* st, void* stream);

/* The same operation in the chunked (64-token WY) form for prefill-sized runs: token-parallel preparation plus a
 * per-chunk state scan instead of a token-by-token loop; results agree with q38_gdn_recurrence to fp32 rounding.
 * Any run lengths are accepted (short runs are padded to a chunk, so q38_gdn_recurrence is the better choice when
 * batch->max_tokens_per_seq is small). `scratch` holds q38_gdn_chunk_scratch_floats(num_tokens, num_seqs,
 * num_v_heads) floats, 16-byte aligned, and may be reused by the next call on the same stream.
 * No counterpart in the reference, whose gdn_recurrence (kernels.h:212-228) is token-sequential. */
size_t q38_gdn_chunk_scratch_floats(int max_tokens, int max_seqs, int num_v_heads);
int q38_gdn_recurrence_chunked(const q38_gdn_recurrence_params* p, const q38_gdn_dims* d,
                               const q38_batch_desc* batch, const q38_gdn_state_desc* st, float* scratch,
                               size_t scratch_floats, void* stream);
/* Which form of the chunk scan q38_gdn_recurrence_chunked launches: 1 (default) = the four per-chunk products on the
 * tensor cores (mma.sync TF32 with every factor split into two TF32 numbers, three MMAs per product: fp32-like
 * accuracy, fp32 sums), 0 = all fp32 on the CUDA cores. Process-wide; applies to launches made after the call. No
 * counterpart in the reference (its recurrence is token-sequential). */
void q38_gdn_set_chunk_scan_tensor_cores(int on);

/* kernels::SamplingParamsDev / SamplingArgs / sample / target_logprobs, kernels.h:233-260 */
typedef struct q38_sampling_params_dev {
  float temperature;
  int top_k;
  float top_p;
  float min_p;
  float presence_penalty;
  float repetition_penalty;
  uint64_t seed;
} q38_sampling_params_dev;
typedef struct q38_sampling_args {
  float* logits;
  int ld;
  int vocab;
  const q38_sampling_params_dev* params;
  const int* row_slot;
  int32_t* history;
  int* history_len;
  int history_cap;
  const int* step;
  int32_t* tokens_out;
  float* logprob_out;
} q38_sampling_args;
int q38_sample(const q38_sampling_args* a, int batch, void* stream);
int q38_target_logprobs(const float* logits, int ld, int vocab, const int32_t* targets, int rows, float* out,
                        void* stream);

/* Ragged-batch packing on the GPU. Replaces the host loops that fill the step metadata
 * (src/model_runner.cpp:458-469 for prefill, :534-560 for decode): expands per-sequence
 * (slot, pos0, count) rows into seq_start / tok_pos / tok_seq. Inputs are device arrays of num_seqs
 * entries; outputs are the arrays a q38_batch_desc points at. num_tokens must equal sum(count). */
int q38_pack_ragged(const int* seq_count, const int* seq_pos0, int num_seqs, int num_tokens, int* seq_start,
                    int* tok_pos, int* tok_seq, void* stream);

/* Diagnostics. */
const char* q38_last_error(void);           /* message of the last failed launcher call on this thread */
/* Programmatic dependent launch (on by default): every launcher allows its kernel to be scheduled while the
 * previous kernel of the stream drains; inside, griddepcontrol.wait precedes the first access to data an earlier
 * kernel produces, so results do not depend on the setting. Off = classic stream order. Applies to launches (and
 * graph captures) made after the call. No counterpart in the reference. */
void q38_set_dependent_launch(int allowed);
unsigned int q38_device_error(int clear);   /* non-zero if a bounded device-side wait ran out (synchronises) */
/* The same status without a synchronisation, as one more node of the caller's stream or graph: a one-thread kernel
 * moves the first non-zero error word of the library into *dst (device memory or mapped pinned host memory) and
 * clears the library's words; *dst is not written when nothing failed. A host engine enqueues it at the end of each
 * step and reads *dst after its stream synchronisation: a step whose pipeline aborted (the results of that launch
 * are meaningless) can then be failed instead of delivered. The first call on a device looks the words up and
 * should come before any stream capture. No counterpart in the reference (its kernels have no bounded waits). */
int q38_device_error_collect(unsigned int* dst, void* stream);
/* Test hook: sets one of the library's error words from the host, as if a kernel had reported `code`. */
int q38_device_error_inject(unsigned int code);
int q38_num_sms(void);                      /* SM count of the current device as cached by the library */

#ifdef __cplusplus
}
#endif
#endif /* Q38_KERNELS_H_ */
