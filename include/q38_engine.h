/* q38_engine.h — C ABI of the host engine (libq38_engine.so) for language bindings.
 *
 * The C++20 API in qwen38/api.h (ModelFile, ModelRunner, KvCache, Engine: the reference engine's own
 * host interfaces, reference include/qwen38/{model_file,model_runner,kv_cache,engine}.h) is the primary
 * interface; this header exposes the same objects as opaque handles with plain-C calls so that tests,
 * benchmarks and other runtimes can drive them through an FFI. Every call returns 0 on success or -1
 * with the message in q38e_last_error() (C++ exceptions never cross the boundary).
 */
#ifndef Q38_ENGINE_H_
#define Q38_ENGINE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct q38e_model q38e_model;     /* qwen38::ModelFile */
typedef struct q38e_runner q38e_runner;   /* qwen38::ModelRunner */
typedef struct q38e_engine q38e_engine;   /* qwen38::Engine */

const char* q38e_last_error(void);

/* qwen38::SamplingParams (model_runner.h:23-31) */
typedef struct q38e_sampling {
  float temperature;
  int top_k;
  float top_p;
  float min_p;
  float presence_penalty;
  float repetition_penalty;
  uint64_t seed;
} q38e_sampling;

/* qwen38::RunnerOptions (model_runner.h:33-44) */
typedef struct q38e_runner_options {
  int max_batch;
  int prefill_chunk;
  int kv_dtype;        /* 0 int8, 1 bf16 */
  int64_t kv_tokens;   /* 0 = everything that fits */
  int max_context;
  size_t reserve_mib;
  int embedding_on_host;
  int cuda_graphs;
  int history_cap;
  int verbose;
} q38e_runner_options;
void q38e_default_runner_options(q38e_runner_options* o);

/* The decision the runner applies to the library's device error word after every step (the word is collected by the
 * step's last kernel, see q38_device_error_collect): 0 for a clean word; -1, with the failure text in
 * q38e_last_error(), for any other value. A failed step delivers no tokens: ModelRunner throws
 * qwen38::DeviceStepError, the Engine ends the step's requests with finish reason "error". Needs no GPU. */
int q38e_step_status(unsigned int device_error_word, const char* where);

/* qwen38::DecodeRow (model_runner.h:46-52) */
typedef struct q38e_decode_row {
  int slot;
  int position;
  int32_t token;
  q38e_sampling sampling;
  int step;
} q38e_decode_row;

/* one sequence's chunk of a ragged prefill step (qwen38::PrefillRow) */
typedef struct q38e_prefill_row {
  int slot;
  int pos0;
  const int32_t* tokens;
  int num_tokens;
  int sample;              /* non-zero: sample after the chunk's last token with `sampling` */
  q38e_sampling sampling;
  int step;
} q38e_prefill_row;

/* GEMM tile-configuration table (qwen38::load_tuning / install_tuning / lookup_tuning, include/qwen38/tuning.h,
 * src/tuning.cpp:24-70): a JSON file {"device": ..., "entries": [{bits, n, k, m_max, config, us}]}, as written by the
 * GEMM sweep (gemm_bench.py --sweep --save). Loading installs the table into the kernel library's dispatcher for this
 * process; an empty path clears it. q38e_tuning_lookup returns the configuration id the table gives for a call, or
 * -1 (the dispatcher's own choice). */
int q38e_tuning_load(const char* path);
int q38e_tuning_lookup(int bits, int n, int k, int m);

/* ModelFile */
int q38e_model_open(const char* path, q38e_model** out);
void q38e_model_close(q38e_model* m);
int q38e_model_vocab(const q38e_model* m);
int q38e_model_hidden(const q38e_model* m);
int q38e_model_layers(const q38e_model* m);
const char* q38e_model_summary(const q38e_model* m);
/* Host spec decoder (qwen38::BQView::dequant_all): out = float[n * k] of tensor `name`. */
int q38e_model_dequant(const q38e_model* m, const char* name, float* out, size_t out_floats);

/* ModelRunner */
int q38e_runner_create(const q38e_model* m, const q38e_runner_options* o, q38e_runner** out);
void q38e_runner_destroy(q38e_runner* r);
int q38e_runner_reset_slot(q38e_runner* r, int slot);
int q38e_runner_kv_ensure(q38e_runner* r, int slot, int tokens, int* ok);
int q38e_runner_kv_release(q38e_runner* r, int slot);
int q38e_runner_kv_pages(q38e_runner* r, int slot, int* pages_out, int capacity, int* count);
int q38e_runner_kv_free_pages(q38e_runner* r, int* count);
int q38e_runner_prefill(q38e_runner* r, const q38e_prefill_row* rows, int num_rows, int32_t* tokens_out,
                        float* logprobs_out, int* num_out);
int q38e_runner_decode(q38e_runner* r, const q38e_decode_row* rows, int num_rows, int32_t* tokens_out,
                       float* logprobs_out);
int q38e_runner_prefill_logits(q38e_runner* r, int slot, int pos0, const int32_t* tokens, int n, float* logits_out);
int q38e_runner_score(q38e_runner* r, int slot, int pos0, const int32_t* tokens, const int32_t* targets, int n,
                      float* logprobs_out);
int q38e_runner_set_profiling(q38e_runner* r, int on);
int q38e_runner_set_graphs(q38e_runner* r, int on);
/* per-op profile as text lines "name ms calls\n" into buf (truncated to cap) */
int q38e_runner_profile(q38e_runner* r, char* buf, size_t cap, int clear);
int q38e_runner_last_step_ms(q38e_runner* r, float* ms);
int q38e_runner_replay_decode_core(q38e_runner* r, int rows, int iters, float* ms_per_step);
int q38e_runner_last_logits(q38e_runner* r, int rows, float* logits_out);
int q38e_runner_memory(q38e_runner* r, size_t* weights, size_t* workspace, size_t* state, size_t* kv, int64_t* kv_tokens);

/* Engine */
typedef struct q38e_engine_options {
  q38e_runner_options runner;
  uint64_t seed;
  int ragged_prefill;
  int mixed_steps;     /* generating sequences' tokens ride in the prefill step while prompts are pending */
} q38e_engine_options;
int q38e_engine_create(const q38e_model* m, const q38e_engine_options* o, q38e_engine** out);
void q38e_engine_destroy(q38e_engine* e);
/* qwen38::GenerationConfig: stop_tokens NULL/0 = model EOS ids */
int q38e_engine_submit(q38e_engine* e, const int32_t* prompt, int n, const q38e_sampling* sampling, int max_new_tokens,
                       const int32_t* stop_tokens, int num_stop, int ignore_eos, int* request_id);
int q38e_engine_step(q38e_engine* e, int* more);
int q38e_engine_run(q38e_engine* e);
int q38e_engine_idle(q38e_engine* e, int* idle);
/* Finished requests are popped one at a time: first _next (sizes), then _take (copies and pops). */
int q38e_engine_finished_next(q38e_engine* e, int* request_id, int* num_tokens, int* finish_reason);
int q38e_engine_finished_take(q38e_engine* e, int32_t* tokens_out, float* logprobs_out, char* error_buf, size_t error_cap,
                              double* times3);
typedef struct q38e_stats {
  int64_t prefill_tokens;
  double prefill_s;
  int64_t decode_tokens;
  double decode_s;
  int64_t decode_steps;
  int64_t requests_done;
} q38e_stats;
int q38e_engine_stats(q38e_engine* e, q38e_stats* out, int reset);
int q38e_engine_runner(q38e_engine* e, q38e_runner** out); /* borrowed; do not destroy */

#ifdef __cplusplus
}
#endif
#endif /* Q38_ENGINE_H_ */
