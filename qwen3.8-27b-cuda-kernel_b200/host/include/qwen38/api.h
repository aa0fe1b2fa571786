// qwen38 host API (C++20), B200 build.
//
// One header declares the whole public host surface of the engine. It is source-compatible with the
// reference engine's public headers (reference include/qwen38/{common,config,model_file,bq,device,
// weights,kv_cache,model_runner,engine,tuning}.h): the same namespaces, type names, member names and
// call signatures, so code written against the reference (its apps and tests) builds against this
// implementation unchanged; the per-file headers next to this one simply include it. Everything below
// the API is new: the kernels are reached through the C ABI of include/q38_kernels.h, the step metadata
// is expanded on the GPU, prompts of several sequences can share one ragged prefill step, and defaults
// are sized for a 180 GB B200 instead of a 24 GB card.
#pragma once

#include <cuda_runtime.h>

#include <bit>
#include <chrono>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <span>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "kernels/kernels.h"

namespace qwen38 {

// ===================================================================================================
// errors and small numeric helpers (reference include/qwen38/common.h)
// ===================================================================================================
class Error : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

// A step whose kernels reported a pipeline abort (a bounded device-side wait ran out, a page id outside the pool, a
// tensor-memory allocation at an unexpected base): the step's outputs are meaningless and were not delivered. The
// CUDA context is intact; later steps can run. Extension: the reference's kernels have no such status.
class DeviceStepError : public Error {
 public:
  DeviceStepError(unsigned int code, const std::string& where);
  unsigned int code() const { return code_; }

 private:
  unsigned int code_ = 0;
};
// Message of a step failure for error word `code` ("" when code == 0): the pure decision the runner applies after
// every step, callable without a GPU.
std::string device_step_failure(unsigned int code, const std::string& where);

[[noreturn]] void fail(const std::string& message);
std::string format_check_failure(const char* expr, const char* file, int line, const std::string& msg);

template <typename... Ts>
std::string strcat_args(const Ts&... parts) {
  std::ostringstream os;
  (os << ... << parts);
  return os.str();
}

#define QWEN38_CHECK(cond, ...)                                                                        \
  do {                                                                                                 \
    if (!(cond))                                                                                       \
      ::qwen38::fail(::qwen38::format_check_failure(#cond, __FILE__, __LINE__, ::qwen38::strcat_args(__VA_ARGS__))); \
  } while (0)

inline float bf16_to_f32(uint16_t bits) { return std::bit_cast<float>(uint32_t(bits) << 16); }
uint16_t f32_to_bf16(float f);   // round to nearest even, NaN stays NaN
inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }
float f16_to_f32(uint16_t h);
uint16_t f32_to_f16(float f);    // round to nearest even, overflow to infinity
inline float round_f16(float f) { return f16_to_f32(f32_to_f16(f)); }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ===================================================================================================
// model configuration (reference include/qwen38/config.h; header block of docs/FORMAT.md 1.1)
// ===================================================================================================
struct ModelConfig {
  int hidden_size = 0, num_layers = 0, vocab_size = 0, intermediate_size = 0;
  int num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0, rotary_dim = 0;
  double rope_theta = 0;
  int linear_num_key_heads = 0, linear_num_value_heads = 0;
  int linear_key_head_dim = 0, linear_value_head_dim = 0, linear_conv_kernel_dim = 0;
  float rms_norm_eps = 1e-6f;
  int max_position_embeddings = 0;
  bool norm_folded = true;
  std::vector<uint8_t> is_attention;   // per layer: 1 full attention, 0 Gated DeltaNet
  std::vector<int32_t> eos_token_ids;

  int num_attention_layers() const;
  int num_gdn_layers() const;
  int attn_index(int layer) const;  // -1 for GDN layers
  int gdn_index(int layer) const;   // -1 for attention layers
  int q_dim() const { return num_attention_heads * head_dim; }
  int kv_dim() const { return num_key_value_heads * head_dim; }
  int attn_group() const { return num_attention_heads / num_key_value_heads; }
  int qkvg_rows() const { return 2 * q_dim() + 2 * kv_dim(); }
  int gdn_key_dim() const { return linear_num_key_heads * linear_key_head_dim; }
  int gdn_value_dim() const { return linear_num_value_heads * linear_value_head_dim; }
  int gdn_conv_dim() const { return 2 * gdn_key_dim() + gdn_value_dim(); }
  int gdn_qkvz_rows() const { return gdn_conv_dim() + gdn_value_dim(); }
  int gdn_v_per_k() const { return linear_num_value_heads / linear_num_key_heads; }
  int norm_blocks() const { return hidden_size / 128; }
  void validate() const;  // throws Error for geometries the kernels do not implement
  std::string summary() const;
};

// ===================================================================================================
// .q38 model file (reference include/qwen38/model_file.h, docs/FORMAT.md 1)
// ===================================================================================================
enum class DType : uint8_t { BQ4, BQ5, BQ6, BQ8, BF16, F32 };
const char* dtype_name(DType dtype);
inline bool is_bq(DType d) { return d <= DType::BQ8; }
inline int bq_bits(DType d) {
  constexpr int kBits[] = {4, 5, 6, 8, 0, 0};
  return kBits[int(d)];
}

struct TensorInfo {
  std::string name;
  DType dtype = DType::F32;
  std::vector<int64_t> shape;
  int64_t rows = 0;                      // logical rows (padded BQ tensors keep shape[0] >= rows)
  int64_t offset = 0, bytes = 0;         // bf16 / f32 payload
  int64_t lo_offset = 0, lo_bytes = 0;   // BQ planes; hi_bytes == 0 for 4-bit
  int64_t hi_offset = 0, hi_bytes = 0;
  int64_t sc_offset = 0, sc_bytes = 0;
  int64_t numel() const;
  int64_t storage_bytes() const { return is_bq(dtype) ? lo_bytes + hi_bytes + sc_bytes : bytes; }
};

class ModelFile {
 public:
  static std::unique_ptr<ModelFile> open(const std::string& path);
  ~ModelFile();
  ModelFile(const ModelFile&) = delete;
  ModelFile& operator=(const ModelFile&) = delete;

  const ModelConfig& config() const { return config_; }
  const std::string& path() const { return path_; }
  const std::string& recipe_name() const { return recipe_; }
  const std::string& header_json() const { return header_; }
  uint64_t data_start() const { return data_start_; }
  bool has_tensor(const std::string& name) const { return tensors_.count(name) != 0; }
  const TensorInfo& tensor(const std::string& name) const;
  const std::map<std::string, TensorInfo>& tensors() const { return tensors_; }
  std::span<const uint8_t> data(int64_t offset, int64_t size) const;   // relative to data_start()
  std::span<const uint8_t> resource(const std::string& name) const;    // empty if absent
  template <typename T>
  std::span<const T> direct(const std::string& name) const {
    const TensorInfo& t = tensor(name);
    const auto d = data(t.offset, t.bytes);
    return {reinterpret_cast<const T*>(d.data()), d.size() / sizeof(T)};
  }
  int64_t total_weight_bytes() const;

 private:
  ModelFile() = default;
  std::string path_, header_, recipe_;
  ModelConfig config_;
  std::map<std::string, TensorInfo> tensors_;
  std::map<std::string, std::pair<int64_t, int64_t>> resources_;
  uint64_t data_start_ = 0, file_size_ = 0;
  const uint8_t* base_ = nullptr;
  size_t mapped_size_ = 0;
  int fd_ = -1;
};

// Host-side spec decoder of BQ tensors (reference include/qwen38/bq.h): the bit-exact definition of
// the dequantised weight, independent of the device decoder.
struct BQView {
  int bits = 4;
  int64_t n = 0, k = 0, rows = 0;
  const uint8_t* lo = nullptr;
  const uint8_t* hi = nullptr;
  const uint16_t* scales = nullptr;
  static BQView from_file(const ModelFile& file, const std::string& name);
  int code(int64_t row, int64_t col) const;
  uint16_t scale_bits(int64_t row, int64_t group) const;
  float scale(int64_t row, int64_t group) const;
  float weight(int64_t row, int64_t col) const;
  void dequant_row(int64_t row, float* out) const;
  std::vector<float> dequant_all() const;
};

// ===================================================================================================
// CUDA resource ownership (reference include/qwen38/device.h)
// ===================================================================================================
void cuda_check(cudaError_t err, const char* expr, const char* file, int line);
#define QWEN38_CUDA(expr) ::qwen38::cuda_check((expr), #expr, __FILE__, __LINE__)

class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t bytes);
  ~DeviceBuffer();
  DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(std::exchange(o.ptr_, nullptr)), bytes_(std::exchange(o.bytes_, 0)) {}
  DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  void* get() const { return ptr_; }
  template <typename T>
  T* as() const { return static_cast<T*>(ptr_); }
  size_t bytes() const { return bytes_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
};

class PinnedBuffer {
 public:
  PinnedBuffer() = default;
  PinnedBuffer(size_t bytes, bool mapped);
  ~PinnedBuffer();
  PinnedBuffer(PinnedBuffer&& o) noexcept
      : ptr_(std::exchange(o.ptr_, nullptr)), bytes_(std::exchange(o.bytes_, 0)), mapped_(o.mapped_) {}
  PinnedBuffer& operator=(PinnedBuffer&& o) noexcept;
  PinnedBuffer(const PinnedBuffer&) = delete;
  PinnedBuffer& operator=(const PinnedBuffer&) = delete;
  void* get() const { return ptr_; }
  template <typename T>
  T* as() const { return static_cast<T*>(ptr_); }
  void* device_ptr() const;  // mapped buffers only
  size_t bytes() const { return bytes_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
  bool mapped_ = false;
};

// Bump allocator over one device block; sub-ranges live as long as the arena.
class DeviceArena {
 public:
  DeviceArena() = default;
  explicit DeviceArena(size_t capacity) : block_(capacity) {}
  void* allocate(size_t bytes, size_t align = 256);
  template <typename T>
  T* allocate_array(size_t count, size_t align = 256) {
    return static_cast<T*>(allocate(count * sizeof(T), align));
  }
  size_t used() const { return used_; }
  size_t capacity() const { return block_.bytes(); }

 private:
  DeviceBuffer block_;
  size_t used_ = 0;
};

class Stream {
 public:
  Stream();
  ~Stream();
  Stream(const Stream&) = delete;
  Stream& operator=(const Stream&) = delete;
  cudaStream_t get() const { return s_; }
  void sync() const;

 private:
  cudaStream_t s_ = nullptr;
};

class Event {
 public:
  explicit Event(bool timing = false);
  ~Event();
  Event(const Event&) = delete;
  Event& operator=(const Event&) = delete;
  cudaEvent_t get() const { return e_; }
  void record(cudaStream_t s) const;
  void sync() const;
  float ms_since(const Event& start) const;

 private:
  cudaEvent_t e_ = nullptr;
};

class Graph {
 public:
  Graph() = default;
  ~Graph();
  Graph(Graph&& o) noexcept : exec_(std::exchange(o.exec_, nullptr)) {}
  Graph& operator=(Graph&& o) noexcept;
  Graph(const Graph&) = delete;
  Graph& operator=(const Graph&) = delete;
  void begin_capture(cudaStream_t s);
  void end_capture(cudaStream_t s);
  void launch(cudaStream_t s) const;
  bool valid() const { return exec_ != nullptr; }

 private:
  cudaGraphExec_t exec_ = nullptr;
};

struct DeviceInfo {
  int device = 0;
  std::string name;
  int sm_major = 0, sm_minor = 0, num_sms = 0;
  size_t total_mem = 0, free_mem = 0, l2_bytes = 0;
  int max_smem_per_block_optin = 0;
  bool can_map_host = false;
};
// Properties of `device`; -1 = the device that is current (one engine replica per process and GPU).
DeviceInfo query_device(int device = -1);

// ===================================================================================================
// weights (reference include/qwen38/weights.h)
// ===================================================================================================
enum class EmbeddingPlacement { Host, Device };

struct LayerWeights {
  bool attention = false;
  kernels::BQWeight in_proj, out_proj, gate_up, down;
  const float* q_norm = nullptr;
  const float* k_norm = nullptr;
  const __nv_bfloat16* ab = nullptr;
  int ab_rows = 0;
  const float* conv = nullptr;
  const float* A = nullptr;
  const float* dt_bias = nullptr;
  const float* gdn_norm = nullptr;
};

class ModelWeights {
 public:
  ModelWeights(const ModelFile& file, EmbeddingPlacement placement);
  const std::vector<LayerWeights>& layers() const { return layers_; }
  const kernels::BQWeight& lm_head() const { return lm_head_; }
  const __nv_bfloat16* embedding() const { return embedding_; }
  EmbeddingPlacement embedding_placement() const { return placement_; }
  size_t device_bytes() const { return arena_.used(); }
  size_t host_bytes() const { return embed_host_.bytes(); }
  static size_t required_device_bytes(const ModelFile& file, EmbeddingPlacement placement);

 private:
  kernels::BQWeight upload_bq(const ModelFile& file, const std::string& name);
  const void* upload_range(const ModelFile& file, int64_t offset, int64_t bytes);
  DeviceArena arena_;
  PinnedBuffer embed_host_;
  EmbeddingPlacement placement_;
  std::vector<LayerWeights> layers_;
  kernels::BQWeight lm_head_;
  const __nv_bfloat16* embedding_ = nullptr;
};

// ===================================================================================================
// paged KV cache + GDN state pool (reference include/qwen38/kv_cache.h)
// ===================================================================================================
class KvCache {
 public:
  KvCache(const ModelConfig& cfg, kernels::KvDtype dtype, int num_pages, int num_slots, int max_pages_per_seq);
  static size_t page_bytes_all_layers(const ModelConfig& cfg, kernels::KvDtype dtype);
  kernels::KvCacheDesc desc() const;
  int num_pages() const { return num_pages_; }
  int free_pages() const { return int(free_.size()); }
  int pages_of(int slot) const { return int(owned_[size_t(slot)].size()); }
  int max_pages_per_seq() const { return max_pages_per_seq_; }
  const std::vector<int>& page_list(int slot) const { return owned_[size_t(slot)]; }
  // Pages for positions [0, tokens) of `slot`; false (nothing changed) if the pool cannot provide them.
  bool ensure(int slot, int tokens);
  void release(int slot);
  void sync(cudaStream_t stream);  // uploads block-table rows that changed

 private:
  int num_pages_, num_slots_, max_pages_per_seq_;
  kernels::KvDtype dtype_;
  int kv_heads_;
  size_t page_bytes_ = 0, layer_stride_ = 0;
  DeviceBuffer pool_, table_dev_;
  PinnedBuffer table_host_;
  std::vector<int> free_;
  std::vector<std::vector<int>> owned_;
  std::vector<bool> dirty_;
};

class GdnStatePool {
 public:
  GdnStatePool(const ModelConfig& cfg, int num_slots);
  static size_t bytes_per_slot(const ModelConfig& cfg);
  kernels::GdnStateDesc desc() const;
  void reset(int slot, cudaStream_t stream);

 private:
  size_t recurrent_per_slot_ = 0, conv_per_slot_ = 0;
  int num_gdn_layers_ = 0;
  DeviceBuffer recurrent_, conv_;
};

// ===================================================================================================
// step executor (reference include/qwen38/model_runner.h)
// ===================================================================================================
struct SamplingParams {
  float temperature = 1.0f;
  int top_k = 20;
  float top_p = 0.95f;
  float min_p = 0.0f;
  float presence_penalty = 0.0f;
  float repetition_penalty = 1.0f;
  uint64_t seed = 0;
};

struct RunnerOptions {
  int max_batch = 8;
  int prefill_chunk = 1024;
  kernels::KvDtype kv_dtype = kernels::KvDtype::Int8;
  int64_t kv_tokens = 0;        // 0 = everything that fits
  int max_context = 262144;
  size_t reserve_mib = 640;
  EmbeddingPlacement embedding = EmbeddingPlacement::Device;  // 180 GB of HBM: the table stays on the GPU
  bool cuda_graphs = true;
  int history_cap = 1024;
  bool verbose = true;
};

struct DecodeRow {
  int slot = 0;
  int position = 0;
  int32_t token = 0;
  SamplingParams sampling;
  int step = 0;
};

// One sequence's share of a ragged prefill step (extension: the reference prefills one sequence per call).
struct PrefillRow {
  int slot = 0;
  int pos0 = 0;
  std::span<const int32_t> tokens;
  const SamplingParams* sample = nullptr;  // set on the last chunk of a prompt
  int step = 0;
};

struct StepResult {
  std::vector<int32_t> tokens;
  std::vector<float> logprobs;
};

struct MemoryPlan {
  size_t free_at_start = 0, weights = 0, embedding_host = 0, workspace = 0, state = 0, kv = 0, reserve = 0;
  int kv_pages = 0;
  int64_t kv_tokens = 0;
  std::string describe() const;
};

struct OpProfile {
  std::map<std::string, double> ms;
  std::map<std::string, int> calls;
};

class ModelRunner {
 public:
  ModelRunner(const ModelFile& file, const RunnerOptions& options);
  ~ModelRunner();
  ModelRunner(const ModelRunner&) = delete;
  ModelRunner& operator=(const ModelRunner&) = delete;

  const ModelConfig& config() const;
  const RunnerOptions& options() const;
  const MemoryPlan& memory() const;
  const DeviceInfo& device() const;
  int num_slots() const;
  KvCache& kv();
  const ModelWeights& weights() const;
  cudaStream_t stream() const;
  const kernels::GemmWorkspace& gemm_workspace() const;

  void reset_slot(int slot);
  StepResult prefill(int slot, int pos0, std::span<const int32_t> tokens, const SamplingParams* sample, int step);
  StepResult decode(std::span<const DecodeRow> rows);
  std::vector<float> score(int slot, int pos0, std::span<const int32_t> tokens, std::span<const int32_t> targets);
  std::vector<float> prefill_logits(int slot, int pos0, std::span<const int32_t> tokens);

  // Ragged prefill: chunks of several sequences in one step (sum of lengths <= prefill_chunk). The result
  // holds one token per row that asked for a sample, in row order.
  StepResult prefill_batch(std::span<const PrefillRow> rows);

  void set_profiling(bool on);
  const OpProfile& profile() const;
  void clear_profile();
  void set_graphs_enabled(bool on);

  // Device-side timing of the last decode()/prefill*() call's kernels (CUDA events on the runner's stream,
  // host<->device copies excluded), milliseconds.
  float last_step_device_ms() const;
  // Benchmark support: replays the device work of the decode step of `rows` sequences (its captured graph
  // without the metadata upload and result download) `iters` times back to back and returns the mean
  // milliseconds per step. decode() must have run once with this batch size.
  float replay_decode_core(int rows, int iters);
  // Test support: the fp32 logits [rows][vocab] the last step's LM head produced (before sampling
  // penalties are applied they equal the model's logits; greedy sampling leaves them untouched).
  std::vector<float> last_logits(int rows);

  struct Impl;

 private:
  std::unique_ptr<Impl> impl_;
};

// ===================================================================================================
// scheduler (reference include/qwen38/engine.h)
// ===================================================================================================
struct GenerationConfig {
  SamplingParams sampling;
  int max_new_tokens = 4096;
  std::vector<int32_t> stop_tokens;
  bool ignore_eos = false;
};

enum class FinishReason { None, Stop, Length, Error };
const char* finish_reason_name(FinishReason r);

struct RequestResult {
  int id = -1;
  std::vector<int32_t> prompt, tokens;
  std::vector<float> logprobs;
  FinishReason finish = FinishReason::None;
  std::string error;
  double submit_s = 0, first_token_s = 0, done_s = 0;
};

using TokenCallback = std::function<void(int request_id, int32_t token, bool finished)>;

struct EngineOptions {
  RunnerOptions runner;
  uint64_t seed = 0x5eed;
  // Extension: let one scheduler iteration prefill chunks of several waiting prompts together (one ragged
  // step of at most prefill_chunk tokens) instead of one sequence's chunk. Off = reference behaviour.
  bool ragged_prefill = false;
  // Extension: while prompts are being prefilled, the generating sequences' next tokens ride in the same ragged step
  // as the prefill chunk (one pass over the weights instead of a prefill step followed by a decode step; the single
  // tokens count against the step's prefill_chunk token budget). Off = reference behaviour.
  bool mixed_steps = false;
};

struct EngineStats {
  int64_t prefill_tokens = 0;
  double prefill_s = 0;
  int64_t decode_tokens = 0;
  double decode_s = 0;
  int64_t decode_steps = 0;
  int64_t requests_done = 0;
  double tokens_per_s_decode() const { return decode_s > 0 ? double(decode_tokens) / decode_s : 0; }
  double tokens_per_s_prefill() const { return prefill_s > 0 ? double(prefill_tokens) / prefill_s : 0; }
  double avg_batch() const { return decode_steps ? double(decode_tokens) / double(decode_steps) : 0; }
};

class Engine {
 public:
  Engine(const ModelFile& file, const EngineOptions& options);
  ~Engine();
  int submit(std::vector<int32_t> prompt, GenerationConfig config, TokenCallback on_token = nullptr);
  bool step();
  void run();
  std::vector<RequestResult> take_finished();
  bool idle() const;
  const EngineStats& stats() const { return stats_; }
  void reset_stats() { stats_ = EngineStats{}; }
  ModelRunner& runner() { return *runner_; }
  const ModelConfig& config() const { return runner_->config(); }

 private:
  struct Sequence;
  void admit();
  void finish(Sequence& s, FinishReason reason, const std::string& error = {});
  bool deliver(Sequence& s, int32_t token, float logprob);
  void drop_finished();
  double now() const;

  EngineOptions opt_;
  std::unique_ptr<ModelRunner> runner_;
  std::vector<int32_t> eos_;
  std::deque<std::unique_ptr<Sequence>> waiting_;
  std::vector<std::unique_ptr<Sequence>> active_;
  std::vector<int> free_slots_;
  std::vector<RequestResult> finished_;
  EngineStats stats_;
  int next_id_ = 0;
  std::chrono::steady_clock::time_point t0_;
};

// ===================================================================================================
// GEMM tuning table (reference include/qwen38/tuning.h)
// ===================================================================================================
struct TuningEntry {
  int bits = 0, n = 0, k = 0;
  int m_max = 0;
  int config = -1;
  double us = 0;
};
void load_tuning(const std::string& path);
void save_tuning(const std::string& path, const std::vector<TuningEntry>& entries, const std::string& device);
void install_tuning(std::vector<TuningEntry> entries);
int lookup_tuning(int bits, int n, int k, int m);

}  // namespace qwen38
