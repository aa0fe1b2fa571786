// ModelRunner: the step executor. Public behaviour follows the reference (src/model_runner.cpp): memory
// plan from the free device memory, one activation arena, eager prefill, CUDA-graph decode per batch-size
// bucket with padding rows on a private dummy slot, per-op event profiling. What is different:
//   * the ragged step metadata is per sequence on the host (count, position, slot) and expanded to per-token
//     arrays on the GPU by q38_pack_ragged, inside the same graph as the step;
//   * prefill_batch() runs chunks of several sequences in one ragged step;
//   * every decode bucket also owns a "core" graph without the host<->device copies, used to time the
//     device work of a step with inputs resident in HBM.
#include <algorithm>
#include <iostream>

#include "qwen38/api.h"

namespace qwen38 {

namespace {

constexpr size_t kMiB = 1024 * 1024;
constexpr int kMaxSplits = 64;
// From this run length on, a step's GDN layers use the chunked recurrence: a 64-token chunk costs about as much as
// a dozen sequential token updates.
constexpr int kGdnChunkedMinRun = 16;
constexpr int kBuckets[] = {1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256};

size_t up256(size_t x) { return (x + 255) / 256 * 256; }

std::string mib(size_t bytes) { return std::to_string((bytes + kMiB / 2) / kMiB) + " MiB"; }

int bucket_for(int n, int max_batch) {
  for (int b : kBuckets)
    if (b >= n && b <= max_batch) return b;
  return max_batch;
}

// Byte offsets of the step metadata block. The first part is written by the host and uploaded with one
// copy; the second part is produced on the device by the packing kernel.
struct MetaMap {
  size_t tokens = 0, seq_count = 0, seq_pos0 = 0, seq_slot = 0, row_slot = 0, step = 0, params = 0, sample_row = 0;
  size_t host_bytes = 0;
  size_t seq_start = 0, tok_pos = 0, tok_seq = 0;
  size_t bytes = 0;
  MetaMap() = default;
  MetaMap(int max_tokens, int max_rows) {
    size_t at = 0;
    auto take = [&](size_t n) {
      const size_t here = at;
      at = up256(at + n);
      return here;
    };
    tokens = take(size_t(max_tokens) * 4);
    seq_count = take(size_t(max_rows) * 4);
    seq_pos0 = take(size_t(max_rows) * 4);
    seq_slot = take(size_t(max_rows) * 4);
    row_slot = take(size_t(max_rows) * 4);
    step = take(size_t(max_rows) * 4);
    params = take(size_t(max_rows) * sizeof(kernels::SamplingParamsDev));
    sample_row = take(size_t(max_rows) * 4);
    host_bytes = at;
    seq_start = take(size_t(max_rows + 1) * 4);
    tok_pos = take(size_t(max_tokens) * 4);
    tok_seq = take(size_t(max_tokens) * 4);
    bytes = at;
  }
};

kernels::SamplingParamsDev to_dev(const SamplingParams& s) {
  return {s.temperature, s.top_k, s.top_p, s.min_p, s.presence_penalty, s.repetition_penalty, s.seed};
}
const kernels::SamplingParamsDev kGreedy{0.0f, 0, 1.0f, 0.0f, 0.0f, 1.0f, 0};

}  // namespace

std::string device_step_failure(unsigned int code, const std::string& where) {
  if (code == 0) return {};
  std::ostringstream os;
  os << where << ": a kernel of the step reported pipeline abort 0x" << std::hex << code
     << " (a bounded device-side wait ran out or an index left its pool); the step's results were discarded";
  return os.str();
}

DeviceStepError::DeviceStepError(unsigned int code, const std::string& where)
    : Error(device_step_failure(code, where)), code_(code) {}

std::string MemoryPlan::describe() const {
  std::ostringstream os;
  os << "device memory free at start " << mib(free_at_start) << ": weights " << mib(weights) << ", workspace "
     << mib(workspace) << ", GDN state " << mib(state) << ", KV " << mib(kv) << " (" << kv_tokens
     << " tokens), headroom " << mib(reserve);
  if (embedding_host) os << "; embedding in pinned host memory " << mib(embedding_host);
  return os.str();
}

struct ModelRunner::Impl {
  const ModelFile& file;
  ModelConfig cfg;
  RunnerOptions opt;
  DeviceInfo dev;
  MemoryPlan plan;
  std::unique_ptr<ModelWeights> weights;
  std::unique_ptr<KvCache> kv;
  std::unique_ptr<GdnStatePool> state;
  Stream stream;
  // side branch of the step: the a/b gate projection of a GDN layer needs only the layer's input, so it runs beside
  // the layer's (much larger) in-projection GEMM; fork / join events make it a parallel branch of the captured graph
  Stream side;
  Event fork_ev, join_ev;
  DeviceArena ws;
  int max_tokens = 0, max_rows = 0, dummy_slot = 0, proj_ld = 0;

  // activations
  float* residual = nullptr;
  __nv_bfloat16* xbf = nullptr;
  float* partials = nullptr;
  __nv_bfloat16* proj = nullptr;
  float* ab = nullptr;
  float* qkv = nullptr;
  __nv_bfloat16* mixer = nullptr;
  __nv_bfloat16* act = nullptr;
  __half* q16 = nullptr;
  float* logits = nullptr;
  float* split = nullptr;
  float* logprob_rows = nullptr;
  __nv_bfloat16* lm_x = nullptr;   // gathered rows for the LM head of ragged prefill steps
  float* lm_partials = nullptr;
  kernels::GemmWorkspace gemm_ws;
  float* gdn_scratch = nullptr;    // chunked GDN recurrence (prefill): per-chunk U0 / W / P
  size_t gdn_scratch_floats = 0;
  int32_t* history = nullptr;
  int* history_len = nullptr;
  int32_t* tokens_out = nullptr;
  float* logprob_out = nullptr;
  int32_t* targets = nullptr;

  MetaMap meta;
  uint8_t* meta_dev = nullptr;
  PinnedBuffer meta_host, out_host;
  // The library's device error status of the current step: one word of mapped pinned memory that the last kernel of
  // every step writes when some kernel of the step aborted its pipeline; read on the host after the step's sync.
  PinnedBuffer status_host;
  unsigned int* status_dev = nullptr;
  struct BucketGraphs {
    Graph step, core;
  };
  std::map<int, BucketGraphs> graphs;
  bool graphs_enabled = true;
  bool profiling = false;
  OpProfile prof;
  std::vector<std::pair<std::string, std::unique_ptr<Event>>> marks;
  Event t_begin{true}, t_end{true};
  bool timed = false;

  Impl(const ModelFile& f, const RunnerOptions& o) : file(f), cfg(f.config()), opt(o) {}

  template <typename T>
  T* hmeta(size_t off) const { return reinterpret_cast<T*>(meta_host.as<uint8_t>() + off); }
  template <typename T>
  T* dmeta(size_t off) const { return reinterpret_cast<T*>(meta_dev + off); }

  kernels::BatchDesc batch_desc(int seqs, int tokens, int max_per_seq) const {
    kernels::BatchDesc b;
    b.num_seqs = seqs;
    b.num_tokens = tokens;
    b.max_tokens_per_seq = max_per_seq;
    b.seq_start = dmeta<int>(meta.seq_start);
    b.seq_slot = dmeta<int>(meta.seq_slot);
    b.seq_pos0 = dmeta<int>(meta.seq_pos0);
    b.tok_pos = dmeta<int>(meta.tok_pos);
    b.tok_seq = dmeta<int>(meta.tok_seq);
    return b;
  }

  // The sequences [first_seq, first_seq + seqs) of the step as a batch of their own. Their token rows stay where they
  // are in the step's arrays (seq_start keeps absolute rows), so the kernels that walk a batch by sequence - attention,
  // the GDN recurrence - can serve the chunk rows and the single-token rows of a mixed step with the kernel that
  // suits each, while embed, the GEMMs, q/k-norm and the conv run once over all tokens.
  kernels::BatchDesc sub_batch(int first_seq, int first_token, int seqs, int tokens, int max_per_seq) const {
    kernels::BatchDesc b = batch_desc(seqs, tokens, max_per_seq);
    b.seq_start += first_seq;
    b.seq_slot += first_seq;
    b.seq_pos0 += first_seq;
    b.tok_pos += first_token;
    b.tok_seq += first_token;
    return b;
  }

  void mark(const char* name) {
    if (!profiling) return;
    auto ev = std::make_unique<Event>(true);
    ev->record(stream.get());
    marks.emplace_back(name, std::move(ev));
  }
  void collect_marks() {
    if (profiling && marks.size() >= 2) {
      marks.back().second->sync();
      for (size_t i = 1; i < marks.size(); ++i) {
        prof.ms[marks[i].first] += marks[i].second->ms_since(*marks[i - 1].second);
        prof.calls[marks[i].first] += 1;
      }
    }
    marks.clear();
  }

  void setup();
  void upload_meta() {
    QWEN38_CUDA(cudaMemcpyAsync(meta_dev, meta_host.get(), meta.host_bytes, cudaMemcpyHostToDevice, stream.get()));
  }
  void pack(int seqs, int tokens) {
    kernels::pack_ragged(dmeta<int>(meta.seq_count), dmeta<int>(meta.seq_pos0), seqs, tokens, dmeta<int>(meta.seq_start),
                         dmeta<int>(meta.tok_pos), dmeta<int>(meta.tok_seq), stream.get());
  }
  void collect_status() { kernels::collect_device_errors(status_dev, stream.get()); }
  // After the step's stream synchronisation: throws if a kernel of the step gave up, and re-arms the word.
  void check_status(const char* where) {
    volatile unsigned int* word = status_host.as<volatile unsigned int>();
    const unsigned int code = *word;
    if (code == 0) return;
    *word = 0;
    throw DeviceStepError(code, where);
  }
  // multi_seqs / multi_tokens: the leading sequences of the batch that bring more than one token, and their tokens;
  // the rest of the batch are single-token rows (a pure decode step has multi_seqs == 0, a pure prefill step none of
  // the latter)
  void forward(int m, const kernels::BatchDesc& batch, bool decode, int multi_seqs = -1, int multi_tokens = 0);
  void lm_head(const __nv_bfloat16* x, const float* part, int rows);
  void run_sampler(int rows);
  void download(int rows) {
    QWEN38_CUDA(cudaMemcpyAsync(out_host.get(), tokens_out, size_t(rows) * 4, cudaMemcpyDeviceToHost, stream.get()));
    QWEN38_CUDA(cudaMemcpyAsync(out_host.as<uint8_t>() + size_t(max_rows) * 4, logprob_out, size_t(rows) * 4,
                                cudaMemcpyDeviceToHost, stream.get()));
  }
  StepResult results(int rows) const {
    StepResult r;
    const int32_t* t = out_host.as<int32_t>();
    const float* lp = reinterpret_cast<const float*>(out_host.as<uint8_t>() + size_t(max_rows) * 4);
    r.tokens.assign(t, t + rows);
    r.logprobs.assign(lp, lp + rows);
    return r;
  }
  // host-side description of one sequence's run in this step
  void set_row(int i, int slot, int pos0, int count, int step, const kernels::SamplingParamsDev& p) {
    hmeta<int>(meta.seq_count)[i] = count;
    hmeta<int>(meta.seq_pos0)[i] = pos0;
    hmeta<int>(meta.seq_slot)[i] = slot;
    hmeta<int>(meta.row_slot)[i] = slot;
    hmeta<int>(meta.step)[i] = step;
    hmeta<kernels::SamplingParamsDev>(meta.params)[i] = p;
  }
  void fill_decode(std::span<const DecodeRow> rows, int bucket, bool all_dummy);
  void decode_body(int bucket) {
    const auto batch = batch_desc(bucket, bucket, 1);
    pack(bucket, bucket);
    forward(bucket, batch, true);
    lm_head(xbf, partials, bucket);
    run_sampler(bucket);
    collect_status();
  }
  void single_chunk_meta(int slot, int pos0, std::span<const int32_t> tokens, const SamplingParams* sample, int step);
};

void ModelRunner::Impl::setup() {
  dev = query_device(-1);
  if (dev.sm_major != 10) {
    std::cerr << "qwen38: warning: kernels are built for sm_100a (B200), running on " << dev.name << " (sm_"
              << dev.sm_major << dev.sm_minor << ")\n";
  }
  if (opt.embedding == EmbeddingPlacement::Host && !dev.can_map_host) opt.embedding = EmbeddingPlacement::Device;
  const int H = cfg.hidden_size, V = cfg.vocab_size;
  QWEN38_CHECK(opt.max_batch > 0, "max_batch must be positive");
  QWEN38_CHECK(opt.prefill_chunk >= 64 && opt.prefill_chunk % 64 == 0, "prefill chunk must be a multiple of 64");
  max_rows = opt.max_batch + 1;
  dummy_slot = opt.max_batch;
  max_tokens = std::max(opt.prefill_chunk, max_rows);

  plan.free_at_start = dev.free_mem;
  plan.weights = ModelWeights::required_device_bytes(file, opt.embedding);
  if (opt.embedding == EmbeddingPlacement::Host) plan.embedding_host = size_t(file.tensor("embed").bytes);
  proj_ld = 0;
  for (int i = 0; i < cfg.num_layers; ++i) {
    const std::string name = std::to_string(i) + (cfg.is_attention[size_t(i)] ? ".attn.qkvg" : ".gdn.qkvz");
    proj_ld = std::max(proj_ld, int(file.tensor(name).shape[0]));
  }
  const size_t T = size_t(max_tokens), R = size_t(max_rows);
  const size_t mixer_w = size_t(std::max(cfg.q_dim(), cfg.gdn_value_dim()));
  const size_t nv2 = 2 * size_t(std::max(1, cfg.linear_num_value_heads));
  const size_t gemm_partials = size_t(2) * size_t(dev.num_sms) * 128 * 512;  // stream-K partial tiles of a 512-token pass
  meta = MetaMap(max_tokens, max_rows);
  gdn_scratch_floats = cfg.linear_num_value_heads > 0 && max_tokens >= kGdnChunkedMinRun
                           ? kernels::gdn_chunk_scratch_floats(max_tokens, max_rows, cfg.linear_num_value_heads)
                           : 0;
  const size_t sizes[] = {
      T * H * 4, T * H * 2, T * size_t(cfg.norm_blocks()) * 4, T * size_t(proj_ld) * 2, T * nv2 * 4,
      T * size_t(std::max(128, cfg.gdn_conv_dim())) * 4, T * mixer_w * 2, T * size_t(cfg.intermediate_size) * 2,
      T * size_t(std::max(256, cfg.q_dim())) * 2, R * size_t(V) * 4,
      R * size_t(std::max(1, cfg.num_attention_heads)) * kMaxSplits * (kernels::kHeadDim + 2) * 4, T * 4,
      R * size_t(H) * 2, R * size_t(cfg.norm_blocks()) * 4, gemm_partials * 4, 65536 * 4,
      R * size_t(opt.history_cap) * 4, R * 4, R * 4, R * 4, T * 4, meta.bytes, gdn_scratch_floats * 4};
  size_t w = 4096;
  for (size_t s : sizes) w += up256(s);
  plan.workspace = w;
  plan.state = GdnStatePool::bytes_per_slot(cfg) * R;
  plan.reserve = opt.reserve_mib * kMiB;
  const size_t page_bytes = std::max<size_t>(KvCache::page_bytes_all_layers(cfg, opt.kv_dtype), 1);
  const size_t fixed = plan.weights + plan.workspace + plan.state + plan.reserve;
  QWEN38_CHECK(plan.free_at_start > fixed + 2 * page_bytes, "not enough GPU memory: need ", (fixed + 2 * page_bytes) / kMiB,
               " MiB before any KV cache, ", plan.free_at_start / kMiB, " MiB free");
  int64_t pages = int64_t((plan.free_at_start - fixed) / page_bytes);
  if (opt.kv_tokens > 0) pages = std::min<int64_t>(pages, ceil_div(opt.kv_tokens, kernels::kPageTokens) + 1);
  pages = std::min<int64_t>(pages, 1 << 22);
  plan.kv_pages = int(pages);
  plan.kv = size_t(pages) * page_bytes;
  plan.kv_tokens = (pages - 1) * kernels::kPageTokens;  // one page belongs to the dummy sequence

  weights = std::make_unique<ModelWeights>(file, opt.embedding);
  const int max_pages_per_seq = int(ceil_div(opt.max_context, kernels::kPageTokens));
  kv = std::make_unique<KvCache>(cfg, opt.kv_dtype, plan.kv_pages, max_rows, max_pages_per_seq);
  QWEN38_CHECK(kv->ensure(dummy_slot, 1), "KV cache too small");
  state = std::make_unique<GdnStatePool>(cfg, max_rows);

  ws = DeviceArena(plan.workspace);
  residual = ws.allocate_array<float>(T * H);
  xbf = ws.allocate_array<__nv_bfloat16>(T * H);
  partials = ws.allocate_array<float>(T * size_t(cfg.norm_blocks()));
  proj = ws.allocate_array<__nv_bfloat16>(T * size_t(proj_ld));
  ab = ws.allocate_array<float>(T * nv2);
  qkv = ws.allocate_array<float>(T * size_t(std::max(128, cfg.gdn_conv_dim())));
  mixer = ws.allocate_array<__nv_bfloat16>(T * mixer_w);
  act = ws.allocate_array<__nv_bfloat16>(T * size_t(cfg.intermediate_size));
  q16 = ws.allocate_array<__half>(T * size_t(std::max(256, cfg.q_dim())));
  logits = ws.allocate_array<float>(R * size_t(V));
  split = ws.allocate_array<float>(R * size_t(std::max(1, cfg.num_attention_heads)) * kMaxSplits * (kernels::kHeadDim + 2));
  logprob_rows = ws.allocate_array<float>(T);
  lm_x = ws.allocate_array<__nv_bfloat16>(R * size_t(H));
  lm_partials = ws.allocate_array<float>(R * size_t(cfg.norm_blocks()));
  gemm_ws.partials = ws.allocate_array<float>(gemm_partials);
  gemm_ws.partial_floats = gemm_partials;
  gemm_ws.counters = ws.allocate_array<int>(65536);
  if (gdn_scratch_floats) gdn_scratch = ws.allocate_array<float>(gdn_scratch_floats);
  gemm_ws.num_counters = 65536;
  history = ws.allocate_array<int32_t>(R * size_t(opt.history_cap));
  history_len = ws.allocate_array<int>(R);
  tokens_out = ws.allocate_array<int32_t>(R);
  logprob_out = ws.allocate_array<float>(R);
  targets = ws.allocate_array<int32_t>(T);
  meta_dev = static_cast<uint8_t*>(ws.allocate(meta.bytes));
  QWEN38_CUDA(cudaMemset(gemm_ws.counters, 0, 65536 * 4));
  QWEN38_CUDA(cudaMemset(history_len, 0, R * 4));
  QWEN38_CUDA(cudaMemset(meta_dev, 0, meta.bytes));
  meta_host = PinnedBuffer(meta.host_bytes, false);
  std::memset(meta_host.get(), 0, meta.host_bytes);
  out_host = PinnedBuffer(R * 8, false);
  status_host = PinnedBuffer(64, true);
  std::memset(status_host.get(), 0, 64);
  status_dev = static_cast<unsigned int*>(status_host.device_ptr());
  collect_status();  // looks the library's error words up once, outside any capture
  stream.sync();
  *status_host.as<volatile unsigned int>() = 0;  // whatever an earlier user of the library left behind is not ours
  graphs_enabled = opt.cuda_graphs;
  if (opt.verbose) std::cerr << "qwen38: " << plan.describe() << "\n";
}

// The kernel sequence of one step over m tokens (reference src/model_runner.cpp:292-410).
void ModelRunner::Impl::forward(int m, const kernels::BatchDesc& batch, bool decode, int multi_seqs, int multi_tokens) {
  cudaStream_t s = stream.get();
  if (multi_seqs < 0 || multi_seqs >= batch.num_seqs) {  // not a mixed step
    multi_seqs = decode ? 0 : batch.num_seqs;
    multi_tokens = decode ? 0 : m;
  }
  const int single_seqs = batch.num_seqs - multi_seqs;  // rows of one token each, placed after the chunk rows
  const bool mixed = multi_seqs > 0 && single_seqs > 0;
  const kernels::BatchDesc chunk_part = mixed ? sub_batch(0, 0, multi_seqs, multi_tokens, batch.max_tokens_per_seq) : batch;
  const kernels::BatchDesc single_part =
      mixed ? sub_batch(multi_seqs, multi_tokens, single_seqs, single_seqs, 1) : batch;
  const int H = cfg.hidden_size;
  const float eps = cfg.rms_norm_eps;
  const kernels::KvCacheDesc kvd = kv->desc();
  const kernels::GdnStateDesc sd = state->desc();
  kernels::GdnDims gd;
  gd.num_k_heads = cfg.linear_num_key_heads;
  gd.num_v_heads = cfg.linear_num_value_heads;
  gd.conv_dim = cfg.gdn_conv_dim();
  gd.ld_proj = proj_ld;

  mark("start");
  kernels::embed(weights->embedding(), dmeta<int32_t>(meta.tokens), m, H, residual, xbf, partials, s);
  mark("embed");

  kernels::GemmEpilogue into_residual;
  into_residual.kind = kernels::Epilogue::Residual;
  into_residual.residual = residual;
  into_residual.xbf = xbf;
  into_residual.partials_out = partials;

  int attn_i = 0, gdn_i = 0;
  for (const LayerWeights& W : weights->layers()) {
    kernels::GemmEpilogue in;
    in.kind = kernels::Epilogue::StoreBF16;
    in.out = proj;
    in.ldo = proj_ld;
    in.n_store = W.in_proj.rows;
    in.partials_in = partials;
    in.hidden = H;
    in.eps = eps;
    const bool side_ab = !W.attention && !profiling;  // the per-op profile keeps everything on one stream
    if (side_ab) {
      fork_ev.record(s);
      QWEN38_CUDA(cudaStreamWaitEvent(side.get(), fork_ev.get(), 0));
      kernels::gdn_ab(xbf, m, H, W.ab, W.ab_rows, partials, eps, ab, side.get());
      join_ev.record(side.get());
    }
    kernels::qgemm(xbf, m, W.in_proj, in, gemm_ws, s);
    mark(W.attention ? "gemm.attn_qkvg" : "gemm.gdn_qkvz");
    if (W.attention) {
      kernels::QkNormRopeParams qp;
      qp.proj = proj;
      qp.ld_proj = proj_ld;
      qp.q_norm = W.q_norm;
      qp.k_norm = W.k_norm;
      qp.eps = eps;
      qp.rope_theta = float(cfg.rope_theta);
      qp.num_q_heads = cfg.num_attention_heads;
      qp.num_kv_heads = cfg.num_key_value_heads;
      qp.q_out = q16;
      qp.attn_layer = attn_i;
      kernels::qk_norm_rope_append(qp, batch, kvd, s);
      mark("attn.qk_norm_rope_kv");
      kernels::AttentionParams ap;
      ap.q = q16;
      ap.gate = proj + cfg.q_dim();
      ap.ld_gate = proj_ld;
      ap.out = mixer;
      ap.num_q_heads = cfg.num_attention_heads;
      ap.num_kv_heads = cfg.num_key_value_heads;
      ap.attn_layer = attn_i;
      ap.split_scratch = split;
      ap.max_splits = kMaxSplits;
      if (decode) {
        kernels::attention_decode(ap, batch, kvd, s);
      } else if (mixed) {
        // chunk rows through the query-tiled kernel (no key split: the scratch serves the single-token rows), the
        // single-token rows through split-KV flash decoding
        kernels::attention_decode(ap, single_part, kvd, s);
        ap.split_scratch = nullptr;
        kernels::attention_prefill(ap, chunk_part, kvd, s);
      } else {  // the scratch of max_rows x kMaxSplits states seen as one row per prompt token of this step
        ap.max_splits = std::min(kMaxSplits, int(size_t(max_rows) * kMaxSplits / size_t(std::max(1, m))));
        ap.scratch_rows = ap.max_splits > 1 ? m : 0;
        kernels::attention_prefill(ap, batch, kvd, s);
      }
      mark(decode ? "attn.decode" : "attn.prefill");
      ++attn_i;
    } else {
      if (side_ab) QWEN38_CUDA(cudaStreamWaitEvent(s, join_ev.get(), 0));
      else kernels::gdn_ab(xbf, m, H, W.ab, W.ab_rows, partials, eps, ab, s);
      mark("gdn.ab");
      kernels::GdnConvParams cp;
      cp.proj = proj;
      cp.conv_w = W.conv;
      cp.qkv = qkv;
      cp.gdn_layer = gdn_i;
      kernels::gdn_conv(cp, gd, batch, sd, s);
      mark("gdn.conv");
      kernels::GdnRecurrenceParams rp;
      rp.qkv = qkv;
      rp.ab = ab;
      rp.A = W.A;
      rp.dt_bias = W.dt_bias;
      rp.z = proj + cfg.gdn_conv_dim();
      rp.ld_z = proj_ld;
      rp.norm_w = W.gdn_norm;
      rp.eps = eps;
      rp.out = mixer;
      rp.gdn_layer = gdn_i;
      // runs of prefill length take the chunked form (token-parallel preparation + per-chunk state scan)
      if (gdn_scratch && chunk_part.max_tokens_per_seq >= kGdnChunkedMinRun)
        kernels::gdn_recurrence_chunked(rp, gd, chunk_part, sd, gdn_scratch, gdn_scratch_floats, s);
      else
        kernels::gdn_recurrence(rp, gd, chunk_part, sd, s);
      if (mixed) kernels::gdn_recurrence(rp, gd, single_part, sd, s);  // the state-streaming decode kernel
      mark("gdn.recurrence");
      ++gdn_i;
    }
    kernels::qgemm(mixer, m, W.out_proj, into_residual, gemm_ws, s);
    mark(W.attention ? "gemm.attn_o" : "gemm.gdn_out");

    kernels::GemmEpilogue mlp;
    mlp.kind = kernels::Epilogue::SwiGLU;
    mlp.out = act;
    mlp.ldo = cfg.intermediate_size;
    mlp.partials_in = partials;
    mlp.hidden = H;
    mlp.eps = eps;
    kernels::qgemm(xbf, m, W.gate_up, mlp, gemm_ws, s);
    mark("gemm.mlp_gate_up");
    kernels::qgemm(act, m, W.down, into_residual, gemm_ws, s);
    mark("gemm.mlp_down");
  }
}

void ModelRunner::Impl::lm_head(const __nv_bfloat16* x, const float* part, int rows) {
  if (rows <= 0) return;
  kernels::GemmEpilogue head;
  head.kind = kernels::Epilogue::StoreF32;
  head.out = logits;
  head.ldo = cfg.vocab_size;
  head.partials_in = part;
  head.hidden = cfg.hidden_size;
  head.eps = cfg.rms_norm_eps;
  kernels::qgemm(x, rows, weights->lm_head(), head, gemm_ws, stream.get());
  mark("gemm.lm_head");
}

void ModelRunner::Impl::run_sampler(int rows) {
  kernels::SamplingArgs sa;
  sa.logits = logits;
  sa.ld = cfg.vocab_size;
  sa.vocab = cfg.vocab_size;
  sa.params = dmeta<kernels::SamplingParamsDev>(meta.params);
  sa.row_slot = dmeta<int>(meta.row_slot);
  sa.history = history;
  sa.history_len = history_len;
  sa.history_cap = opt.history_cap;
  sa.step = dmeta<int>(meta.step);
  sa.tokens_out = tokens_out;
  sa.logprob_out = logprob_out;
  kernels::sample(sa, rows, stream.get());
  mark("sample");
}

ModelRunner::ModelRunner(const ModelFile& file, const RunnerOptions& options)
    : impl_(std::make_unique<Impl>(file, options)) {
  impl_->setup();
}
ModelRunner::~ModelRunner() = default;

const ModelConfig& ModelRunner::config() const { return impl_->cfg; }
const RunnerOptions& ModelRunner::options() const { return impl_->opt; }
const MemoryPlan& ModelRunner::memory() const { return impl_->plan; }
const DeviceInfo& ModelRunner::device() const { return impl_->dev; }
int ModelRunner::num_slots() const { return impl_->opt.max_batch; }
KvCache& ModelRunner::kv() { return *impl_->kv; }
const ModelWeights& ModelRunner::weights() const { return *impl_->weights; }
cudaStream_t ModelRunner::stream() const { return impl_->stream.get(); }
const kernels::GemmWorkspace& ModelRunner::gemm_workspace() const { return impl_->gemm_ws; }
void ModelRunner::set_profiling(bool on) { impl_->profiling = on; }
const OpProfile& ModelRunner::profile() const { return impl_->prof; }
void ModelRunner::clear_profile() { impl_->prof = OpProfile{}; }
void ModelRunner::set_graphs_enabled(bool on) { impl_->graphs_enabled = on; }

float ModelRunner::last_step_device_ms() const {
  if (!impl_->timed) return 0.0f;
  impl_->t_end.sync();
  return impl_->t_end.ms_since(impl_->t_begin);
}

void ModelRunner::reset_slot(int slot) {
  QWEN38_CHECK(slot >= 0 && slot < impl_->opt.max_batch, "reset_slot: slot out of range");
  impl_->state->reset(slot, impl_->stream.get());
  QWEN38_CUDA(cudaMemsetAsync(impl_->history_len + slot, 0, sizeof(int), impl_->stream.get()));
}

void ModelRunner::Impl::single_chunk_meta(int slot, int pos0, std::span<const int32_t> tokens,
                                          const SamplingParams* sample, int step) {
  std::memcpy(hmeta<int32_t>(meta.tokens), tokens.data(), tokens.size() * 4);
  set_row(0, slot, pos0, int(tokens.size()), step, sample ? to_dev(*sample) : kGreedy);
}

StepResult ModelRunner::prefill(int slot, int pos0, std::span<const int32_t> tokens, const SamplingParams* sample,
                                int step) {
  PrefillRow row;
  row.slot = slot;
  row.pos0 = pos0;
  row.tokens = tokens;
  row.sample = sample;
  row.step = step;
  return prefill_batch(std::span<const PrefillRow>(&row, 1));
}

StepResult ModelRunner::prefill_batch(std::span<const PrefillRow> rows) {
  Impl& I = *impl_;
  const int nseq = int(rows.size());
  QWEN38_CHECK(nseq > 0 && nseq <= I.opt.max_batch, "prefill: ", nseq, " sequences in one step (max ", I.opt.max_batch, ")");
  // Order inside the step: rows that bring a chunk of several tokens first, single-token rows (a generating sequence's
  // next token, or a one-token tail of a prompt) after them, each group in the caller's order. The forward pass then
  // serves the two groups with the attention / recurrence kernel that suits each; results keep the caller's order.
  std::vector<int> order;
  order.reserve(size_t(nseq));
  int multi_seqs = 0, multi_tokens = 0;
  for (int pass = 0; pass < 2; ++pass)
    for (int i = 0; i < nseq; ++i) {
      const bool single = rows[size_t(i)].tokens.size() == 1;
      if (single == (pass == 1)) order.push_back(i);
    }
  std::vector<int> last_token_row(size_t(nseq), 0);  // per caller row: the step's token row of its last token
  int total = 0, longest = 0, samples = 0;
  for (int k = 0; k < nseq; ++k) {
    const int i = order[size_t(k)];
    const PrefillRow& r = rows[size_t(i)];
    const int n = int(r.tokens.size());
    QWEN38_CHECK(n > 0, "prefill: empty chunk");
    QWEN38_CHECK(r.slot >= 0 && r.slot < I.opt.max_batch, "prefill: slot out of range");
    QWEN38_CHECK(I.kv->pages_of(r.slot) * kernels::kPageTokens >= r.pos0 + n, "prefill: KV pages not reserved");
    for (int j = 0; j < i; ++j) QWEN38_CHECK(rows[size_t(j)].slot != r.slot, "prefill: a slot appears twice in one step");
    QWEN38_CHECK(total + n <= I.max_tokens, "prefill: step of more than ", I.max_tokens, " tokens");
    std::memcpy(I.hmeta<int32_t>(I.meta.tokens) + total, r.tokens.data(), size_t(n) * 4);
    I.set_row(k, r.slot, r.pos0, n, 0, kGreedy);
    total += n;
    longest = std::max(longest, n);
    last_token_row[size_t(i)] = total - 1;
    if (n > 1) {
      ++multi_seqs;
      multi_tokens += n;
    }
  }
  QWEN38_CHECK(total <= I.opt.prefill_chunk, "prefill: chunk of ", total, " tokens (max ", I.opt.prefill_chunk, ")");
  // sampler rows are compact: row j of the sampler = j-th sequence (in the caller's order) that asked for a sample
  for (int i = 0; i < nseq; ++i) {
    const PrefillRow& r = rows[size_t(i)];
    if (!r.sample) continue;
    I.hmeta<int>(I.meta.row_slot)[samples] = r.slot;
    I.hmeta<int>(I.meta.step)[samples] = r.step;
    I.hmeta<kernels::SamplingParamsDev>(I.meta.params)[samples] = to_dev(*r.sample);
    I.hmeta<int>(I.meta.sample_row)[samples] = last_token_row[size_t(i)];
    ++samples;
  }
  cudaStream_t s = I.stream.get();
  I.kv->sync(s);
  I.upload_meta();
  I.t_begin.record(s);
  I.pack(nseq, total);
  I.forward(total, I.batch_desc(nseq, total, longest), false, multi_seqs, multi_tokens);
  StepResult result;
  if (samples > 0) {
    const int H = I.cfg.hidden_size, nb = I.cfg.norm_blocks();
    if (samples == 1) {
      const int row = I.hmeta<int>(I.meta.sample_row)[0];
      I.lm_head(I.xbf + size_t(row) * H, I.partials + size_t(row) * nb, 1);
    } else {
      kernels::gather_rows(I.xbf, I.partials, I.dmeta<int>(I.meta.sample_row), samples, H, I.lm_x, I.lm_partials, s);
      I.lm_head(I.lm_x, I.lm_partials, samples);
    }
    I.run_sampler(samples);
  }
  I.collect_status();
  I.t_end.record(s);
  I.timed = true;
  if (samples > 0) I.download(samples);
  I.stream.sync();
  I.collect_marks();
  I.check_status("prefill step");
  if (samples > 0) result = I.results(samples);
  return result;
}

void ModelRunner::Impl::fill_decode(std::span<const DecodeRow> rows, int bucket, bool all_dummy) {
  const int n = int(rows.size());
  int32_t* tok = hmeta<int32_t>(meta.tokens);
  for (int i = 0; i < bucket; ++i) {
    if (i < n && !all_dummy) {
      const DecodeRow& r = rows[size_t(i)];
      tok[i] = r.token;
      set_row(i, r.slot, r.position, 1, r.step, to_dev(r.sampling));
    } else {
      tok[i] = 0;
      set_row(i, dummy_slot, 0, 1, 0, kGreedy);
    }
  }
}

StepResult ModelRunner::decode(std::span<const DecodeRow> rows) {
  Impl& I = *impl_;
  const int n = int(rows.size());
  QWEN38_CHECK(n > 0 && n <= I.opt.max_batch, "decode: batch of ", n, " rows (max ", I.opt.max_batch, ")");
  for (const DecodeRow& r : rows) {
    QWEN38_CHECK(r.slot >= 0 && r.slot < I.opt.max_batch, "decode: slot out of range");
    QWEN38_CHECK(I.kv->pages_of(r.slot) * kernels::kPageTokens > r.position, "decode: KV page missing");
  }
  const bool use_graph = I.graphs_enabled && !I.profiling;
  const int bucket = use_graph ? bucket_for(n, I.opt.max_batch) : n;
  cudaStream_t s = I.stream.get();
  I.kv->sync(s);
  if (use_graph) {
    auto it = I.graphs.find(bucket);
    if (it == I.graphs.end()) {
      // warm-up outside capture on the dummy slot only, so that no live sequence advances
      I.fill_decode(rows, bucket, true);
      I.upload_meta();
      I.decode_body(bucket);
      I.stream.sync();
      Impl::BucketGraphs g;
      g.step.begin_capture(s);
      I.upload_meta();  // a memcpy node: reads the pinned block at launch time
      I.decode_body(bucket);
      I.download(bucket);
      g.step.end_capture(s);
      g.core.begin_capture(s);
      I.decode_body(bucket);
      g.core.end_capture(s);
      it = I.graphs.emplace(bucket, std::move(g)).first;
    }
    I.fill_decode(rows, bucket, false);
    I.t_begin.record(s);
    it->second.step.launch(s);
    I.t_end.record(s);
  } else {
    I.fill_decode(rows, bucket, false);
    I.upload_meta();
    I.t_begin.record(s);
    I.decode_body(bucket);
    I.t_end.record(s);
    I.download(bucket);
  }
  I.timed = true;
  I.stream.sync();
  I.collect_marks();
  I.check_status("decode step");
  StepResult r = I.results(bucket);
  r.tokens.resize(size_t(n));
  r.logprobs.resize(size_t(n));
  return r;
}

std::vector<float> ModelRunner::score(int slot, int pos0, std::span<const int32_t> tokens,
                                      std::span<const int32_t> targets) {
  Impl& I = *impl_;
  QWEN38_CHECK(tokens.size() == targets.size(), "score: tokens/targets size");
  std::vector<float> out;
  out.reserve(tokens.size());
  const int H = I.cfg.hidden_size, nb = I.cfg.norm_blocks(), V = I.cfg.vocab_size;
  cudaStream_t s = I.stream.get();
  int pos = pos0;
  for (size_t off = 0; off < tokens.size(); off += size_t(I.opt.prefill_chunk)) {
    const int n = int(std::min<size_t>(size_t(I.opt.prefill_chunk), tokens.size() - off));
    QWEN38_CHECK(I.kv->ensure(slot, pos + n), "score: KV cache full");
    I.single_chunk_meta(slot, pos, tokens.subspan(off, size_t(n)), nullptr, 0);
    I.kv->sync(s);
    I.upload_meta();
    QWEN38_CUDA(cudaMemcpyAsync(I.targets, targets.data() + off, size_t(n) * 4, cudaMemcpyHostToDevice, s));
    I.pack(1, n);
    I.forward(n, I.batch_desc(1, n, n), false);
    for (int r0 = 0; r0 < n; r0 += I.max_rows) {
      const int rows = std::min(I.max_rows, n - r0);
      I.lm_head(I.xbf + size_t(r0) * H, I.partials + size_t(r0) * nb, rows);
      kernels::target_logprobs(I.logits, V, V, I.targets + r0, rows, I.logprob_rows + r0, s);
    }
    std::vector<float> chunk(static_cast<size_t>(n));
    QWEN38_CUDA(cudaMemcpyAsync(chunk.data(), I.logprob_rows, size_t(n) * 4, cudaMemcpyDeviceToHost, s));
    I.collect_status();
    I.stream.sync();
    I.collect_marks();
    I.check_status("score step");
    out.insert(out.end(), chunk.begin(), chunk.end());
    pos += n;
  }
  return out;
}

std::vector<float> ModelRunner::prefill_logits(int slot, int pos0, std::span<const int32_t> tokens) {
  Impl& I = *impl_;
  const int n = int(tokens.size());
  QWEN38_CHECK(n > 0 && n <= I.opt.prefill_chunk, "prefill_logits: chunk size");
  QWEN38_CHECK(I.kv->ensure(slot, pos0 + n), "prefill_logits: KV cache full");
  const int H = I.cfg.hidden_size, nb = I.cfg.norm_blocks(), V = I.cfg.vocab_size;
  cudaStream_t s = I.stream.get();
  I.single_chunk_meta(slot, pos0, tokens, nullptr, 0);
  I.kv->sync(s);
  I.upload_meta();
  I.pack(1, n);
  I.forward(n, I.batch_desc(1, n, n), false);
  std::vector<float> out(size_t(n) * size_t(V));
  for (int r0 = 0; r0 < n; r0 += I.max_rows) {
    const int rows = std::min(I.max_rows, n - r0);
    I.lm_head(I.xbf + size_t(r0) * H, I.partials + size_t(r0) * nb, rows);
    QWEN38_CUDA(cudaMemcpyAsync(out.data() + size_t(r0) * V, I.logits, size_t(rows) * V * 4, cudaMemcpyDeviceToHost, s));
    I.collect_status();
    I.stream.sync();
  }
  I.collect_marks();
  I.check_status("prefill step");
  return out;
}

std::vector<float> ModelRunner::last_logits(int rows) {
  Impl& I = *impl_;
  QWEN38_CHECK(rows > 0 && rows <= I.max_rows, "last_logits: rows");
  std::vector<float> out(size_t(rows) * size_t(I.cfg.vocab_size));
  QWEN38_CUDA(cudaMemcpyAsync(out.data(), I.logits, out.size() * 4, cudaMemcpyDeviceToHost, I.stream.get()));
  I.stream.sync();
  return out;
}

float ModelRunner::replay_decode_core(int rows, int iters) {
  Impl& I = *impl_;
  const int bucket = bucket_for(rows, I.opt.max_batch);
  auto it = I.graphs.find(bucket);
  QWEN38_CHECK(it != I.graphs.end() && it->second.core.valid(), "replay: run decode() with this batch size first");
  cudaStream_t s = I.stream.get();
  Event a(true), b(true);
  a.record(s);
  for (int i = 0; i < iters; ++i) it->second.core.launch(s);
  b.record(s);
  b.sync();
  return b.ms_since(a) / float(std::max(1, iters));
}

}  // namespace qwen38
