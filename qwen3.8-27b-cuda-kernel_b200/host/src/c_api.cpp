// C ABI over the C++ host API (include/q38_engine.h): opaque handles, status codes, no exceptions across
// the boundary.
#include <cstdio>
#include <deque>

#include "q38_engine.h"
#include "qwen38/api.h"

using namespace qwen38;

struct q38e_model {
  std::unique_ptr<ModelFile> file;
  std::string summary;
};
struct q38e_runner {
  std::unique_ptr<ModelRunner> owned;
  ModelRunner* r = nullptr;
};
struct q38e_engine {
  std::unique_ptr<Engine> e;
  std::deque<RequestResult> done;
  q38e_runner runner_view;
};

namespace {
thread_local std::string g_err;

template <typename F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
  } catch (...) {
    g_err = "unknown error";
  }
  return -1;
}

SamplingParams from_c(const q38e_sampling& s) {
  SamplingParams p;
  p.temperature = s.temperature;
  p.top_k = s.top_k;
  p.top_p = s.top_p;
  p.min_p = s.min_p;
  p.presence_penalty = s.presence_penalty;
  p.repetition_penalty = s.repetition_penalty;
  p.seed = s.seed;
  return p;
}

RunnerOptions from_c(const q38e_runner_options& o) {
  RunnerOptions r;
  r.max_batch = o.max_batch;
  r.prefill_chunk = o.prefill_chunk;
  r.kv_dtype = o.kv_dtype == 0 ? kernels::KvDtype::Int8 : kernels::KvDtype::BF16;
  r.kv_tokens = o.kv_tokens;
  r.max_context = o.max_context;
  r.reserve_mib = o.reserve_mib;
  r.embedding = o.embedding_on_host ? EmbeddingPlacement::Host : EmbeddingPlacement::Device;
  r.cuda_graphs = o.cuda_graphs != 0;
  r.history_cap = o.history_cap;
  r.verbose = o.verbose != 0;
  return r;
}
}  // namespace

extern "C" {

const char* q38e_last_error(void) { return g_err.c_str(); }

void q38e_default_runner_options(q38e_runner_options* o) {
  const RunnerOptions d;
  o->max_batch = d.max_batch;
  o->prefill_chunk = d.prefill_chunk;
  o->kv_dtype = int(d.kv_dtype);
  o->kv_tokens = d.kv_tokens;
  o->max_context = d.max_context;
  o->reserve_mib = d.reserve_mib;
  o->embedding_on_host = d.embedding == EmbeddingPlacement::Host;
  o->cuda_graphs = d.cuda_graphs;
  o->history_cap = d.history_cap;
  o->verbose = d.verbose;
}

int q38e_step_status(unsigned int device_error_word, const char* where) {
  return guard([&] {
    if (device_error_word != 0) throw DeviceStepError(device_error_word, where ? where : "step");
  });
}

int q38e_tuning_load(const char* path) {
  return guard([&] {
    if (path == nullptr || path[0] == '\0') install_tuning({});
    else load_tuning(path);
  });
}
int q38e_tuning_lookup(int bits, int n, int k, int m) { return lookup_tuning(bits, n, k, m); }

int q38e_model_open(const char* path, q38e_model** out) {
  return guard([&] {
    auto m = std::make_unique<q38e_model>();
    m->file = ModelFile::open(path);
    m->summary = m->file->config().summary();
    *out = m.release();
  });
}
void q38e_model_close(q38e_model* m) { delete m; }
int q38e_model_vocab(const q38e_model* m) { return m->file->config().vocab_size; }
int q38e_model_hidden(const q38e_model* m) { return m->file->config().hidden_size; }
int q38e_model_layers(const q38e_model* m) { return m->file->config().num_layers; }
const char* q38e_model_summary(const q38e_model* m) { return m->summary.c_str(); }
int q38e_model_dequant(const q38e_model* m, const char* name, float* out, size_t out_floats) {
  return guard([&] {
    const BQView v = BQView::from_file(*m->file, name);
    QWEN38_CHECK(size_t(v.n * v.k) <= out_floats, "dequant: output buffer too small");
    for (int64_t r = 0; r < v.n; ++r) v.dequant_row(r, out + r * v.k);
  });
}

int q38e_runner_create(const q38e_model* m, const q38e_runner_options* o, q38e_runner** out) {
  return guard([&] {
    auto h = std::make_unique<q38e_runner>();
    h->owned = std::make_unique<ModelRunner>(*m->file, from_c(*o));
    h->r = h->owned.get();
    *out = h.release();
  });
}
void q38e_runner_destroy(q38e_runner* r) { delete r; }
int q38e_runner_reset_slot(q38e_runner* r, int slot) { return guard([&] { r->r->reset_slot(slot); }); }
int q38e_runner_kv_ensure(q38e_runner* r, int slot, int tokens, int* ok) {
  return guard([&] { *ok = r->r->kv().ensure(slot, tokens) ? 1 : 0; });
}
int q38e_runner_kv_release(q38e_runner* r, int slot) { return guard([&] { r->r->kv().release(slot); }); }
int q38e_runner_kv_pages(q38e_runner* r, int slot, int* pages_out, int capacity, int* count) {
  return guard([&] {
    const auto& pages = r->r->kv().page_list(slot);
    *count = int(pages.size());
    for (int i = 0; i < int(pages.size()) && i < capacity; ++i) pages_out[i] = pages[size_t(i)];
  });
}
int q38e_runner_kv_free_pages(q38e_runner* r, int* count) { return guard([&] { *count = r->r->kv().free_pages(); }); }

int q38e_runner_prefill(q38e_runner* r, const q38e_prefill_row* rows, int num_rows, int32_t* tokens_out,
                        float* logprobs_out, int* num_out) {
  return guard([&] {
    std::vector<PrefillRow> pr(static_cast<size_t>(num_rows));
    std::vector<SamplingParams> sp(static_cast<size_t>(num_rows));
    for (int i = 0; i < num_rows; ++i) {
      pr[size_t(i)].slot = rows[i].slot;
      pr[size_t(i)].pos0 = rows[i].pos0;
      pr[size_t(i)].tokens = std::span<const int32_t>(rows[i].tokens, size_t(rows[i].num_tokens));
      sp[size_t(i)] = from_c(rows[i].sampling);
      pr[size_t(i)].sample = rows[i].sample ? &sp[size_t(i)] : nullptr;
      pr[size_t(i)].step = rows[i].step;
    }
    const StepResult res = r->r->prefill_batch(pr);
    if (num_out) *num_out = int(res.tokens.size());
    for (size_t i = 0; i < res.tokens.size(); ++i) {
      if (tokens_out) tokens_out[i] = res.tokens[i];
      if (logprobs_out) logprobs_out[i] = res.logprobs[i];
    }
  });
}

int q38e_runner_decode(q38e_runner* r, const q38e_decode_row* rows, int num_rows, int32_t* tokens_out,
                       float* logprobs_out) {
  return guard([&] {
    std::vector<DecodeRow> dr(static_cast<size_t>(num_rows));
    for (int i = 0; i < num_rows; ++i) {
      dr[size_t(i)].slot = rows[i].slot;
      dr[size_t(i)].position = rows[i].position;
      dr[size_t(i)].token = rows[i].token;
      dr[size_t(i)].sampling = from_c(rows[i].sampling);
      dr[size_t(i)].step = rows[i].step;
    }
    const StepResult res = r->r->decode(dr);
    for (size_t i = 0; i < res.tokens.size(); ++i) {
      tokens_out[i] = res.tokens[i];
      if (logprobs_out) logprobs_out[i] = res.logprobs[i];
    }
  });
}

int q38e_runner_prefill_logits(q38e_runner* r, int slot, int pos0, const int32_t* tokens, int n, float* logits_out) {
  return guard([&] {
    const auto v = r->r->prefill_logits(slot, pos0, std::span<const int32_t>(tokens, size_t(n)));
    std::memcpy(logits_out, v.data(), v.size() * sizeof(float));
  });
}

int q38e_runner_score(q38e_runner* r, int slot, int pos0, const int32_t* tokens, const int32_t* targets, int n,
                      float* logprobs_out) {
  return guard([&] {
    const auto v = r->r->score(slot, pos0, std::span<const int32_t>(tokens, size_t(n)),
                               std::span<const int32_t>(targets, size_t(n)));
    std::memcpy(logprobs_out, v.data(), v.size() * sizeof(float));
  });
}

int q38e_runner_set_profiling(q38e_runner* r, int on) { return guard([&] { r->r->set_profiling(on != 0); }); }
int q38e_runner_set_graphs(q38e_runner* r, int on) { return guard([&] { r->r->set_graphs_enabled(on != 0); }); }
int q38e_runner_profile(q38e_runner* r, char* buf, size_t cap, int clear) {
  return guard([&] {
    std::string text;
    const OpProfile& p = r->r->profile();
    for (const auto& [name, ms] : p.ms) {
      char line[160];
      std::snprintf(line, sizeof(line), "%s %.6f %d\n", name.c_str(), ms, p.calls.at(name));
      text += line;
    }
    if (cap) {
      std::snprintf(buf, cap, "%s", text.c_str());
    }
    if (clear) r->r->clear_profile();
  });
}
int q38e_runner_last_step_ms(q38e_runner* r, float* ms) { return guard([&] { *ms = r->r->last_step_device_ms(); }); }
int q38e_runner_replay_decode_core(q38e_runner* r, int rows, int iters, float* ms_per_step) {
  return guard([&] { *ms_per_step = r->r->replay_decode_core(rows, iters); });
}
int q38e_runner_last_logits(q38e_runner* r, int rows, float* logits_out) {
  return guard([&] {
    const auto v = r->r->last_logits(rows);
    std::memcpy(logits_out, v.data(), v.size() * sizeof(float));
  });
}
int q38e_runner_memory(q38e_runner* r, size_t* weights, size_t* workspace, size_t* state, size_t* kv, int64_t* kv_tokens) {
  return guard([&] {
    const MemoryPlan& p = r->r->memory();
    *weights = p.weights;
    *workspace = p.workspace;
    *state = p.state;
    *kv = p.kv;
    *kv_tokens = p.kv_tokens;
  });
}

int q38e_engine_create(const q38e_model* m, const q38e_engine_options* o, q38e_engine** out) {
  return guard([&] {
    EngineOptions eo;
    eo.runner = from_c(o->runner);
    eo.seed = o->seed;
    eo.ragged_prefill = o->ragged_prefill != 0;
    eo.mixed_steps = o->mixed_steps != 0;
    auto h = std::make_unique<q38e_engine>();
    h->e = std::make_unique<Engine>(*m->file, eo);
    h->runner_view.r = &h->e->runner();
    *out = h.release();
  });
}
void q38e_engine_destroy(q38e_engine* e) { delete e; }

int q38e_engine_submit(q38e_engine* e, const int32_t* prompt, int n, const q38e_sampling* sampling, int max_new_tokens,
                       const int32_t* stop_tokens, int num_stop, int ignore_eos, int* request_id) {
  return guard([&] {
    GenerationConfig g;
    g.sampling = from_c(*sampling);
    g.max_new_tokens = max_new_tokens;
    if (stop_tokens && num_stop > 0) g.stop_tokens.assign(stop_tokens, stop_tokens + num_stop);
    g.ignore_eos = ignore_eos != 0;
    const int id = e->e->submit(std::vector<int32_t>(prompt, prompt + n), g);
    if (request_id) *request_id = id;
  });
}
int q38e_engine_step(q38e_engine* e, int* more) { return guard([&] { *more = e->e->step() ? 1 : 0; }); }
int q38e_engine_run(q38e_engine* e) { return guard([&] { e->e->run(); }); }
int q38e_engine_idle(q38e_engine* e, int* idle) { return guard([&] { *idle = e->e->idle() ? 1 : 0; }); }

int q38e_engine_finished_next(q38e_engine* e, int* request_id, int* num_tokens, int* finish_reason) {
  return guard([&] {
    for (auto& r : e->e->take_finished()) e->done.push_back(std::move(r));
    if (e->done.empty()) {
      *request_id = -1;
      *num_tokens = 0;
      *finish_reason = 0;
      return;
    }
    *request_id = e->done.front().id;
    *num_tokens = int(e->done.front().tokens.size());
    *finish_reason = int(e->done.front().finish);
  });
}
int q38e_engine_finished_take(q38e_engine* e, int32_t* tokens_out, float* logprobs_out, char* error_buf, size_t error_cap,
                              double* times3) {
  return guard([&] {
    QWEN38_CHECK(!e->done.empty(), "no finished request");
    const RequestResult& r = e->done.front();
    for (size_t i = 0; i < r.tokens.size(); ++i) {
      if (tokens_out) tokens_out[i] = r.tokens[i];
      if (logprobs_out) logprobs_out[i] = r.logprobs[i];
    }
    if (error_buf && error_cap) std::snprintf(error_buf, error_cap, "%s", r.error.c_str());
    if (times3) {
      times3[0] = r.submit_s;
      times3[1] = r.first_token_s;
      times3[2] = r.done_s;
    }
    e->done.pop_front();
  });
}
int q38e_engine_stats(q38e_engine* e, q38e_stats* out, int reset) {
  return guard([&] {
    const EngineStats& s = e->e->stats();
    *out = {s.prefill_tokens, s.prefill_s, s.decode_tokens, s.decode_s, s.decode_steps, s.requests_done};
    if (reset) e->e->reset_stats();
  });
}
int q38e_engine_runner(q38e_engine* e, q38e_runner** out) {
  return guard([&] { *out = &e->runner_view; });
}

}  // extern "C"
