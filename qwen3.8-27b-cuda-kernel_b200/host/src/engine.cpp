// Engine: FIFO admission with whole-sequence KV reservation, then per scheduler iteration at most one
// prefill step and one batched decode step. Scheduling rules, stop conditions, error results and the
// statistics follow the reference (src/engine.cpp:19-194); `ragged_prefill` additionally lets the prefill
// step carry chunks of several prompts, `mixed_steps` lets it carry the generating sequences' tokens as well.
#include <algorithm>

#include "qwen38/api.h"

namespace qwen38 {

const char* finish_reason_name(FinishReason r) {
  switch (r) {
    case FinishReason::None: return "none";
    case FinishReason::Stop: return "stop";
    case FinishReason::Length: return "length";
    case FinishReason::Error: return "error";
  }
  return "?";
}

struct Engine::Sequence {
  RequestResult result;
  GenerationConfig config;
  TokenCallback on_token;
  int slot = -1;
  int prefilled = 0;     // prompt tokens already in the cache
  int position = 0;      // next position to be written
  int32_t pending = -1;  // sampled token that the next decode step consumes
  int samples = 0;
  bool generating() const { return prefilled == int(result.prompt.size()); }
};

Engine::Engine(const ModelFile& file, const EngineOptions& options)
    : opt_(options), t0_(std::chrono::steady_clock::now()) {
  runner_ = std::make_unique<ModelRunner>(file, opt_.runner);
  eos_ = file.config().eos_token_ids;
  for (int s = runner_->num_slots() - 1; s >= 0; --s) free_slots_.push_back(s);  // slot 0 is handed out first
}

Engine::~Engine() = default;

double Engine::now() const { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0_).count(); }

int Engine::submit(std::vector<int32_t> prompt, GenerationConfig config, TokenCallback on_token) {
  auto s = std::make_unique<Sequence>();
  const int id = next_id_++;
  s->result.id = id;
  s->result.prompt = std::move(prompt);
  s->result.submit_s = now();
  if (config.sampling.seed == 0) config.sampling.seed = opt_.seed + uint64_t(id) * 0x9E3779B97F4A7C15ull;
  if (config.stop_tokens.empty() && !config.ignore_eos) config.stop_tokens = eos_;
  s->config = std::move(config);
  s->on_token = std::move(on_token);
  if (s->result.prompt.empty()) {
    s->result.finish = FinishReason::Error;
    s->result.error = "empty prompt";
    finished_.push_back(std::move(s->result));
  } else {
    waiting_.push_back(std::move(s));
  }
  return id;
}

bool Engine::idle() const { return waiting_.empty() && active_.empty(); }

void Engine::finish(Sequence& s, FinishReason reason, const std::string& error) {
  s.result.finish = reason;
  s.result.error = error;
  s.result.done_s = now();
  if (s.slot >= 0) {
    runner_->kv().release(s.slot);
    free_slots_.push_back(s.slot);
    s.slot = -1;
  }
  ++stats_.requests_done;
  finished_.push_back(std::move(s.result));
}

void Engine::admit() {
  const int max_ctx = runner_->options().max_context;
  while (!waiting_.empty() && !free_slots_.empty()) {
    Sequence& s = *waiting_.front();
    const int prompt = int(s.result.prompt.size());
    auto reject = [&](const char* why) {
      auto seq = std::move(waiting_.front());
      waiting_.pop_front();
      finish(*seq, FinishReason::Error, why);
    };
    if (prompt >= max_ctx) {
      reject("prompt longer than the context limit");
      continue;
    }
    const int want = int(std::min<int64_t>(int64_t(prompt) + s.config.max_new_tokens, max_ctx));
    const int slot = free_slots_.back();
    if (!runner_->kv().ensure(slot, want)) {  // the whole sequence is reserved up front: no preemption later
      if (active_.empty()) {
        reject("request needs more KV cache than the engine has");
        continue;
      }
      break;  // pages come back when running sequences finish
    }
    free_slots_.pop_back();
    s.slot = slot;
    runner_->reset_slot(slot);
    active_.push_back(std::move(waiting_.front()));
    waiting_.pop_front();
  }
}

// Books one sampled token; true if the sequence finished with it.
bool Engine::deliver(Sequence& s, int32_t token, float logprob) {
  s.result.tokens.push_back(token);
  s.result.logprobs.push_back(logprob);
  if (s.result.first_token_s == 0) s.result.first_token_s = now();
  ++s.samples;
  s.pending = token;
  const auto& stops = s.config.stop_tokens;
  const bool stop = std::find(stops.begin(), stops.end(), token) != stops.end();
  const bool length = int(s.result.tokens.size()) >= s.config.max_new_tokens ||
                      s.position >= runner_->options().max_context;  // position = where `token` would go
  if (s.on_token) s.on_token(s.result.id, token, stop || length);
  if (!stop && !length) return false;
  finish(s, stop ? FinishReason::Stop : FinishReason::Length);
  return true;
}

void Engine::drop_finished() {
  active_.erase(std::remove_if(active_.begin(), active_.end(), [](const auto& p) { return p->slot < 0; }), active_.end());
}

bool Engine::step() {
  admit();
  if (active_.empty()) return !waiting_.empty();
  const int chunk = runner_->options().prefill_chunk;

  // Rows of the decode step: every generating sequence with a sampled token to consume (up to the batch capacity).
  std::vector<DecodeRow> drows;
  std::vector<Sequence*> downers;
  auto collect_decode_rows = [&] {
    drows.clear();
    downers.clear();
    for (auto& sp : active_) {
      Sequence& s = *sp;
      if (!s.generating() || s.pending < 0 || int(drows.size()) == runner_->num_slots()) continue;
      DecodeRow r;
      r.slot = s.slot;
      r.position = s.position;
      r.token = s.pending;
      r.sampling = s.config.sampling;
      r.step = s.samples;
      drows.push_back(r);
      downers.push_back(&s);
    }
  };
  bool prompts_pending = false;
  for (auto& sp : active_) prompts_pending = prompts_pending || !sp->generating();
  // A mixed step carries the decode rows inside the prefill step; it needs room for them and for at least as many
  // prompt tokens again (otherwise the two separate steps serve the prompts better).
  bool mixed = false;
  if (opt_.mixed_steps && prompts_pending) {
    collect_decode_rows();
    mixed = !drows.empty() && 2 * int(drows.size()) <= chunk;
  }

  // 1) one prefill step: the oldest unfinished prompt's next chunk (plus, with ragged_prefill, chunks of
  //    the following prompts while the token budget lasts; plus, in a mixed step, the decode rows)
  {
    std::vector<PrefillRow> rows;
    std::vector<Sequence*> owners;
    int budget = chunk - (mixed ? int(drows.size()) : 0);
    for (auto& sp : active_) {
      Sequence& s = *sp;
      if (s.generating() || budget <= 0) continue;
      if (int(rows.size()) + (mixed ? int(drows.size()) : 0) >= runner_->num_slots()) break;
      const int prompt = int(s.result.prompt.size());
      const int n = std::min(budget, prompt - s.prefilled);
      PrefillRow r;
      r.slot = s.slot;
      r.pos0 = s.prefilled;
      r.tokens = std::span<const int32_t>(s.result.prompt).subspan(size_t(s.prefilled), size_t(n));
      r.sample = s.prefilled + n == prompt ? &s.config.sampling : nullptr;
      r.step = s.samples;
      rows.push_back(r);
      owners.push_back(&s);
      budget -= n;
      if (!opt_.ragged_prefill) break;
    }
    const size_t prompt_rows = rows.size();
    std::vector<int32_t> pending_tokens;  // storage the decode rows' one-token spans point into
    if (mixed && prompt_rows > 0) {
      pending_tokens.reserve(drows.size());
      for (size_t i = 0; i < drows.size(); ++i) {
        pending_tokens.push_back(drows[i].token);
        PrefillRow r;
        r.slot = drows[i].slot;
        r.pos0 = drows[i].position;
        r.tokens = std::span<const int32_t>(pending_tokens.data() + i, 1);
        r.sample = &downers[i]->config.sampling;
        r.step = drows[i].step;
        rows.push_back(r);
        owners.push_back(downers[i]);
      }
    } else {
      mixed = false;
    }
    if (!rows.empty()) {
      const double t = now();
      StepResult res;
      bool step_ok = true;
      try {
        res = runner_->prefill_batch(rows);
      } catch (const DeviceStepError& e) {
        // the step's kernels gave up: nothing of it is delivered; its sequences end with an error result, the
        // engine and the other sequences carry on
        step_ok = false;
        for (Sequence* s : owners) finish(*s, FinishReason::Error, e.what());
      }
      stats_.prefill_s += now() - t;
      size_t sampled = 0;
      for (size_t i = 0; step_ok && i < rows.size(); ++i) {
        Sequence& s = *owners[i];
        if (i < prompt_rows) {
          const int n = int(rows[i].tokens.size());
          stats_.prefill_tokens += n;
          s.prefilled += n;
          s.position = s.prefilled;
        } else {
          s.position += 1;  // the consumed token now sits in the cache
        }
        if (rows[i].sample) {
          deliver(s, res.tokens[sampled], res.logprobs[sampled]);
          ++sampled;
        }
      }
      if (step_ok && mixed) {
        stats_.decode_tokens += int64_t(drows.size());
        ++stats_.decode_steps;
      }
      drop_finished();
    }
  }
  if (mixed) return true;

  // 2) one decode step over every generating sequence (up to the batch capacity)
  collect_decode_rows();
  const std::vector<DecodeRow>& rows = drows;
  const std::vector<Sequence*>& owners = downers;
  if (!rows.empty()) {
    const double t = now();
    StepResult res;
    bool step_ok = true;
    try {
      res = runner_->decode(rows);
    } catch (const DeviceStepError& e) {
      step_ok = false;
      for (Sequence* s : owners) finish(*s, FinishReason::Error, e.what());
    }
    stats_.decode_s += now() - t;
    if (step_ok) {
      stats_.decode_tokens += int64_t(rows.size());
      ++stats_.decode_steps;
      for (size_t i = 0; i < owners.size(); ++i) {
        owners[i]->position += 1;  // the consumed token now sits in the cache
        deliver(*owners[i], res.tokens[i], res.logprobs[i]);
      }
    }
    drop_finished();
  }
  return true;
}

void Engine::run() {
  while (!idle()) step();
}

std::vector<RequestResult> Engine::take_finished() {
  std::vector<RequestResult> out;
  out.swap(finished_);
  return out;
}

}  // namespace qwen38
