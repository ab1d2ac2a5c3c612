// SLO-aware continuous batcher.
//
// `decide` is a pure function of the request, the load and the latency estimator:
//   Reject{PromptTooLong}  predicted prefill time (prefill_per_token_us x prompt) exceeds the TTFT SLO
//   Delay{until}           the in-flight set is full, the predicted TPOT at one more sequence
//                          (base x batch^exponent) exceeds the TPOT SLO, or the KV cache has no room;
//                          retry after one predicted step
//   Admit                  otherwise
// Admitted requests prefill in chunks (ContinuousChunked policy) or at once, then join the decode
// batch. Every step the driver asks for `next_step_batch`, runs it, reports tokens with
// `accept_token`, and finished requests are retired (KV pages released).
//
// Same decision rule and life cycle as the reference (crates/skein_runtime/src/batcher/
// admission.rs:9-100, mod.rs:47-240, chunking.rs:8-41, queue.rs:10-49, retire.rs:11-23), with KV
// reservation folded into admission instead of being done by the driver afterwards.
#pragma once
#include "kv.hpp"
#include <algorithm>
#include <cmath>
#include <optional>

namespace skein {

struct LatencyEstimator {
  double per_token_decode_us_at_b1 = 8000.0, batch_scaling_exponent = 0.7, prefill_per_token_us = 25.0;
  double predict_prefill_ms(uint32_t prompt_tokens) const { return prefill_per_token_us * prompt_tokens / 1000.0; }
  // time of one decode step at a given batch = time per output token of every sequence in it:
  // base x batch^exponent
  double predict_step_ms(uint32_t batch) const { return per_token_decode_us_at_b1 * std::pow((double)std::max(1u, batch), batch_scaling_exponent) / 1000.0; }
  double predict_tpot_ms(uint32_t concurrent) const { return predict_step_ms(concurrent); }
};

struct SloTargets { double ttft_ms = 500, tpot_ms = 50; };

enum class Decision { Admit, Delay, Reject };
struct AdmissionDecision {
  Decision kind = Decision::Admit;
  uint64_t until_ms = 0;            // Delay
  std::string reason;               // Reject / Delay
};

struct IncomingRequest {
  uint64_t id = 0;
  std::vector<int32_t> prompt;
  uint32_t max_new_tokens = 32;
  uint64_t arrival_ms = 0;
};

enum class Phase { Prefill, Decode, Finished };

struct InflightRequest {
  IncomingRequest req;
  Phase phase = Phase::Prefill;
  uint32_t prefilled = 0;           // prompt tokens whose KV is computed (starts at the prefix-cache hit)
  std::vector<int32_t> generated;
  uint64_t admitted_ms = 0, first_token_ms = 0, last_token_ms = 0;
  uint32_t prefix_hit_tokens = 0;
};

struct PrefillChunk { uint64_t id; uint32_t start, end; bool last; };
struct StepBatch {
  std::vector<PrefillChunk> prefill;
  std::vector<uint64_t> decode;
  bool empty() const { return prefill.empty() && decode.empty(); }
};

struct AcceptOutcome { bool finished = false; uint32_t generated = 0; };

class ContinuousBatcher {
 public:
  ContinuousBatcher(uint32_t max_batch, uint32_t chunk_tokens, SloTargets slo, LatencyEstimator est, KvBlockManager* kv,
                    uint32_t max_prefill_tokens_per_step = 8192, uint32_t interleave_prefill_tokens = 0)
      : max_batch_(max_batch), chunk_tokens_(chunk_tokens), slo_(slo), est_(est), kv_(kv), max_prefill_tokens_(max_prefill_tokens_per_step),
        interleave_tokens_(interleave_prefill_tokens) {}

  AdmissionDecision decide(const IncomingRequest& r, uint64_t now_ms) const {
    AdmissionDecision d;
    if (est_.predict_prefill_ms((uint32_t)r.prompt.size()) > slo_.ttft_ms) {
      d.kind = Decision::Reject;
      d.reason = "prompt_too_long";
      return d;
    }
    const uint32_t n = (uint32_t)inflight_.size();
    const uint64_t retry = now_ms + (uint64_t)std::ceil(est_.predict_step_ms(std::max(1u, n)));
    if (n >= max_batch_) { d.kind = Decision::Delay; d.until_ms = retry; d.reason = "batch_full"; return d; }
    if (est_.predict_step_ms(n + 1) > slo_.tpot_ms) { d.kind = Decision::Delay; d.until_ms = retry; d.reason = "tpot_slo"; return d; }
    if (kv_ && !kv_->can_admit(r.prompt, r.max_new_tokens)) { d.kind = Decision::Delay; d.until_ms = retry; d.reason = "kv_full"; return d; }
    return d;
  }

  // Applies `decide`: Admit -> in flight (KV pages reserved), Delay -> queued, Reject -> dropped.
  AdmissionDecision submit(const IncomingRequest& r, uint64_t now_ms) {
    AdmissionDecision d = decide(r, now_ms);
    if (d.kind == Decision::Admit) start(r, now_ms);
    else if (d.kind == Decision::Delay) queue_.push_back({r, d.until_ms});
    else ++rejected_;
    return d;
  }

  // Moves queued requests whose retry time has come into flight, in FIFO order, while they are admissible.
  void promote_ready(uint64_t now_ms) {
    while (!queue_.empty() && queue_.front().ready_at_ms <= now_ms) {
      AdmissionDecision d = decide(queue_.front().req, now_ms);
      if (d.kind == Decision::Admit) { start(queue_.front().req, now_ms); queue_.pop_front(); }
      else if (d.kind == Decision::Reject) { ++rejected_; queue_.pop_front(); }
      else { queue_.front().ready_at_ms = d.until_ms; break; }
    }
  }

  StepBatch next_step_batch() {
    StepBatch b;
    uint32_t budget = max_prefill_tokens_;
    for (auto& kv : inflight_) {
      InflightRequest& r = kv.second;
      if (r.phase == Phase::Decode) b.decode.push_back(kv.first);
    }
    // while sequences are decoding, a step carries only a slice of the waiting prompts, so that a long
    // prompt delays the decoding sequences' next token by one slice and not by its whole prefill
    if (interleave_tokens_ > 0 && !b.decode.empty()) budget = std::min(budget, interleave_tokens_);
    for (auto& kv : inflight_) {
      InflightRequest& r = kv.second;
      if (r.phase != Phase::Prefill || budget == 0) continue;
      const uint32_t total = (uint32_t)r.req.prompt.size();
      uint32_t len = total - r.prefilled;
      if (chunk_tokens_ > 0) len = std::min(len, chunk_tokens_);
      len = std::min(len, budget);
      if (len == 0) continue;
      b.prefill.push_back({kv.first, r.prefilled, r.prefilled + len, r.prefilled + len == total});
      budget -= len;
    }
    return b;
  }

  // Called after a prefill chunk ran; the last chunk's sampled token arrives through accept_token.
  void prefill_advanced(uint64_t id, uint32_t new_end) {
    auto it = inflight_.find(id);
    if (it == inflight_.end()) return;
    it->second.prefilled = new_end;
    // only now may other requests share these pages through the prefix cache
    if (kv_ && kv_->table(id)) kv_->mark_computed(id, it->second.req.prompt, new_end);
  }

  std::optional<AcceptOutcome> accept_token(uint64_t id, int32_t token, uint64_t now_ms, int32_t eos_token = -1) {
    auto it = inflight_.find(id);
    if (it == inflight_.end()) return std::nullopt;
    InflightRequest& r = it->second;
    if (r.phase == Phase::Prefill) {
      r.phase = Phase::Decode; r.first_token_ms = now_ms; r.prefilled = (uint32_t)r.req.prompt.size();
      if (kv_ && kv_->table(id)) kv_->mark_computed(id, r.req.prompt, r.prefilled);
    }
    r.generated.push_back(token);
    r.last_token_ms = now_ms;
    AcceptOutcome o;
    o.generated = (uint32_t)r.generated.size();
    o.finished = o.generated >= r.req.max_new_tokens || (eos_token >= 0 && token == eos_token);
    if (o.finished) r.phase = Phase::Finished;
    else if (kv_) kv_->advance(id, 1);   // room for the token that the next step writes
    return o;
  }

  // `failed`: the request is dropped after a step that did not complete; its pages leave the prefix cache.
  // The host inputs of a decode step, written straight into the step's staging arrays (pinned memory that one
  // host-to-device copy then moves): row i feeds request ids[i] its last token at its position; id 0 and the rows
  // from ids.size() to `rows` are padding (position -1, length 0). Block-table rows are `max_blocks` wide.
  void fill_decode_inputs(const std::vector<uint64_t>& ids, int32_t* tok, int32_t* pos, int32_t* lens, int32_t* block_table,
                          size_t max_blocks, size_t rows) const {
    if (ids.size() > rows) throw RuntimeError("decode batch is larger than its staging buffer");
    for (size_t i = 0; i < ids.size(); ++i) {
      if (ids[i] == 0) { tok[i] = 0; pos[i] = -1; lens[i] = 0; continue; }   // a padding row inside the batch
      const InflightRequest* r = get(ids[i]);
      if (!r || r->generated.empty()) throw RuntimeError("request " + std::to_string(ids[i]) + " is not decoding");
      const int32_t p = (int32_t)(r->req.prompt.size() + r->generated.size()) - 1;
      tok[i] = r->generated.back();
      pos[i] = p;
      lens[i] = p + 1;
      if (kv_) {
        const PageTable* t = kv_->table(ids[i]);
        if (!t || t->pages.size() > max_blocks) throw RuntimeError("request " + std::to_string(ids[i]) + ": page table does not fit the block table");
        std::copy(t->pages.begin(), t->pages.end(), block_table + i * max_blocks);
      }
    }
    for (size_t i = ids.size(); i < rows; ++i) { tok[i] = 0; pos[i] = -1; lens[i] = 0; }
  }
  // accept_token for a whole decode batch; out[i] = (finished, tokens generated so far) of ids[i].
  std::vector<AcceptOutcome> accept_tokens(const std::vector<uint64_t>& ids, const int32_t* tokens, uint64_t now_ms, int32_t eos_token = -1) {
    std::vector<AcceptOutcome> out;
    out.reserve(ids.size());
    for (size_t i = 0; i < ids.size(); ++i) {
      if (ids[i] == 0) { out.push_back(AcceptOutcome{}); continue; }
      auto o = accept_token(ids[i], tokens[i], now_ms, eos_token);
      out.push_back(o ? *o : AcceptOutcome{});
    }
    return out;
  }

  void retire(uint64_t id, bool failed = false) {
    auto it = inflight_.find(id);
    if (it == inflight_.end()) throw RuntimeError("retire: unknown request " + std::to_string(id));
    if (kv_ && kv_->table(id)) kv_->release(id, failed);
    inflight_.erase(it);
    ++retired_;
  }
  // Failure path: drop everything in flight (a step threw); queued requests stay queued.
  std::vector<uint64_t> retire_all() {
    std::vector<uint64_t> ids;
    for (auto& kv : inflight_) ids.push_back(kv.first);
    for (uint64_t id : ids) retire(id, true);
    return ids;
  }

  const InflightRequest* get(uint64_t id) const { auto it = inflight_.find(id); return it == inflight_.end() ? nullptr : &it->second; }
  std::vector<int32_t> current_sequence(uint64_t id) const {
    std::vector<int32_t> s;
    if (auto* r = get(id)) { s = r->req.prompt; s.insert(s.end(), r->generated.begin(), r->generated.end()); }
    return s;
  }
  size_t inflight_len() const { return inflight_.size(); }
  size_t queued_len() const { return queue_.size(); }
  uint64_t rejected() const { return rejected_; }
  uint64_t retired() const { return retired_; }
  uint32_t max_batch() const { return max_batch_; }
  std::vector<uint64_t> inflight_ids() const { std::vector<uint64_t> v; for (auto& kv : inflight_) v.push_back(kv.first); return v; }

 private:
  struct Queued { IncomingRequest req; uint64_t ready_at_ms; };
  uint32_t max_batch_, chunk_tokens_;
  SloTargets slo_;
  LatencyEstimator est_;
  KvBlockManager* kv_;
  uint32_t max_prefill_tokens_, interleave_tokens_;
  std::map<uint64_t, InflightRequest> inflight_;
  std::deque<Queued> queue_;
  uint64_t rejected_ = 0, retired_ = 0;

  void start(const IncomingRequest& r, uint64_t now_ms) {
    InflightRequest f;
    f.req = r;
    f.admitted_ms = now_ms;
    if (kv_) {
      PageTable pt = kv_->admit(r.id, r.prompt);
      f.prefix_hit_tokens = pt.prefix_hit_tokens;
      f.prefilled = pt.prefix_hit_tokens;
    }
    inflight_[r.id] = std::move(f);
  }
};

}  // namespace skein
