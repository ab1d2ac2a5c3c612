// Small host-side runtime pieces: parity math, workload drift monitor, speculative-decoding
// acceptance, CPU reference collectives, and metric ring buffers with Prometheus text output.
#pragma once
#include "kv.hpp"
#include <algorithm>
#include <atomic>
#include <cmath>
#include <functional>
#include <mutex>
#include <sstream>

namespace skein {

// ---- parity math (crates/skein_parity/src/comparison.rs:16,43,72) ----------------------------------------
inline double mse(const std::vector<float>& a, const std::vector<float>& b) {
  if (a.size() != b.size()) throw RuntimeError("mse: length mismatch");
  if (a.empty()) return 0;
  double s = 0;
  for (size_t i = 0; i < a.size(); ++i) { const double d = (double)a[i] - (double)b[i]; s += d * d; }
  return s / (double)a.size();
}
inline std::vector<double> log_softmax(const std::vector<float>& x) {
  double mx = -INFINITY;
  for (float v : x) mx = std::max(mx, (double)v);
  double s = 0;
  for (float v : x) s += std::exp((double)v - mx);
  const double lse = mx + std::log(s);
  std::vector<double> out(x.size());
  for (size_t i = 0; i < x.size(); ++i) out[i] = (double)x[i] - lse;
  return out;
}
// KL(softmax(reference) || softmax(candidate)); stable for logits of magnitude 1e4.
inline double kl_divergence(const std::vector<float>& reference_logits, const std::vector<float>& candidate_logits) {
  if (reference_logits.size() != candidate_logits.size()) throw RuntimeError("kl_divergence: length mismatch");
  const auto lp = log_softmax(reference_logits), lq = log_softmax(candidate_logits);
  double kl = 0;
  for (size_t i = 0; i < lp.size(); ++i) { const double p = std::exp(lp[i]); if (p > 0) kl += p * (lp[i] - lq[i]); }
  return std::max(0.0, kl);
}

// ---- workload drift monitor (crates/skein_runtime/src/drift_monitor.rs:22-108) -----------------------------
class WorkloadProfile {
 public:
  static constexpr uint32_t EDGES[9] = {16, 32, 64, 128, 256, 512, 1024, 2048, 4096};
  static WorkloadProfile from_lengths(const std::vector<uint32_t>& lengths) {
    WorkloadProfile p;
    p.b_.assign(10, 1.0);  // Laplace smoothing
    for (uint32_t l : lengths) {
      size_t k = 9;
      for (size_t i = 0; i < 9; ++i) if (l <= EDGES[i]) { k = i; break; }
      p.b_[k] += 1.0;
    }
    double tot = 0;
    for (double v : p.b_) tot += v;
    for (double& v : p.b_) v /= tot;
    return p;
  }
  double kl_to(const WorkloadProfile& o) const {
    double s = 0;
    for (size_t i = 0; i < b_.size(); ++i) if (b_[i] > 0) s += b_[i] * std::log(b_[i] / o.b_[i]);
    return s;
  }
  const std::vector<double>& buckets() const { return b_; }

 private:
  std::vector<double> b_;
};
struct DriftAssessment { double kl; bool drifted; size_t samples; };
class DriftMonitor {
 public:
  static constexpr size_t MIN_SAMPLES = 32;
  DriftMonitor(WorkloadProfile baseline, double threshold_kl) : base_(std::move(baseline)), thr_(threshold_kl) {}
  double threshold() const { return thr_; }
  DriftAssessment assess(const std::vector<uint32_t>& lengths) const {
    const double kl = WorkloadProfile::from_lengths(lengths).kl_to(base_);
    return {kl, lengths.size() >= MIN_SAMPLES && kl > thr_, lengths.size()};
  }

 private:
  WorkloadProfile base_;
  double thr_;
};

// ---- speculative decoding acceptance (crates/skein_runtime/src/speculative.rs:55-184) -------------------------
struct SpecOutcome { std::vector<int32_t> accepted; int32_t correction = 0; };

inline std::vector<float> normalize_dist(const std::vector<float>& p) {
  double s = 0;
  for (float v : p) s += v;
  if (s <= 0) return p;
  std::vector<float> o(p.size());
  for (size_t i = 0; i < p.size(); ++i) o[i] = (float)(p[i] / s);
  return o;
}
inline std::vector<float> residual_distribution(const std::vector<float>& p, const std::vector<float>& q) {
  std::vector<float> r(p.size());
  double s = 0;
  for (size_t i = 0; i < p.size(); ++i) { r[i] = std::max(0.0f, p[i] - q[i]); s += r[i]; }
  if (s <= 0) return normalize_dist(p);
  for (float& v : r) v = (float)(v / s);
  return r;
}
inline int32_t sample_from(const std::vector<float>& dist, float u) {
  double run = 0;
  for (size_t i = 0; i < dist.size(); ++i) { run += dist[i]; if (u < run) return (int32_t)i; }
  int32_t best = 0;
  for (size_t i = 1; i < dist.size(); ++i) if (dist[i] > dist[best]) best = (int32_t)i;
  return best;
}
// Leviathan et al. accept/reject: token x_i drawn from draft q_i is kept with probability min(1, p_i(x)/q_i(x));
// the first rejection resamples from normalise(max(0, p - q)); if all k are kept a bonus token comes from p_{k}.
// uniforms needs k + 1 values (the last one draws the correction / bonus token).
inline SpecOutcome speculative_verify(const std::vector<int32_t>& draft_tokens, const std::vector<std::vector<float>>& draft_probs,
                                      const std::vector<std::vector<float>>& target_probs, const std::vector<float>& uniforms) {
  const size_t k = draft_tokens.size();
  if (draft_probs.size() != k || target_probs.size() != k + 1) throw RuntimeError("speculative_verify: shape mismatch");
  if (uniforms.size() < k + 1) throw RuntimeError("speculative_verify: need k + 1 uniforms");
  SpecOutcome out;
  for (size_t i = 0; i < k; ++i) {
    const size_t x = (size_t)draft_tokens[i];
    const auto &p = target_probs[i], &q = draft_probs[i];
    if (draft_tokens[i] < 0 || x >= p.size() || x >= q.size()) throw RuntimeError("speculative_verify: token out of range");
    const float ratio = q[x] > 0 ? std::min(1.0f, p[x] / q[x]) : 1.0f;
    if (uniforms[i] <= ratio) { out.accepted.push_back(draft_tokens[i]); continue; }
    out.correction = sample_from(residual_distribution(p, q), uniforms[k]);
    return out;
  }
  out.correction = sample_from(normalize_dist(target_probs[k]), uniforms[k]);
  return out;
}

// ---- CPU reference collectives (crates/skein_runtime/src/collectives/mod.rs:54-127) ---------------------------
// bufs[r] is rank r's buffer; results are written the way each rank would see them.
inline void cpu_all_reduce_sum(std::vector<std::vector<float>>& bufs) {
  if (bufs.empty()) return;
  std::vector<float> s(bufs[0].size(), 0.f);
  for (auto& b : bufs) { if (b.size() != s.size()) throw RuntimeError("all_reduce: length mismatch"); for (size_t i = 0; i < s.size(); ++i) s[i] += b[i]; }
  for (auto& b : bufs) b = s;
}
inline void cpu_all_gather(std::vector<std::vector<float>>& bufs) {
  std::vector<float> cat;
  for (auto& b : bufs) cat.insert(cat.end(), b.begin(), b.end());
  for (auto& b : bufs) b = cat;
}
inline void cpu_reduce_scatter(std::vector<std::vector<float>>& bufs) {
  const size_t n = bufs.size();
  if (n == 0) return;
  const size_t len = bufs[0].size();
  if (len % n) throw RuntimeError("reduce_scatter: length not divisible by ranks");
  std::vector<float> s(len, 0.f);
  for (auto& b : bufs) for (size_t i = 0; i < len; ++i) s[i] += b[i];
  const size_t per = len / n;
  for (size_t r = 0; r < n; ++r) bufs[r].assign(s.begin() + r * per, s.begin() + (r + 1) * per);
}
inline void cpu_all_to_all(std::vector<std::vector<float>>& bufs) {
  const size_t n = bufs.size();
  if (n == 0) return;
  const size_t len = bufs[0].size();
  if (len % n) throw RuntimeError("all_to_all: length not divisible by ranks");
  const size_t per = len / n;
  std::vector<std::vector<float>> out(n, std::vector<float>(len));
  for (size_t src = 0; src < n; ++src)
    for (size_t dst = 0; dst < n; ++dst)
      std::copy(bufs[src].begin() + dst * per, bufs[src].begin() + (dst + 1) * per, out[dst].begin() + src * per);
  bufs = out;
}
inline void cpu_broadcast(std::vector<std::vector<float>>& bufs, size_t root) {
  for (size_t r = 0; r < bufs.size(); ++r) if (r != root) bufs[r] = bufs.at(root);
}

// ---- metrics (crates/skein_runtime/src/observability/prometheus.rs:21-107, metrics.rs:6-18) ---------------------
struct StepMetrics { uint64_t step = 0; uint32_t batch_size = 0; double compute_us = 0, comm_us = 0; uint32_t kv_pages_in_use = 0; };
struct RequestMetrics { uint64_t id = 0; std::string status; double ttft_ms = 0, tpot_ms = 0; uint32_t prefix_hit_tokens = 0, output_tokens = 0; };

class Histogram {
 public:
  explicit Histogram(std::vector<double> bounds) : bounds_(std::move(bounds)), counts_(bounds_.size() + 1, 0) {}
  void observe(double v) {
    size_t i = 0;
    while (i < bounds_.size() && v > bounds_[i]) ++i;
    ++counts_[i]; sum_ += v; ++n_; samples_.push_back(v);
    if (samples_.size() > 65536) samples_.erase(samples_.begin(), samples_.begin() + 32768);
  }
  double quantile(double q) const {
    if (samples_.empty()) return 0;
    std::vector<double> s = samples_;
    std::sort(s.begin(), s.end());
    return s[std::min(s.size() - 1, (size_t)(q * (double)s.size()))];
  }
  void render(std::ostringstream& o, const std::string& name, const std::string& help) const {
    o << "# HELP " << name << " " << help << "\n# TYPE " << name << " histogram\n";
    uint64_t cum = 0;
    for (size_t i = 0; i < bounds_.size(); ++i) { cum += counts_[i]; o << name << "_bucket{le=\"" << Json_fmt(bounds_[i]) << "\"} " << cum << "\n"; }
    o << name << "_bucket{le=\"+Inf\"} " << n_ << "\n" << name << "_sum " << Json_fmt(sum_) << "\n" << name << "_count " << n_ << "\n";
  }
  uint64_t count() const { return n_; }

 private:
  static std::string Json_fmt(double v) { std::ostringstream s; s << v; return s.str(); }
  std::vector<double> bounds_;
  std::vector<uint64_t> counts_;
  std::vector<double> samples_;
  double sum_ = 0;
  uint64_t n_ = 0;
};

class MetricsRegistry {
 public:
  explicit MetricsRegistry(size_t capacity = 100000)
      // bucket bounds as in the reference's instruments (the decode-latency histogram gains 1 and 2 ms
      // buckets: a B200 step is far below the reference's smallest 5 ms bound)
      : cap_(capacity), batch_hist_({1, 2, 4, 8, 16, 32, 64, 128}), ttft_hist_({25, 50, 100, 250, 500, 1000, 2000}),
        tpot_hist_({1, 2, 5, 10, 25, 50, 100, 250, 500}) {}
  void record_step(const StepMetrics& m) {
    std::lock_guard<std::mutex> g(mu_);
    ++steps_; compute_us_ += m.compute_us; comm_us_ += m.comm_us; kv_pages_ = m.kv_pages_in_use;
    batch_hist_.observe(m.batch_size);
    steps_buf_.push_back(m);
    if (steps_buf_.size() > cap_) steps_buf_.pop_front();
  }
  void record_request(const RequestMetrics& m) {
    std::lock_guard<std::mutex> g(mu_);
    ++requests_[m.status];
    if (m.status == "ok") { ttft_hist_.observe(m.ttft_ms); if (m.output_tokens > 1) tpot_hist_.observe(m.tpot_ms); }
    prefix_hits_ += m.prefix_hit_tokens;
    req_buf_.push_back(m);
    if (req_buf_.size() > cap_) req_buf_.pop_front();
  }
  void count(const std::string& name, uint64_t n = 1) { std::lock_guard<std::mutex> g(mu_); extra_[name] += n; }
  void set_gauge(const std::string& name, double v) { std::lock_guard<std::mutex> g(mu_); gauges_[name] = v; }
  size_t steps_buffered() const { return steps_buf_.size(); }
  size_t requests_buffered() const { return req_buf_.size(); }
  double ttft_p50() const { return ttft_hist_.quantile(0.5); }
  double tpot_p99() const { return tpot_hist_.quantile(0.99); }
  std::string render() const {
    std::lock_guard<std::mutex> g(mu_);
    std::ostringstream o;
    o << "# HELP skein_steps_total Decode/prefill steps executed\n# TYPE skein_steps_total counter\nskein_steps_total " << steps_ << "\n";
    o << "# HELP skein_step_compute_us_total Device time spent in compute\n# TYPE skein_step_compute_us_total counter\nskein_step_compute_us_total " << compute_us_ << "\n";
    o << "# HELP skein_step_comm_us_total Device time spent in exposed communication\n# TYPE skein_step_comm_us_total counter\nskein_step_comm_us_total " << comm_us_ << "\n";
    o << "# HELP skein_kv_pages_in_use KV pages referenced by live requests\n# TYPE skein_kv_pages_in_use gauge\nskein_kv_pages_in_use " << kv_pages_ << "\n";
    batch_hist_.render(o, "skein_batch_size_histogram", "Sequences per step");
    o << "# HELP skein_requests_total Requests by final status\n# TYPE skein_requests_total counter\n";
    for (auto& kv : requests_) o << "skein_requests_total{status=\"" << kv.first << "\"} " << kv.second << "\n";
    ttft_hist_.render(o, "skein_ttft_ms_histogram", "Time to first token (ms)");
    tpot_hist_.render(o, "skein_tpot_ms_histogram", "Time per output token (ms)");
    o << "# HELP skein_prefix_cache_hit_tokens_total Prompt tokens served from the prefix cache\n# TYPE skein_prefix_cache_hit_tokens_total counter\nskein_prefix_cache_hit_tokens_total " << prefix_hits_ << "\n";
    for (auto& kv : extra_) o << "# TYPE " << kv.first << " counter\n" << kv.first << " " << kv.second << "\n";
    for (auto& kv : gauges_) o << "# TYPE " << kv.first << " gauge\n" << kv.first << " " << kv.second << "\n";
    return o.str();
  }

 private:
  size_t cap_;
  mutable std::mutex mu_;
  uint64_t steps_ = 0, prefix_hits_ = 0;
  double compute_us_ = 0, comm_us_ = 0;
  uint32_t kv_pages_ = 0;
  Histogram batch_hist_, ttft_hist_, tpot_hist_;
  std::map<std::string, uint64_t> requests_, extra_;
  std::map<std::string, double> gauges_;
  std::deque<StepMetrics> steps_buf_;
  std::deque<RequestMetrics> req_buf_;
};

}  // namespace skein
