// Cluster description (TOML with [[node]] / [[link]] tables), its validation, the device graph
// with bottleneck-bandwidth shortest paths, the TP x PP x EP device grid, the workload trace (JSONL
// with an SLO header line) and synthetic trace generators.
//
// Same file formats and rejection cases as the reference (crates/skein_ir/src/cluster.rs:19-109,
// workload.rs:21-99; crates/skein_cost/src/topology.rs:95,170, cluster.rs:100-186). An NVSwitch
// domain is written as all-pairs links of kind nvlink_gen5, which makes every pair's path one hop.
#pragma once
#include "ir.hpp"
#include "plan.hpp"
#include "toml_lite.hpp"
#include <algorithm>
#include <cmath>
#include <limits>
#include <queue>
#include <random>
#include <set>
#include <sstream>

namespace skein {

struct ClusterError : std::runtime_error { using std::runtime_error::runtime_error; };
struct WorkloadError : std::runtime_error { using std::runtime_error::runtime_error; };
struct CostError : std::runtime_error { using std::runtime_error::runtime_error; };

inline bool link_kind_known(const std::string& k) {
  static const char* kinds[] = {"nvlink_gen4", "nvlink_gen5", "pcie5", "infiniband400g", "roce100g", "tcp10g"};
  for (auto* x : kinds) if (k == x) return true;
  return false;
}

struct Node {
  std::string id, device_kind;
  std::vector<std::string> devices;
  uint32_t device_memory_gb = 0;
};
struct Link {
  std::string a, b, kind;
  double bandwidth_gbps = 0, latency_us = 0;
};

struct ClusterSpec {
  uint32_t num_devices = 0;
  std::vector<Node> nodes;
  std::vector<Link> links;

  static ClusterSpec from_json(const Json& j) {
    ClusterSpec s;
    if (!j.has("num_devices")) throw ClusterError("cluster: missing `num_devices`");
    s.num_devices = (uint32_t)j.at("num_devices").as_int();
    if (const Json* ns = j.find("node")) {
      for (auto& n : ns->items()) {
        Node x;
        x.id = n.at("id").as_string();
        x.device_kind = n.at("device_kind").as_string();
        x.device_memory_gb = (uint32_t)n.at("device_memory_gb").as_int();
        for (auto& d : n.at("devices").items()) x.devices.push_back(d.as_string());
        s.nodes.push_back(x);
      }
    }
    if (const Json* ls = j.find("link")) {
      for (auto& l : ls->items()) {
        Link x;
        const auto& ep = l.at("endpoints").items();
        if (ep.size() != 2) throw ClusterError("cluster: a link needs exactly two endpoints");
        x.a = ep[0].as_string(); x.b = ep[1].as_string();
        x.kind = l.at("kind").as_string();
        if (!link_kind_known(x.kind)) throw ClusterError("cluster: unknown link kind `" + x.kind + "`");
        x.bandwidth_gbps = l.at("bandwidth_gbps").as_double();
        x.latency_us = l.at("latency_us").as_double();
        s.links.push_back(x);
      }
    }
    s.validate();
    return s;
  }
  static ClusterSpec from_toml_str(const std::string& text) {
    try {
      return from_json(parse_toml(text));
    } catch (const TomlError& e) {
      throw ClusterError(std::string("cluster TOML: ") + e.what());
    } catch (const JsonError& e) {
      throw ClusterError(std::string("cluster TOML: ") + e.what());
    }
  }
  void validate() const {
    std::set<std::string> node_ids, dev_ids;
    uint32_t total = 0;
    for (auto& n : nodes) {
      if (!node_ids.insert(n.id).second) throw ClusterError("duplicate node id `" + n.id + "`");
      for (auto& d : n.devices) {
        if (!dev_ids.insert(d).second) throw ClusterError("duplicate device id `" + d + "`");
        ++total;
      }
    }
    if (total != num_devices)
      throw ClusterError("num_devices = " + std::to_string(num_devices) + " but the nodes list " + std::to_string(total) + " devices");
    for (auto& l : links) {
      if (l.a == l.b) throw ClusterError("link from `" + l.a + "` to itself");
      if (!dev_ids.count(l.a)) throw ClusterError("link names unknown device `" + l.a + "`");
      if (!dev_ids.count(l.b)) throw ClusterError("link names unknown device `" + l.b + "`");
    }
  }
  std::vector<std::string> all_devices() const {
    std::vector<std::string> v;
    for (auto& n : nodes) for (auto& d : n.devices) v.push_back(d);
    return v;
  }
  Json to_json() const {
    Json ns = Json::array(), ls = Json::array();
    for (auto& n : nodes) {
      Json ds = Json::array();
      for (auto& d : n.devices) ds.push(d);
      ns.push(Json::object().set("id", n.id).set("devices", ds).set("device_kind", n.device_kind).set("device_memory_gb", n.device_memory_gb));
    }
    for (auto& l : links) {
      Json ep = Json::array(); ep.push(l.a); ep.push(l.b);
      ls.push(Json::object().set("endpoints", ep).set("kind", l.kind).set("bandwidth_gbps", l.bandwidth_gbps).set("latency_us", l.latency_us));
    }
    return Json::object().set("num_devices", num_devices).set("node", ns).set("link", ls);
  }
};

// ---- device graph ----------------------------------------------------------------------------------
struct PathInfo {
  double min_bandwidth_gbps = std::numeric_limits<double>::infinity();
  double total_latency_us = 0;
  int hops = 0;
};

class Cluster {
 public:
  explicit Cluster(const ClusterSpec& spec) : spec_(spec) {
    for (auto& n : spec.nodes)
      for (auto& d : n.devices) { index_[d] = (int)names_.size(); names_.push_back(d); kinds_.push_back(n.device_kind); mem_gb_.push_back(n.device_memory_gb); }
    adj_.assign(names_.size(), {});
    for (auto& l : spec.links) {
      int a = index_.at(l.a), b = index_.at(l.b);
      adj_[a].push_back({b, l.bandwidth_gbps, l.latency_us});
      adj_[b].push_back({a, l.bandwidth_gbps, l.latency_us});
    }
  }
  size_t num_devices() const { return names_.size(); }
  const std::string& device_kind(size_t d) const { check(d); return kinds_[d]; }
  uint64_t device_memory_bytes(size_t d) const { check(d); return (uint64_t)mem_gb_[d] * 1000000000ull; }
  const ClusterSpec& spec() const { return spec_; }

  // Minimum-latency path (Dijkstra); its bandwidth is the slowest link on it.
  PathInfo pair_path(size_t a, size_t b) const {
    check(a); check(b);
    if (a == b) return PathInfo{std::numeric_limits<double>::infinity(), 0, 0};
    const size_t n = names_.size();
    std::vector<double> dist(n, std::numeric_limits<double>::infinity()), bw(n, std::numeric_limits<double>::infinity());
    std::vector<int> hops(n, 0);
    using Q = std::pair<double, size_t>;
    std::priority_queue<Q, std::vector<Q>, std::greater<Q>> pq;
    dist[a] = 0;
    pq.push({0, a});
    while (!pq.empty()) {
      auto [d, u] = pq.top();
      pq.pop();
      if (d > dist[u]) continue;
      for (auto& e : adj_[u]) {
        double nd = d + e.lat;
        double nbw = std::min(bw[u], e.bw);
        if (nd < dist[e.to] || (nd == dist[e.to] && nbw > bw[e.to])) {
          dist[e.to] = nd; bw[e.to] = nbw; hops[e.to] = hops[u] + 1;
          pq.push({nd, (size_t)e.to});
        }
      }
    }
    if (!std::isfinite(dist[b])) throw CostError("no path between devices " + names_[a] + " and " + names_[b]);
    return PathInfo{bw[b], dist[b], hops[b]};
  }
  // The critical pair of a collective: lowest bandwidth, then highest latency.
  PathInfo collective_path(const std::vector<size_t>& parts) const {
    if (parts.size() < 2) throw CostError("a collective needs at least two participants");
    PathInfo worst;
    bool first = true;
    for (size_t i = 0; i < parts.size(); ++i)
      for (size_t j = i + 1; j < parts.size(); ++j) {
        PathInfo p = pair_path(parts[i], parts[j]);
        if (first || p.min_bandwidth_gbps < worst.min_bandwidth_gbps ||
            (p.min_bandwidth_gbps == worst.min_bandwidth_gbps && p.total_latency_us > worst.total_latency_us)) {
          worst = p; first = false;
        }
      }
    return worst;
  }

 private:
  struct Edge { int to; double bw, lat; };
  ClusterSpec spec_;
  std::map<std::string, int> index_;
  std::vector<std::string> names_, kinds_;
  std::vector<uint32_t> mem_gb_;
  std::vector<std::vector<Edge>> adj_;
  void check(size_t d) const { if (d >= names_.size()) throw CostError("device index " + std::to_string(d) + " out of range"); }
};

// ---- TP x PP x EP grid: device = (stage * ep + ep_idx) * tp + tp_idx -------------------------------
struct Placement {
  uint32_t tp = 1, pp = 1, ep = 1;
  static Placement from_plan(const Plan& p) { return {p.parallelism.tp, p.parallelism.pp, p.parallelism.ep}; }
  uint32_t devices() const { return tp * pp * ep; }
  bool holds(size_t d) const { return d < devices(); }
  uint32_t stage_of(size_t d) const { return (uint32_t)(d / (tp * ep)); }
  uint32_t ep_idx(size_t d) const { return (uint32_t)((d / tp) % ep); }
  uint32_t tp_idx(size_t d) const { return (uint32_t)(d % tp); }
  std::vector<size_t> tp_group(size_t d) const {
    std::vector<size_t> g; size_t base = d - tp_idx(d);
    for (uint32_t i = 0; i < tp; ++i) g.push_back(base + i);
    return g;
  }
  std::vector<size_t> ep_group(size_t d) const {
    std::vector<size_t> g; size_t base = (size_t)stage_of(d) * tp * ep + tp_idx(d);
    for (uint32_t i = 0; i < ep; ++i) g.push_back(base + (size_t)i * tp);
    return g;
  }
  std::vector<size_t> pp_group(size_t d) const {
    std::vector<size_t> g; size_t inner = d % ((size_t)tp * ep);
    for (uint32_t s = 0; s < pp; ++s) g.push_back(inner + (size_t)s * tp * ep);
    return g;
  }
};

// Block b of n lives on stage: the remainder is spread over the first stages.
inline uint32_t block_to_stage(size_t b, size_t n, uint32_t pp) {
  size_t base = n / pp, rem = n % pp, start = 0;
  for (uint32_t s = 0; s < pp; ++s) {
    size_t len = base + (s < rem ? 1 : 0);
    if (b < start + len) return s;
    start += len;
  }
  return pp - 1;
}

// ---- workload ----------------------------------------------------------------------------------------
struct Slo {
  double ttft_p95_ms = 500, tpot_p95_ms = 50, max_accuracy_drift = 0.01, recompile_drift_threshold_kl = 0.05;
};
struct RequestRecord { uint64_t prompt_tokens = 0, output_tokens = 0, arrival_ms = 0; };

struct Workload {
  Slo slo;
  std::vector<RequestRecord> requests;

  static Workload from_jsonl_str(const std::string& text) {
    std::istringstream in(text);
    std::string line;
    int lineno = 0;
    bool have_header = false;
    Workload w;
    uint64_t prev = 0;
    while (std::getline(in, line)) {
      ++lineno;
      if (toml_detail::trim(line).empty()) continue;
      Json j;
      try { j = Json::parse(line); } catch (const JsonError& e) {
        throw WorkloadError("trace line " + std::to_string(lineno) + ": " + e.what());
      }
      if (!have_header) {
        const Json* s = j.find("slo");
        if (!s) throw WorkloadError("trace: the first line must be the {\"slo\": ...} header");
        try {
          w.slo.ttft_p95_ms = s->at("ttft_p95_ms").as_double();
          w.slo.tpot_p95_ms = s->at("tpot_p95_ms").as_double();
          w.slo.max_accuracy_drift = s->at("max_accuracy_drift").as_double();
          w.slo.recompile_drift_threshold_kl = s->at("recompile_drift_threshold_kl").as_double();
        } catch (const JsonError& e) { throw WorkloadError(std::string("trace SLO header: ") + e.what()); }
        have_header = true;
        continue;
      }
      RequestRecord r;
      try {
        r.prompt_tokens = j.at("prompt_tokens").as_int();
        r.output_tokens = j.at("output_tokens").as_int();
        r.arrival_ms = j.at("arrival_ms").as_int();
      } catch (const JsonError& e) { throw WorkloadError("trace line " + std::to_string(lineno) + ": " + e.what()); }
      if (r.arrival_ms < prev)
        throw WorkloadError("trace line " + std::to_string(lineno) + ": arrival " + std::to_string(r.arrival_ms) +
                            " ms is earlier than the previous request (" + std::to_string(prev) + " ms)");
      prev = r.arrival_ms;
      w.requests.push_back(r);
    }
    if (!have_header) throw WorkloadError("trace is empty");
    return w;
  }
  std::string to_jsonl() const {
    std::string out = Json::object().set("slo", Json::object().set("ttft_p95_ms", slo.ttft_p95_ms).set("tpot_p95_ms", slo.tpot_p95_ms)
                                                     .set("max_accuracy_drift", slo.max_accuracy_drift)
                                                     .set("recompile_drift_threshold_kl", slo.recompile_drift_threshold_kl)).dump() + "\n";
    for (auto& r : requests)
      out += Json::object().set("prompt_tokens", r.prompt_tokens).set("output_tokens", r.output_tokens).set("arrival_ms", r.arrival_ms).dump() + "\n";
    return out;
  }
  double mean_prompt() const { double s = 0; for (auto& r : requests) s += r.prompt_tokens; return requests.empty() ? 0 : s / requests.size(); }
  double mean_output() const { double s = 0; for (auto& r : requests) s += r.output_tokens; return requests.empty() ? 0 : s / requests.size(); }
};

// Uniform prompt/output lengths, Poisson arrivals at `rate_per_s`.
inline Workload synth_uniform_trace(size_t n, uint64_t seed, uint64_t p_lo, uint64_t p_hi, uint64_t o_lo, uint64_t o_hi, double rate_per_s) {
  std::mt19937_64 rng(seed);
  std::uniform_int_distribution<uint64_t> pd(p_lo, p_hi), od(o_lo, o_hi);
  std::exponential_distribution<double> gap(rate_per_s);
  Workload w;
  double t = 0;
  for (size_t i = 0; i < n; ++i) {
    RequestRecord r{pd(rng), od(rng), (uint64_t)std::llround(t * 1000.0)};
    w.requests.push_back(r);
    t += gap(rng);
  }
  return w;
}

// On/off Poisson bursts (rate alternates every `period_s`), log-normal prompt lengths, uniform outputs.
inline Workload synth_burst_trace(size_t n, uint64_t seed, double hi_rate, double lo_rate, double period_s, double prompt_median,
                                  uint64_t prompt_max, uint64_t o_lo, uint64_t o_hi) {
  std::mt19937_64 rng(seed);
  std::lognormal_distribution<double> pl(std::log(prompt_median), 0.8);
  std::uniform_int_distribution<uint64_t> od(o_lo, o_hi);
  std::uniform_real_distribution<double> u(0.0, 1.0);
  Workload w;
  double t = 0;
  for (size_t i = 0; i < n; ++i) {
    uint64_t p = (uint64_t)std::max(1.0, std::min((double)prompt_max, pl(rng)));
    w.requests.push_back({p, od(rng), (uint64_t)std::llround(t * 1000.0)});
    const bool on = ((long long)std::floor(t / period_s)) % 2 == 0;
    t += -std::log(1.0 - u(rng)) / (on ? hi_rate : lo_rate);
  }
  return w;
}

}  // namespace skein
