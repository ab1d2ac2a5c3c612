// Placement search: enumerate global configurations (TP x PP x EP, KV layout, batch policy), reject
// the impossible ones, choose the per-layer (weight, activation, kv) dtypes of each survivor with a
// knapsack DP over (block, memory bucket, drift bucket), score with the cost model, keep the argmin.
//
// Structure and defaults follow the reference (crates/skein_extract/src/enumerate.rs:20-165,
// constraints.rs:20-95, dp.rs:42-251, budgets.rs:22-29, drift_table.rs:20-245, lib.rs:49-175,
// disaggregate.rs:27-73). Differences: CUDA graphs are enabled with the runtime's real capture
// classes (the reference pins them off), TP must also divide the head counts, and a disaggregated
// plan moves KV over NVLink peer copies.
#pragma once
#include "cost.hpp"
#include <array>
#include <functional>

namespace skein {

struct ExtractError : std::runtime_error { using std::runtime_error::runtime_error; };

// ---- drift table --------------------------------------------------------------------------------------
class DriftTable {
 public:
  static constexpr std::array<Dtype, 6> DTYPES = {Dtype::Bf16, Dtype::Fp16, Dtype::Fp8E4m3, Dtype::Fp8E5m2, Dtype::Int8, Dtype::Int4};
  static constexpr std::array<Component, 3> COMPONENTS = {Component::Weight, Component::Activation, Component::KvCache};

  static DriftTable from_toml_str(const std::string& text) {
    Json j;
    try { j = parse_toml(text); } catch (const TomlError& e) { throw ExtractError(std::string("drift table: ") + e.what()); }
    DriftTable t;
    const Json* def = j.find("default");
    if (!def) throw ExtractError("drift table: missing [default.*] sections");
    for (Component c : COMPONENTS) {
      const Json* sec = def->find(component_name(c));
      if (!sec) throw ExtractError(std::string("drift table: missing [default.") + component_name(c) + "]");
      for (Dtype d : DTYPES) {
        const Json* v = sec->find(dtype_name(d));
        if (!v) throw ExtractError(std::string("drift table: [default.") + component_name(c) + "] lacks " + dtype_name(d));
        t.defaults_[{(int)c, (int)d}] = v->as_double();
      }
    }
    if (const Json* layers = j.find("layer")) {
      for (auto& lk : layers->members()) {
        const size_t layer = (size_t)std::stoul(lk.first);
        for (Component c : COMPONENTS) {
          const Json* sec = lk.second.find(component_name(c));
          if (!sec) continue;
          for (auto& kv : sec->members()) t.overrides_[{layer, (int)c, (int)dtype_from(kv.first)}] = kv.second.as_double();
        }
      }
    }
    return t;
  }
  static DriftTable uniform(double v) {
    DriftTable t;
    for (Component c : COMPONENTS) for (Dtype d : DTYPES) t.defaults_[{(int)c, (int)d}] = d == Dtype::Bf16 ? 0.0 : v;
    return t;
  }
  double lookup(size_t layer, Component c, Dtype d) const {
    auto it = overrides_.find({layer, (int)c, (int)d});
    if (it != overrides_.end()) return it->second;
    auto jt = defaults_.find({(int)c, (int)d});
    return jt == defaults_.end() ? std::numeric_limits<double>::infinity() : jt->second;
  }
  std::optional<double> lookup_raw(size_t layer, Component c, Dtype d) const {
    auto it = overrides_.find({layer, (int)c, (int)d});
    if (it == overrides_.end()) return std::nullopt;
    return it->second;
  }
  double block_contribution(size_t layer, Dtype w, Dtype a, Dtype kv) const {
    return lookup(layer, Component::Weight, w) + lookup(layer, Component::Activation, a) + lookup(layer, Component::KvCache, kv);
  }
  void set_layer_override(size_t layer, Component c, Dtype d, double v) { overrides_[{layer, (int)c, (int)d}] = v; }
  void set_default(Component c, Dtype d, double v) { defaults_[{(int)c, (int)d}] = v; }
  // Monotonic raise: a measured failure may only make a dtype look worse (crates/skein_parity/src/drift_update.rs:30).
  bool raise_layer_override(size_t layer, Component c, Dtype d, double v) {
    auto cur = lookup_raw(layer, c, d);
    if (cur && *cur >= v) return false;
    set_layer_override(layer, c, d, v);
    return true;
  }
  // Canonical text: defaults in component/dtype order, then overrides sorted by (layer, component, dtype).
  std::string serialize_to_toml() const {
    std::string out;
    for (Component c : COMPONENTS) {
      out += std::string("[default.") + component_name(c) + "]\n";
      for (Dtype d : DTYPES) {
        auto it = defaults_.find({(int)c, (int)d});
        if (it != defaults_.end()) out += std::string(dtype_name(d)) + " = " + Json::fmt_double(it->second) + "\n";
      }
      out += "\n";
    }
    std::tuple<size_t, int> cur{(size_t)-1, -1};
    for (auto& kv : overrides_) {  // std::map iterates in (layer, component, dtype-enum) order
      auto [layer, comp, dt] = kv.first;
      if (std::make_tuple(layer, comp) != cur) {
        if (std::get<1>(cur) != -1) out += "\n";
        out += "[layer." + std::to_string(layer) + "." + component_name((Component)comp) + "]\n";
        cur = {layer, comp};
      }
      out += std::string(dtype_name((Dtype)dt)) + " = " + Json::fmt_double(kv.second) + "\n";
    }
    return out;
  }
  size_t num_overrides() const { return overrides_.size(); }

 private:
  std::map<std::pair<int, int>, double> defaults_;
  std::map<std::tuple<size_t, int, int>, double> overrides_;
};

// ---- candidates -----------------------------------------------------------------------------------------
struct GlobalConfig {
  ParallelismPlacement parallelism;
  KVCacheSpec kv;
  BatchPolicy batch;
  ExecutionConfig execution;
};

inline std::vector<uint32_t> capture_batch_sizes(uint32_t max_batch) {
  std::vector<uint32_t> v;
  for (uint32_t b = 1; b < max_batch; b *= 2) v.push_back(b);
  v.push_back(max_batch);
  return v;
}

inline std::vector<ParallelismPlacement> enumerate_parallelism(uint32_t num_devices, const Graph& ir) {
  std::vector<ParallelismPlacement> out;
  const uint32_t ep_max = ir.meta.is_moe() ? std::min<uint32_t>((uint32_t)*ir.meta.num_experts, 8) : 1;
  for (uint32_t tp : {1u, 2u, 4u, 8u})
    for (uint32_t pp : {1u, 2u, 4u})
      for (uint32_t ep = 1; ep <= ep_max; ep *= 2) {
        if (tp * pp * ep > num_devices) break;
        out.push_back({tp, pp, ep});
      }
  return out;
}

struct SearchOptions {
  std::optional<uint32_t> force_tp, force_pp, force_ep, force_batch;
  bool enable_cuda_graphs = true;
  // false: minimise the decode-step latency (the reference's objective; it favours batch 1).
  // true: minimise time per generated token (step time / max_batch) among plans whose step time meets the TPOT SLO.
  bool objective_throughput = false;
  std::vector<uint32_t> batch_ladder = {1, 2, 4, 8, 16, 32, 64};
};

inline std::vector<GlobalConfig> enumerate_global_configs(const Cluster& cl, const Graph& ir, const SearchOptions& opt) {
  std::vector<GlobalConfig> out;
  std::vector<KVCacheSpec> kvs;
  // The cost model does not distinguish KV layouts, so ties go to the first one listed: paged with
  // 16-token pages and head-sharded KV, the layout the runtime's kernels use.
  for (uint32_t n : {16u, 32u, 64u, 128u}) { kvs.push_back({true, n, true}); kvs.push_back({true, n, false}); }
  kvs.push_back({false, 0, true});
  kvs.push_back({false, 0, false});
  std::vector<uint32_t> ladder = opt.batch_ladder;
  if (opt.force_batch && std::find(ladder.begin(), ladder.end(), *opt.force_batch) == ladder.end()) ladder.push_back(*opt.force_batch);
  for (auto& par : enumerate_parallelism((uint32_t)cl.num_devices(), ir))
    for (auto& kv : kvs)
      for (uint32_t mb : ladder)
        for (int chunked = 0; chunked < 2; ++chunked) {
          GlobalConfig g;
          g.parallelism = par;
          g.kv = kv;
          g.batch = chunked ? BatchPolicy{BatchKind::ContinuousChunked, mb, 1024} : BatchPolicy{BatchKind::Continuous, mb, 0};
          g.execution.cuda_graphs = opt.enable_cuda_graphs;
          if (opt.enable_cuda_graphs) for (uint32_t b : capture_batch_sizes(mb)) g.execution.capture_classes.push_back({b, 0});
          g.execution.spec_decode = false;
          g.execution.prefix_cache = true;
          out.push_back(g);
        }
  return out;
}

enum class RejectReason { None, TpDivisibility, EpDivisibility, DeviceCount, GlobalMemory };
inline const char* reject_name(RejectReason r) {
  switch (r) {
    case RejectReason::TpDivisibility: return "tp_divisibility"; case RejectReason::EpDivisibility: return "ep_divisibility";
    case RejectReason::DeviceCount: return "device_count"; case RejectReason::GlobalMemory: return "global_memory";
    default: return "none";
  }
}

inline uint64_t min_device_memory(const Cluster& cl) {
  uint64_t m = std::numeric_limits<uint64_t>::max();
  for (size_t d = 0; d < cl.num_devices(); ++d) m = std::min(m, cl.device_memory_bytes(d));
  return m;
}

inline RejectReason reject(const GlobalConfig& g, const Cluster& cl, const Graph& ir, const CostConstants& c) {
  const auto& p = g.parallelism;
  if (ir.meta.hidden % p.tp || ir.meta.num_attention_heads % p.tp || ir.meta.num_kv_heads % p.tp || ir.meta.intermediate % p.tp)
    return RejectReason::TpDivisibility;
  if (ir.meta.is_moe() ? (*ir.meta.num_experts % p.ep != 0) : (p.ep != 1)) return RejectReason::EpDivisibility;
  if (p.devices_used() > cl.num_devices()) return RejectReason::DeviceCount;
  // optimistic fit: int4 weights, fp8 KV
  const Placement pl{p.tp, p.pp, p.ep};
  const WorkloadCtx wl{g.batch.max_batch, 1, c.decode_kv_tokens};
  uint64_t total = 0;
  for (size_t b = 0; b < ir.meta.num_layers; ++b)
    total += block_weight_bytes(b, ir, Dtype::Int4, pl) / p.pp + block_kv_bytes(ir, Dtype::Fp8E4m3, pl, wl, g.kv.kv_sharded) / p.pp;
  total += non_decoder_weight_bytes(ir, pl);
  if (total > min_device_memory(cl)) return RejectReason::GlobalMemory;
  return RejectReason::None;
}

// ---- per-layer dtype DP -------------------------------------------------------------------------------------
struct Budgets { uint64_t memory_bytes = 0; double drift = 0; };

inline Budgets budgets_after_global(const GlobalConfig& g, const Cluster& cl, const Workload& wl, const Graph& ir) {
  const Placement pl{g.parallelism.tp, g.parallelism.pp, g.parallelism.ep};
  const uint64_t cap = min_device_memory(cl), reserved = non_decoder_weight_bytes(ir, pl);
  return {cap > reserved ? cap - reserved : 0, wl.slo.max_accuracy_drift};
}

inline std::vector<PerLayerDtype> all_combos() {
  std::vector<PerLayerDtype> out;
  for (Dtype w : {Dtype::Bf16, Dtype::Fp8E4m3, Dtype::Int8, Dtype::Int4})
    for (Dtype a : {Dtype::Bf16, Dtype::Fp8E4m3})
      for (Dtype k : {Dtype::Bf16, Dtype::Fp8E4m3, Dtype::Int8}) out.push_back({w, a, k});
  return out;
}

struct DpResult { double cost_us = 0; std::vector<PerLayerDtype> dtype_map; };

// Minimises the summed block compute time subject to memory and drift budgets. Returns nullopt when
// no assignment fits. `allowed` optionally restricts the combos (e.g. to dtypes the kernels implement).
inline std::optional<DpResult> layer_dtype_dp(const Graph& ir, const CostModel& cm, const Cluster& cl, const GlobalConfig& g, Budgets bud,
                                              const DriftTable& drift, const std::vector<PerLayerDtype>* allowed = nullptr) {
  const CostConstants& c = cm.constants();
  const size_t MB = c.memory_buckets, DB = c.drift_buckets, NB = ir.meta.num_layers;
  const Placement pl{g.parallelism.tp, g.parallelism.pp, g.parallelism.ep};
  const WorkloadCtx wl{g.batch.max_batch, 1, c.decode_kv_tokens};
  if (bud.memory_bytes == 0) return std::nullopt;
  const uint64_t bytes_per_bucket = std::max<uint64_t>(1, (bud.memory_bytes + MB - 1) / MB);
  const double drift_per_bucket = std::max(bud.drift / (double)DB, std::numeric_limits<double>::min());
  const std::vector<PerLayerDtype> combos = allowed ? *allowed : all_combos();
  const size_t NC = combos.size();
  std::vector<size_t> mem_step(NB * NC), drift_step(NB * NC);
  std::vector<double> cost(NB * NC);
  std::vector<char> ok(NB * NC, 1);
  for (size_t b = 0; b < NB; ++b)
    for (size_t ci = 0; ci < NC; ++ci) {
      const auto& cb = combos[ci];
      const uint64_t mem = block_weight_bytes(b, ir, cb.weight, pl) / pl.pp + block_kv_bytes(ir, cb.kv_cache, pl, wl, g.kv.kv_sharded) / pl.pp;
      const double dr = drift.block_contribution(b, cb.weight, cb.activation, cb.kv_cache);
      if (!std::isfinite(dr)) { ok[b * NC + ci] = 0; continue; }
      mem_step[b * NC + ci] = (size_t)((mem + bytes_per_bucket - 1) / bytes_per_bucket);
      drift_step[b * NC + ci] = (size_t)std::max(0.0, std::ceil(dr / drift_per_bucket));
      cost[b * NC + ci] = block_compute_time(b, ir, cb.weight, cb.kv_cache, pl, cl, c, wl, 0);
    }
  const size_t MD = MB + 1, DD = DB + 1;
  const double INF = std::numeric_limits<double>::infinity();
  std::vector<double> dp((NB + 1) * MD * DD, INF);
  struct Back { uint16_t combo, pm, pd; bool set = false; };
  std::vector<Back> back((NB + 1) * MD * DD);
  auto idx = [&](size_t b, size_t m, size_t d) { return (b * MD + m) * DD + d; };
  dp[idx(0, 0, 0)] = 0;
  for (size_t b = 0; b < NB; ++b)
    for (size_t m = 0; m < MD; ++m)
      for (size_t d = 0; d < DD; ++d) {
        const double base = dp[idx(b, m, d)];
        if (!std::isfinite(base)) continue;
        for (size_t ci = 0; ci < NC; ++ci) {
          if (!ok[b * NC + ci]) continue;
          const size_t m2 = m + mem_step[b * NC + ci], d2 = d + drift_step[b * NC + ci];
          if (m2 > MB || d2 > DB) continue;
          const double nc = base + cost[b * NC + ci];
          const size_t i2 = idx(b + 1, m2, d2);
          if (nc < dp[i2]) { dp[i2] = nc; back[i2] = {(uint16_t)ci, (uint16_t)m, (uint16_t)d, true}; }
        }
      }
  double best = INF;
  size_t bm = 0, bd = 0;
  for (size_t m = 0; m < MD; ++m)
    for (size_t d = 0; d < DD; ++d)
      if (dp[idx(NB, m, d)] < best) { best = dp[idx(NB, m, d)]; bm = m; bd = d; }
  if (!std::isfinite(best)) return std::nullopt;
  DpResult r;
  r.cost_us = best;
  r.dtype_map.assign(NB, PerLayerDtype{});
  for (size_t b = NB; b-- > 0;) {
    const Back& bp = back[idx(b + 1, bm, bd)];
    r.dtype_map[b] = combos[bp.combo];
    bm = bp.pm; bd = bp.pd;
  }
  return r;
}

// ---- driver ---------------------------------------------------------------------------------------------------
struct SearchCounters {
  uint64_t raw = 0, survivors = 0, dp_infeasible = 0, scored = 0, rejected_tp = 0, rejected_ep = 0, rejected_devices = 0, rejected_memory = 0;
  Json to_json() const {
    return Json::object().set("raw", raw).set("survivors", survivors).set("dp_infeasible", dp_infeasible).set("scored", scored)
        .set("rejected_tp_divisibility", rejected_tp).set("rejected_ep_divisibility", rejected_ep)
        .set("rejected_device_count", rejected_devices).set("rejected_global_memory", rejected_memory);
  }
};

struct ExtractResult { Plan plan; double cost_us = 0; SearchCounters counters; };

inline Plan compose_plan(const GlobalConfig& g, std::vector<PerLayerDtype> dm, const ModelMeta& meta) {
  Plan p;
  p.parallelism = g.parallelism; p.kv = g.kv; p.batching = g.batch; p.dtype_map = std::move(dm); p.execution = g.execution; p.model_meta = meta;
  return p;
}

inline ExtractResult extract_plan(const Graph& ir, const Cluster& cl, const Workload& wl, const DriftTable& drift, const CostModel& cm,
                                  const SearchOptions& opt = {}, const std::vector<PerLayerDtype>* allowed = nullptr) {
  ExtractResult res;
  bool have = false;
  double best_score = 0;
  std::map<std::tuple<uint32_t, uint32_t, uint32_t, uint32_t, bool>, std::optional<std::vector<PerLayerDtype>>> memo;
  // throughput objective: the prompt length that 95 % of the trace's requests stay below; its prefill has to fit the TTFT target
  uint32_t p95_prompt = 0;
  if (opt.objective_throughput && !wl.requests.empty()) {
    std::vector<uint64_t> lens;
    for (auto& r : wl.requests) lens.push_back(r.prompt_tokens);
    std::sort(lens.begin(), lens.end());
    p95_prompt = (uint32_t)lens[std::min(lens.size() - 1, (size_t)(0.95 * (double)lens.size()))];
  }
  // kept in case no plan meets both targets (a plan that misses a target is still better than none): the best plan by the
  // objective among those that meet the TPOT target but not the TTFT one, else the plan with the shortest step
  ExtractResult fallback, fallback_tpot;
  bool have_fallback = false, have_fallback_tpot = false;
  double fallback_tpot_score = 0;
  for (auto& g : enumerate_global_configs(cl, ir, opt)) {
    ++res.counters.raw;
    if ((opt.force_tp && g.parallelism.tp != *opt.force_tp) || (opt.force_pp && g.parallelism.pp != *opt.force_pp) ||
        (opt.force_ep && g.parallelism.ep != *opt.force_ep) || (opt.force_batch && g.batch.max_batch != *opt.force_batch))
      continue;
    switch (reject(g, cl, ir, cm.constants())) {
      case RejectReason::TpDivisibility: ++res.counters.rejected_tp; continue;
      case RejectReason::EpDivisibility: ++res.counters.rejected_ep; continue;
      case RejectReason::DeviceCount: ++res.counters.rejected_devices; continue;
      case RejectReason::GlobalMemory: ++res.counters.rejected_memory; continue;
      default: break;
    }
    ++res.counters.survivors;
    auto key = std::make_tuple(g.parallelism.tp, g.parallelism.pp, g.parallelism.ep, g.batch.max_batch, g.kv.kv_sharded);
    auto it = memo.find(key);
    if (it == memo.end()) {
      auto r = layer_dtype_dp(ir, cm, cl, g, budgets_after_global(g, cl, wl, ir), drift, allowed);
      it = memo.emplace(key, r ? std::optional<std::vector<PerLayerDtype>>(r->dtype_map) : std::nullopt).first;
    }
    if (!it->second) { ++res.counters.dp_infeasible; continue; }
    Plan plan = compose_plan(g, *it->second, ir.meta);
    const double total = cm.total_cost(plan, ir, cl);
    ++res.counters.scored;
    double score = total;
    if (opt.objective_throughput) {
      if (!have_fallback || total < fallback.cost_us) { fallback.plan = plan; fallback.cost_us = total; have_fallback = true; }
      if (total / 1000.0 > wl.slo.tpot_p95_ms) continue;
      const double tput_score = total / (double)g.batch.max_batch;
      if (!have_fallback_tpot || tput_score < fallback_tpot_score) {
        fallback_tpot.plan = plan; fallback_tpot.cost_us = total; fallback_tpot_score = tput_score; have_fallback_tpot = true;
      }
      if (p95_prompt > 0) {
        // one sequence of that length through every stage in turn (tensor- and expert-parallel ranks of a stage work side by side)
        const Placement pl = Placement::from_plan(plan);
        Plan one = plan;
        one.batching.max_batch = 1;
        const WorkloadCtx pw{1, p95_prompt, p95_prompt};
        std::vector<double> stage_us(std::max(1u, plan.parallelism.pp), 0.0);
        for (size_t d = 0; d < cl.num_devices(); ++d)
          if (pl.holds(d)) stage_us[pl.stage_of(d)] = std::max(stage_us[pl.stage_of(d)], cm.compute_on_device(one, ir, cl, pw, d));
        double prefill_us = 0;
        for (double t : stage_us) prefill_us += t;
        if (prefill_us / 1000.0 > wl.slo.ttft_p95_ms) continue;
      }
      score = total / (double)g.batch.max_batch;
    }
    if (!have || score < best_score) { res.plan = plan; res.cost_us = total; best_score = score; have = true; }
  }
  if (!have && have_fallback_tpot) {
    res.plan = fallback_tpot.plan; res.cost_us = fallback_tpot.cost_us; have = true;
  } else if (!have && have_fallback) {
    res.plan = fallback.plan; res.cost_us = fallback.cost_us; have = true;
  }
  if (!have) {
    const auto& c = res.counters;
    const char* dom = "none";
    uint64_t mx = 0;
    for (auto [n, name] : {std::pair<uint64_t, const char*>{c.rejected_tp, "tp_divisibility"}, {c.rejected_ep, "ep_divisibility"},
                           {c.rejected_devices, "device_count"}, {c.rejected_memory, "global_memory"}})
      if (n > mx) { mx = n; dom = name; }
    throw ExtractError("no feasible plan: " + std::to_string(c.raw) + " candidates, " + std::to_string(c.dp_infeasible) +
                       " failed the dtype DP, dominant rejection: " + dom);
  }
  return res;
}

// ---- prefill/decode disaggregation -------------------------------------------------------------------------------
inline ClusterSpec sub_cluster_spec(const ClusterSpec& spec, const std::set<std::string>& keep) {
  ClusterSpec s;
  for (auto& n : spec.nodes) {
    Node x = n;
    x.devices.clear();
    for (auto& d : n.devices) if (keep.count(d)) x.devices.push_back(d);
    if (!x.devices.empty()) s.nodes.push_back(x);
  }
  for (auto& l : spec.links) if (keep.count(l.a) && keep.count(l.b)) s.links.push_back(l);
  s.num_devices = (uint32_t)keep.size();
  return s;
}

inline ExtractResult extract_disaggregated_plan(const Graph& ir, const Cluster& cl, const Workload& wl, const DriftTable& drift,
                                                const CostModel& cm, size_t decode_devices, const SearchOptions& opt = {}) {
  auto devs = cl.spec().all_devices();
  if (decode_devices == 0 || decode_devices >= devs.size())
    throw ExtractError("invalid disaggregation: " + std::to_string(decode_devices) + " decode devices of " + std::to_string(devs.size()));
  std::set<std::string> dset(devs.begin(), devs.begin() + decode_devices), pset(devs.begin() + decode_devices, devs.end());
  Cluster dcl(sub_cluster_spec(cl.spec(), dset)), pcl(sub_cluster_spec(cl.spec(), pset));
  ExtractResult d = extract_plan(ir, dcl, wl, drift, cm, opt), p = extract_plan(ir, pcl, wl, drift, cm, opt);
  ExtractResult out = d;
  Disaggregation dis;
  dis.prefill = std::make_shared<Plan>(p.plan);
  dis.decode = std::make_shared<Plan>(d.plan);
  dis.mode = KvTransferMode::NvlinkP2p;
  dis.layer_overlap = true;
  out.plan.disaggregation = dis;
  out.cost_us = std::max(d.cost_us, p.cost_us);
  return out;
}

}  // namespace skein
