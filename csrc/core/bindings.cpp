// Python bindings of the C++ host core (module skein_b200._native._skein_core).
// Structured values cross the boundary as JSON text (the same text the CLI reads and writes);
// stateful runtime objects (KV manager, batcher, metrics, drift table) are bound as classes.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../runtime/batcher.hpp"
#include "../runtime/misc.hpp"
#include "emit.hpp"
#include "importer.hpp"
#include "planner.hpp"

namespace py = pybind11;
using namespace skein;

namespace {

SearchOptions options_from(const py::dict& d) {
  SearchOptions o;
  auto geti = [&](const char* k) -> std::optional<uint32_t> {
    if (d.contains(k) && !d[k].is_none()) return d[k].cast<uint32_t>();
    return std::nullopt;
  };
  o.force_tp = geti("force_tp"); o.force_pp = geti("force_pp"); o.force_ep = geti("force_ep"); o.force_batch = geti("force_batch");
  if (d.contains("enable_cuda_graphs")) o.enable_cuda_graphs = d["enable_cuda_graphs"].cast<bool>();
  if (d.contains("objective")) o.objective_throughput = d["objective"].cast<std::string>() == "throughput";
  if (d.contains("batch_ladder")) o.batch_ladder = d["batch_ladder"].cast<std::vector<uint32_t>>();
  return o;
}

std::vector<PerLayerDtype> combos_from(const std::vector<std::vector<std::string>>& v) {
  std::vector<PerLayerDtype> out;
  for (auto& c : v) {
    if (c.size() != 3) throw ExtractError("each allowed combo is [weight, activation, kv_cache]");
    out.push_back({dtype_from(c[0]), dtype_from(c[1]), dtype_from(c[2])});
  }
  return out;
}

struct PlannerInputs {
  Graph ir;
  Cluster cluster;
  Workload workload;
  CostModel cost;
  PlannerInputs(const std::string& config_json, const std::string& cluster_toml, const std::string& trace_jsonl, const std::string& constants_toml)
      : ir(import_model_str(config_json)), cluster(ClusterSpec::from_toml_str(cluster_toml)), workload(Workload::from_jsonl_str(trace_jsonl)),
        cost(CostConstants::from_toml_str(constants_toml)) {}
};

py::dict result_to_py(const ExtractResult& r) {
  py::dict d;
  d["plan_json"] = r.plan.to_json().dump();
  d["cost_us"] = r.cost_us;
  d["counters_json"] = r.counters.to_json().dump();
  d["content_hash"] = r.plan.content_hash();
  return d;
}

}  // namespace

PYBIND11_MODULE(_skein_core, m) {
  m.doc() = "skein_b200 host core: IR, plan, cost model, planner, lowering, KV manager, batcher, metrics";

  py::register_exception<ImportError>(m, "ImportError_");
  py::register_exception<ClusterError>(m, "ClusterError");
  py::register_exception<WorkloadError>(m, "WorkloadError");
  py::register_exception<PlanError>(m, "PlanError");
  py::register_exception<CostError>(m, "CostError");
  py::register_exception<ExtractError>(m, "ExtractError");
  py::register_exception<RuntimeError>(m, "RuntimeError_");
  py::register_exception<JsonError>(m, "JsonError");
  py::register_exception<TomlError>(m, "TomlError");

  // ---- utilities ----
  m.def("blake3_hex", [](py::bytes b) { return blake3_hex(std::string(b)); });
  m.def("toml_to_json", [](const std::string& s) { return parse_toml(s).dump(); });
  m.def("json_canonical", [](const std::string& s) { return Json::parse(s).dump(); });
  m.def("dtype_bits", [](const std::string& d) { return dtype_bits(dtype_from(d)); });
  m.def("dtype_bytes_for", [](const std::string& d, uint64_t n) { return dtype_bytes_for(dtype_from(d), n); });

  // ---- IR / plan ----
  m.def("import_model", [](const std::string& cfg) { return import_model_str(cfg).to_json().dump(); });
  m.def("model_param_count", [](const std::string& cfg) { return import_model_str(cfg).param_count(); });
  m.def("model_meta", [](const std::string& cfg) { return import_model_str(cfg).meta.to_json().dump(); });
  m.def("plan_roundtrip", [](const std::string& p) { Plan x = Plan::from_json(Json::parse(p)); x.validate(); return x.to_json().dump(); });
  m.def("plan_hash", [](const std::string& p) { return Plan::from_json(Json::parse(p)).content_hash(); });
  m.def("plan_validate", [](const std::string& p) { Plan::from_json(Json::parse(p)).validate(); });
  m.def("cluster_validate", [](const std::string& toml) { return ClusterSpec::from_toml_str(toml).to_json().dump(); });
  m.def("workload_parse", [](const std::string& s) {
    Workload w = Workload::from_jsonl_str(s);
    py::dict d;
    d["n"] = w.requests.size(); d["ttft_p95_ms"] = w.slo.ttft_p95_ms; d["tpot_p95_ms"] = w.slo.tpot_p95_ms;
    d["max_accuracy_drift"] = w.slo.max_accuracy_drift; d["recompile_drift_threshold_kl"] = w.slo.recompile_drift_threshold_kl;
    d["mean_prompt"] = w.mean_prompt(); d["mean_output"] = w.mean_output();
    return d;
  });
  m.def("synth_uniform_trace", [](size_t n, uint64_t seed, uint64_t p_lo, uint64_t p_hi, uint64_t o_lo, uint64_t o_hi, double rate) {
    return synth_uniform_trace(n, seed, p_lo, p_hi, o_lo, o_hi, rate).to_jsonl();
  });
  m.def("synth_burst_trace", [](size_t n, uint64_t seed, double hi, double lo, double period, double median, uint64_t pmax, uint64_t o_lo, uint64_t o_hi) {
    return synth_burst_trace(n, seed, hi, lo, period, median, pmax, o_lo, o_hi).to_jsonl();
  });

  // ---- topology / placement ----
  m.def("pair_path", [](const std::string& cluster_toml, size_t a, size_t b) {
    Cluster c(ClusterSpec::from_toml_str(cluster_toml));
    PathInfo p = c.pair_path(a, b);
    return py::make_tuple(p.min_bandwidth_gbps, p.total_latency_us, p.hops);
  });
  m.def("collective_path", [](const std::string& cluster_toml, const std::vector<size_t>& parts) {
    Cluster c(ClusterSpec::from_toml_str(cluster_toml));
    PathInfo p = c.collective_path(parts);
    return py::make_tuple(p.min_bandwidth_gbps, p.total_latency_us, p.hops);
  });
  m.def("placement_groups", [](uint32_t tp, uint32_t pp, uint32_t ep, size_t device) {
    Placement pl{tp, pp, ep};
    py::dict d;
    d["stage"] = pl.stage_of(device); d["tp_group"] = pl.tp_group(device); d["ep_group"] = pl.ep_group(device); d["pp_group"] = pl.pp_group(device);
    return d;
  });
  m.def("block_to_stage", &block_to_stage);
  m.def("collective_factor", [](const std::string& kind, size_t n) {
    for (CollectiveKind k : {CollectiveKind::RingAllReduce, CollectiveKind::AllGather, CollectiveKind::ReduceScatter, CollectiveKind::AllToAll,
                             CollectiveKind::Broadcast, CollectiveKind::SendRecv})
      if (kind == collective_name(k)) return collective_factor(k, n);
    throw CostError("unknown collective `" + kind + "`");
  });

  // ---- cost model ----
  m.def("total_cost", [](const std::string& plan, const std::string& cfg, const std::string& cluster_toml, const std::string& constants_toml) {
    Graph ir = import_model_str(cfg);
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    CostModel cm(CostConstants::from_toml_str(constants_toml));
    return cm.total_cost(Plan::from_json(Json::parse(plan)), ir, cl);
  });
  m.def("cost_breakdown", [](const std::string& plan, const std::string& cfg, const std::string& cluster_toml, const std::string& constants_toml, size_t device) {
    Graph ir = import_model_str(cfg);
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    CostModel cm(CostConstants::from_toml_str(constants_toml));
    Plan p = Plan::from_json(Json::parse(plan));
    CostBreakdown b = cm.per_device(p, ir, cl, WorkloadCtx::decode_step(p, cm.constants()), device);
    py::dict d;
    d["compute"] = b.compute; d["comm"] = b.comm; d["memory"] = b.memory; d["bubble"] = b.bubble; d["launch"] = b.launch; d["total"] = b.total();
    d["weight_bytes"] = weight_bytes_on_device(p, ir, device); d["kv_bytes"] = kv_bytes_on_device(p, ir, cm.constants(), device);
    d["activation_bytes"] = activation_bytes_on_device(p, ir, device); d["kernels"] = kernels_per_step_on_device(ir, p, device);
    d["collectives"] = collectives_on_device(p, ir, device).size();
    return d;
  });
  m.def("comm_time", [](const std::string& kind, const std::vector<size_t>& parts, uint64_t bytes, const std::string& cluster_toml, const std::string& constants_toml) {
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    CostConstants c = CostConstants::from_toml_str(constants_toml);
    for (CollectiveKind k : {CollectiveKind::RingAllReduce, CollectiveKind::AllGather, CollectiveKind::ReduceScatter, CollectiveKind::AllToAll,
                             CollectiveKind::Broadcast, CollectiveKind::SendRecv})
      if (kind == collective_name(k)) return comm_time(Collective{k, parts, bytes}, cl, c);
    throw CostError("unknown collective `" + kind + "`");
  });
  m.def("bubble_time", [](const std::string& plan, double stage_us) { return bubble_time(Plan::from_json(Json::parse(plan)), stage_us); });
  m.def("cuda_graph_coverage", [](const std::string& plan) { return cuda_graph_coverage(Plan::from_json(Json::parse(plan))); });
  m.def("cost_constants_json", [](const std::string& toml) { return CostConstants::from_toml_str(toml).raw.dump(); });

  // ---- planner ----
  m.def("extract_plan", [](const std::string& cfg, const std::string& cluster_toml, const std::string& trace, const std::string& drift_toml,
                           const std::string& constants_toml, const py::dict& options, const std::vector<std::vector<std::string>>& allowed) {
    PlannerInputs in(cfg, cluster_toml, trace, constants_toml);
    DriftTable dt = DriftTable::from_toml_str(drift_toml);
    auto combos = combos_from(allowed);
    const SearchOptions opt = options_from(options);
    ExtractResult r;
    {
      py::gil_scoped_release rel;  // the search touches no Python object
      r = extract_plan(in.ir, in.cluster, in.workload, dt, in.cost, opt, combos.empty() ? nullptr : &combos);
    }
    return result_to_py(r);
  }, py::arg("config_json"), py::arg("cluster_toml"), py::arg("trace_jsonl"), py::arg("drift_toml"), py::arg("constants_toml"),
     py::arg("options") = py::dict(), py::arg("allowed_combos") = std::vector<std::vector<std::string>>{});
  m.def("extract_disaggregated_plan", [](const std::string& cfg, const std::string& cluster_toml, const std::string& trace, const std::string& drift_toml,
                                         const std::string& constants_toml, size_t decode_devices, const py::dict& options) {
    PlannerInputs in(cfg, cluster_toml, trace, constants_toml);
    DriftTable dt = DriftTable::from_toml_str(drift_toml);
    return result_to_py(extract_disaggregated_plan(in.ir, in.cluster, in.workload, dt, in.cost, decode_devices, options_from(options)));
  }, py::arg("config_json"), py::arg("cluster_toml"), py::arg("trace_jsonl"), py::arg("drift_toml"), py::arg("constants_toml"),
     py::arg("decode_devices"), py::arg("options") = py::dict());
  m.def("enumerate_count", [](const std::string& cfg, const std::string& cluster_toml) {
    Graph ir = import_model_str(cfg);
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    return enumerate_global_configs(cl, ir, SearchOptions{}).size();
  });
  m.def("enumerate_parallelism", [](const std::string& cfg, uint32_t n) {
    Graph ir = import_model_str(cfg);
    std::vector<std::tuple<uint32_t, uint32_t, uint32_t>> out;
    for (auto& p : enumerate_parallelism(n, ir)) out.emplace_back(p.tp, p.pp, p.ep);
    return out;
  });
  m.def("reject_reason", [](const std::string& cfg, const std::string& cluster_toml, const std::string& constants_toml, uint32_t tp, uint32_t pp, uint32_t ep,
                            uint32_t max_batch, bool kv_sharded) {
    Graph ir = import_model_str(cfg);
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    GlobalConfig g;
    g.parallelism = {tp, pp, ep}; g.batch = {BatchKind::Continuous, max_batch, 0}; g.kv = {true, 16, kv_sharded};
    return std::string(reject_name(reject(g, cl, ir, CostConstants::from_toml_str(constants_toml))));
  });
  m.def("layer_dtype_dp", [](const std::string& cfg, const std::string& cluster_toml, const std::string& constants_toml, const std::string& drift_toml,
                             uint32_t tp, uint32_t pp, uint32_t ep, uint32_t max_batch, bool kv_sharded, uint64_t memory_bytes, double drift_budget) -> py::object {
    Graph ir = import_model_str(cfg);
    Cluster cl(ClusterSpec::from_toml_str(cluster_toml));
    CostModel cm(CostConstants::from_toml_str(constants_toml));
    GlobalConfig g;
    g.parallelism = {tp, pp, ep}; g.batch = {BatchKind::Continuous, max_batch, 0}; g.kv = {true, 16, kv_sharded};
    auto r = layer_dtype_dp(ir, cm, cl, g, Budgets{memory_bytes, drift_budget}, DriftTable::from_toml_str(drift_toml));
    if (!r) return py::none();
    std::vector<std::tuple<std::string, std::string, std::string>> dm;
    for (auto& d : r->dtype_map) dm.emplace_back(dtype_name(d.weight), dtype_name(d.activation), dtype_name(d.kv_cache));
    return py::make_tuple(r->cost_us, dm);
  });

  // ---- lowering ----
  m.def("emit_topology", [](const std::string& plan, const std::string& cfg) {
    Plan p = Plan::from_json(Json::parse(plan));
    return topology_to_json(emit_topology(p, import_model_str(cfg)), p).dump();
  });
  m.def("lower_device", [](const std::string& plan, const std::string& cfg, size_t device) {
    return lowered_to_json(lower_device(Plan::from_json(Json::parse(plan)), import_model_str(cfg), device)).dump();
  });
  // the same lowering for a placement given by its three degrees (the decoder asks for the program of its own rank
  // when it is built without an artifact: benchmarks, tests)
  m.def("lower_device_for", [](const std::string& cfg, uint32_t tp, uint32_t pp, uint32_t ep, size_t device) {
    Plan p;
    p.parallelism.tp = tp; p.parallelism.pp = pp; p.parallelism.ep = ep;
    return lowered_to_json(lower_device(p, import_model_str(cfg), device)).dump();
  });
  m.def("io_manifest", [](const std::string& plan, const std::string& cfg, size_t device) {
    return io_manifest(Plan::from_json(Json::parse(plan)), import_model_str(cfg), device).dump();
  });
  m.def("param_kind_for", [](const std::string& name) {
    ParamRole r = param_kind_for(name);
    const char* k = r.kind == ParamKind::Replicated ? "replicated" : r.kind == ParamKind::ColumnParallel ? "column" : r.kind == ParamKind::RowParallel ? "row" : "expert";
    return py::make_tuple(std::string(k), r.expert_idx, r.expert_column);
  });

  // ---- drift table ----
  py::class_<DriftTable>(m, "DriftTable")
      .def_static("from_toml", &DriftTable::from_toml_str)
      .def_static("uniform", &DriftTable::uniform)
      .def("lookup", [](const DriftTable& t, size_t layer, const std::string& comp, const std::string& dt) {
        return t.lookup(layer, comp == "weight" ? Component::Weight : comp == "activation" ? Component::Activation : Component::KvCache, dtype_from(dt));
      })
      .def("block_contribution", [](const DriftTable& t, size_t layer, const std::string& w, const std::string& a, const std::string& k) {
        return t.block_contribution(layer, dtype_from(w), dtype_from(a), dtype_from(k));
      })
      .def("set_layer_override", [](DriftTable& t, size_t layer, const std::string& comp, const std::string& dt, double v) {
        t.set_layer_override(layer, comp == "weight" ? Component::Weight : comp == "activation" ? Component::Activation : Component::KvCache, dtype_from(dt), v);
      })
      .def("raise_layer_override", [](DriftTable& t, size_t layer, const std::string& comp, const std::string& dt, double v) {
        return t.raise_layer_override(layer, comp == "weight" ? Component::Weight : comp == "activation" ? Component::Activation : Component::KvCache, dtype_from(dt), v);
      })
      .def("set_default", [](DriftTable& t, const std::string& comp, const std::string& dt, double v) {
        t.set_default(comp == "weight" ? Component::Weight : comp == "activation" ? Component::Activation : Component::KvCache, dtype_from(dt), v);
      })
      .def("to_toml", &DriftTable::serialize_to_toml)
      .def("num_overrides", &DriftTable::num_overrides);

  // ---- KV manager ----
  py::class_<PageTable>(m, "PageTable")
      .def_readonly("request_id", &PageTable::request_id).def_readonly("pages", &PageTable::pages).def_readonly("num_tokens", &PageTable::num_tokens)
      .def_readonly("prefix_hit_tokens", &PageTable::prefix_hit_tokens).def_readonly("registered_pages", &PageTable::registered_pages);
  py::class_<KvBlockManager>(m, "KvBlockManager")
      .def(py::init<uint32_t, uint32_t, bool, uint32_t>(), py::arg("total_pages"), py::arg("page_size"), py::arg("prefix_cache") = true, py::arg("radix_max_depth") = 4096)
      .def_static("with_capacity", &KvBlockManager::with_capacity, py::arg("total_kv_bytes"), py::arg("bytes_per_token"), py::arg("page_size"), py::arg("prefix_cache") = true)
      .def_property_readonly("page_size", &KvBlockManager::page_size).def_property_readonly("total_pages", &KvBlockManager::total_pages)
      .def_property_readonly("available_pages", &KvBlockManager::available_pages).def_property_readonly("in_use_pages", &KvBlockManager::in_use_pages)
      .def_property_readonly("utilization", &KvBlockManager::utilization).def_property_readonly("prefix_enabled", &KvBlockManager::prefix_enabled)
      .def_property_readonly("prefix_hit_tokens_total", &KvBlockManager::prefix_hit_tokens_total).def_property_readonly("num_requests", &KvBlockManager::num_requests)
      .def("generation_of", &KvBlockManager::generation_of).def("try_prefix_reuse", &KvBlockManager::try_prefix_reuse)
      .def("can_admit", &KvBlockManager::can_admit, py::arg("prompt"), py::arg("reserve_tokens") = 0)
      .def("admit", &KvBlockManager::admit).def("advance", &KvBlockManager::advance)
      .def("release", &KvBlockManager::release, py::arg("request_id"), py::arg("discard") = false)
      .def("mark_computed", &KvBlockManager::mark_computed).def("clear_prefix_cache", &KvBlockManager::clear_prefix_cache)
      .def("pages_for", [](const KvBlockManager& k, uint64_t id) -> py::object { auto* t = k.table(id); if (!t) return py::none(); return py::cast(t->pages); })
      .def("table", [](const KvBlockManager& k, uint64_t id) -> py::object { auto* t = k.table(id); if (!t) return py::none(); return py::cast(*t); });

  // ---- batcher ----
  py::class_<AdmissionDecision>(m, "AdmissionDecision")
      .def_property_readonly("kind", [](const AdmissionDecision& d) { return d.kind == Decision::Admit ? "admit" : d.kind == Decision::Delay ? "delay" : "reject"; })
      .def_readonly("until_ms", &AdmissionDecision::until_ms).def_readonly("reason", &AdmissionDecision::reason);
  py::class_<ContinuousBatcher>(m, "ContinuousBatcher")
      .def(py::init([](uint32_t max_batch, uint32_t chunk_tokens, double ttft_ms, double tpot_ms, double base_us, double exponent, double prefill_us,
                       KvBlockManager* kv, uint32_t max_prefill_tokens, uint32_t interleave_prefill_tokens) {
             return new ContinuousBatcher(max_batch, chunk_tokens, SloTargets{ttft_ms, tpot_ms}, LatencyEstimator{base_us, exponent, prefill_us}, kv, max_prefill_tokens,
                                          interleave_prefill_tokens);
           }),
           py::arg("max_batch"), py::arg("chunk_tokens") = 0, py::arg("ttft_ms") = 500.0, py::arg("tpot_ms") = 50.0, py::arg("decode_us_at_b1") = 8000.0,
           py::arg("batch_exponent") = 0.7, py::arg("prefill_per_token_us") = 25.0, py::arg("kv") = nullptr, py::arg("max_prefill_tokens") = 8192,
           py::arg("interleave_prefill_tokens") = 0, py::keep_alive<1, 9>())
      .def("decide", [](const ContinuousBatcher& b, uint64_t id, const std::vector<int32_t>& prompt, uint32_t max_new, uint64_t now) {
        return b.decide(IncomingRequest{id, prompt, max_new, now}, now);
      })
      .def("submit", [](ContinuousBatcher& b, uint64_t id, const std::vector<int32_t>& prompt, uint32_t max_new, uint64_t now) {
        return b.submit(IncomingRequest{id, prompt, max_new, now}, now);
      })
      .def("promote_ready", &ContinuousBatcher::promote_ready)
      .def("next_step_batch", [](ContinuousBatcher& b) {
        StepBatch s = b.next_step_batch();
        py::list pre;
        for (auto& c : s.prefill) pre.append(py::make_tuple(c.id, c.start, c.end, c.last));
        return py::make_tuple(pre, s.decode);
      })
      .def("prefill_advanced", &ContinuousBatcher::prefill_advanced)
      .def("accept_token", [](ContinuousBatcher& b, uint64_t id, int32_t tok, uint64_t now, int32_t eos) -> py::object {
        auto o = b.accept_token(id, tok, now, eos);
        if (!o) return py::none();
        return py::make_tuple(o->finished, o->generated);
      }, py::arg("id"), py::arg("token"), py::arg("now_ms"), py::arg("eos_token") = -1)
      .def("retire", &ContinuousBatcher::retire, py::arg("id"), py::arg("failed") = false).def("retire_all", &ContinuousBatcher::retire_all)
      .def("current_sequence", &ContinuousBatcher::current_sequence)
      .def("request_info", [](const ContinuousBatcher& b, uint64_t id) -> py::object {
        auto* r = b.get(id);
        if (!r) return py::none();
        py::dict d;
        d["phase"] = r->phase == Phase::Prefill ? "prefill" : r->phase == Phase::Decode ? "decode" : "finished";
        d["prefilled"] = r->prefilled; d["generated"] = r->generated; d["prompt_len"] = r->req.prompt.size(); d["max_new_tokens"] = r->req.max_new_tokens;
        d["admitted_ms"] = r->admitted_ms; d["first_token_ms"] = r->first_token_ms; d["last_token_ms"] = r->last_token_ms; d["arrival_ms"] = r->req.arrival_ms;
        d["prefix_hit_tokens"] = r->prefix_hit_tokens;
        return d;
      })
      .def("prompt", [](const ContinuousBatcher& b, uint64_t id) { auto* r = b.get(id); return r ? r->req.prompt : std::vector<int32_t>{}; })
      // position of the token each listed request feeds into its next decode step (-1 for unknown ids)
      .def("decode_positions", [](const ContinuousBatcher& b, const std::vector<uint64_t>& ids) {
        std::vector<int32_t> out;
        out.reserve(ids.size());
        for (uint64_t id : ids) {
          auto* r = b.get(id);
          out.push_back(r ? (int32_t)(r->req.prompt.size() + r->generated.size()) - 1 : -1);
        }
        return out;
      })
      // raw host addresses of int32 arrays (the runner's pinned staging buffer): no per-row Python objects on the hot path
      .def("fill_decode_inputs", [](const ContinuousBatcher& b, const std::vector<uint64_t>& ids, uintptr_t tok, uintptr_t pos, uintptr_t lens,
                                    uintptr_t bt, size_t max_blocks, size_t rows) {
        b.fill_decode_inputs(ids, reinterpret_cast<int32_t*>(tok), reinterpret_cast<int32_t*>(pos), reinterpret_cast<int32_t*>(lens),
                             reinterpret_cast<int32_t*>(bt), max_blocks, rows);
      })
      .def("accept_tokens", [](ContinuousBatcher& b, const std::vector<uint64_t>& ids, uintptr_t tokens, uint64_t now, int32_t eos) {
        auto o = b.accept_tokens(ids, reinterpret_cast<const int32_t*>(tokens), now, eos);
        std::vector<uint8_t> fin(o.size());
        std::vector<uint32_t> n(o.size());
        for (size_t i = 0; i < o.size(); ++i) { fin[i] = o[i].finished; n[i] = o[i].generated; }
        return py::make_tuple(fin, n);
      }, py::arg("ids"), py::arg("tokens_addr"), py::arg("now_ms"), py::arg("eos_token") = -1)
      .def_property_readonly("inflight_len", &ContinuousBatcher::inflight_len).def_property_readonly("queued_len", &ContinuousBatcher::queued_len)
      .def_property_readonly("rejected", &ContinuousBatcher::rejected).def_property_readonly("retired", &ContinuousBatcher::retired)
      .def_property_readonly("max_batch", &ContinuousBatcher::max_batch).def("inflight_ids", &ContinuousBatcher::inflight_ids);

  // ---- misc runtime ----
  m.def("mse", &mse);
  m.def("kl_divergence", &kl_divergence);
  m.def("log_softmax", &log_softmax);
  m.def("speculative_verify", [](const std::vector<int32_t>& t, const std::vector<std::vector<float>>& q, const std::vector<std::vector<float>>& p, const std::vector<float>& u) {
    SpecOutcome o = speculative_verify(t, q, p, u);
    return py::make_tuple(o.accepted, o.correction);
  });
  m.def("cpu_collective", [](const std::string& kind, std::vector<std::vector<float>> bufs, size_t root) {
    if (kind == "ring_allreduce") cpu_all_reduce_sum(bufs);
    else if (kind == "allgather") cpu_all_gather(bufs);
    else if (kind == "reducescatter") cpu_reduce_scatter(bufs);
    else if (kind == "alltoall") cpu_all_to_all(bufs);
    else if (kind == "broadcast") cpu_broadcast(bufs, root);
    else throw RuntimeError("unsupported collective `" + kind + "`");
    return bufs;
  }, py::arg("kind"), py::arg("bufs"), py::arg("root") = 0);
  py::class_<DriftMonitor>(m, "DriftMonitor")
      .def(py::init([](const std::vector<uint32_t>& baseline_lengths, double thr) { return new DriftMonitor(WorkloadProfile::from_lengths(baseline_lengths), thr); }))
      .def_property_readonly("threshold", &DriftMonitor::threshold)
      .def("assess", [](const DriftMonitor& d, const std::vector<uint32_t>& l) { auto a = d.assess(l); return py::make_tuple(a.kl, a.drifted, a.samples); });
  py::class_<MetricsRegistry>(m, "MetricsRegistry")
      .def(py::init<size_t>(), py::arg("capacity") = 100000)
      .def("record_step", [](MetricsRegistry& r, uint64_t step, uint32_t batch, double compute_us, double comm_us, uint32_t kv_pages) {
        r.record_step(StepMetrics{step, batch, compute_us, comm_us, kv_pages});
      })
      .def("record_request", [](MetricsRegistry& r, uint64_t id, const std::string& status, double ttft, double tpot, uint32_t hit, uint32_t out) {
        r.record_request(RequestMetrics{id, status, ttft, tpot, hit, out});
      })
      .def("count", &MetricsRegistry::count, py::arg("name"), py::arg("n") = 1)
      .def("set_gauge", &MetricsRegistry::set_gauge)
      .def("render", &MetricsRegistry::render).def("ttft_p50", &MetricsRegistry::ttft_p50).def("tpot_p99", &MetricsRegistry::tpot_p99)
      .def_property_readonly("steps_buffered", &MetricsRegistry::steps_buffered).def_property_readonly("requests_buffered", &MetricsRegistry::requests_buffered);
}
