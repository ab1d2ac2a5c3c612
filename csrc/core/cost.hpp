// Five-term placement cost model: compute + comm + memory penalty + pipeline bubble + launch
// overhead, per device, maximum over devices. Formulas follow the reference
// (crates/skein_cost/src/compute.rs:76-171,232-242; comm.rs:29-151; collectives.rs:39; memory.rs:43-229;
// bubble.rs:11; launch.rs:20-40; model.rs:62-145) with two additions for B200-class parts:
//   * a memory roofline for compute: a layer cannot finish faster than its weight (+ KV) bytes over
//     HBM bandwidth when `[hbm_gbps.<device_kind>]` is given (decode is bandwidth-bound, and that is
//     what makes narrower weight dtypes pay);
//   * `fused_overlap.<collective>`: the fraction of a collective's transfer hidden under the kernel
//     that produces its input (GEMM epilogue push), so the comm term shrinks to its exposed part.
// Both are absent from the reference's constants file; without them the model reduces to the
// reference's.
#pragma once
#include "cluster.hpp"

namespace skein {

enum class OpKind { Gemm, Attention, Elementwise };
inline const char* op_kind_name(OpKind k) { return k == OpKind::Gemm ? "gemm" : k == OpKind::Attention ? "attention" : "elementwise"; }
inline OpKind op_kind_of(LayerKind k) {
  switch (k) {
    case LayerKind::Embedding: case LayerKind::RmsNorm: return OpKind::Elementwise;
    case LayerKind::Attention: return OpKind::Attention;
    default: return OpKind::Gemm;
  }
}

enum class CollectiveKind { RingAllReduce, AllGather, ReduceScatter, AllToAll, Broadcast, SendRecv };
inline const char* collective_name(CollectiveKind k) {
  switch (k) {
    case CollectiveKind::RingAllReduce: return "ring_allreduce"; case CollectiveKind::AllGather: return "allgather";
    case CollectiveKind::ReduceScatter: return "reducescatter"; case CollectiveKind::AllToAll: return "alltoall";
    case CollectiveKind::Broadcast: return "broadcast"; case CollectiveKind::SendRecv: return "send_recv";
  }
  return "?";
}
inline double collective_factor(CollectiveKind k, size_t n) {
  const double nf = (double)n;
  switch (k) {
    case CollectiveKind::RingAllReduce: return 2.0 * (nf - 1.0) / nf;
    case CollectiveKind::AllGather: case CollectiveKind::ReduceScatter: case CollectiveKind::AllToAll: return (nf - 1.0) / nf;
    default: return 1.0;
  }
}
struct Collective {
  CollectiveKind kind;
  std::vector<size_t> participants;
  uint64_t bytes;
};

struct CostConstants {
  double launch_us_per_kernel = 7.0, overshoot_us_per_gb = 1e6;
  // Device-side fixed cost of one kernel of a decode step beyond its roofline time (ramp-up, tail and the dependent-launch
  // gap): it is paid inside a CUDA graph too, so graph coverage does not reduce it. Optional, 0 when the file has none.
  double kernel_overhead_us = 0.0;
  // Pipeline parallelism as this runtime executes a decode step: the batch goes through the stages as
  // pp x pipeline_micro_per_stage micro-batches, and (pipeline_drain) the step ends when the last of them has left the
  // last stage. 0 micro-batches per stage (no [pipeline] table) keeps the reference's form: every stage runs the whole
  // batch once and idles for (pp-1)/pp of that time.
  uint32_t pipeline_micro_per_stage = 0;
  bool pipeline_drain = true;
  std::map<std::string, double> collective_fixed_us;                 // collective -> exposed fixed cost per call beyond
                                                                     // the link latency (flag wait, rank skew); optional
  std::map<std::string, std::map<std::string, double>> peak_tflops;  // device kind -> dtype -> TFLOP/s
  std::map<std::string, std::map<std::string, double>> efficiency;   // op kind -> dtype -> fraction
  std::map<std::string, double> collective_efficiency;
  std::map<std::string, double> hbm_gbps;                            // device kind -> GB/s (optional)
  std::map<std::string, double> stream_efficiency;                   // weight dtype -> measured fraction of hbm_gbps the
                                                                     // weight-streaming kernels reach (optional, default 1)
  std::map<std::string, double> fused_overlap;                       // collective -> hidden fraction (optional)
  std::map<std::string, double> parity_tolerance_mse;
  uint32_t prefill_tokens = 1024, decode_kv_tokens = 2048;
  uint32_t memory_buckets = 100, drift_buckets = 50;
  // runtime section
  uint32_t metrics_buffer_capacity = 100000, drain_timeout_seconds = 60, prometheus_port = 9090, radix_max_depth = 4096;
  double per_token_decode_us_at_b1 = 8000.0, batch_scaling_exponent = 0.7, prefill_per_token_us = 25.0;
  Json raw;  // the parsed file, kept so that a writer can preserve entries it does not touch

  static std::map<std::string, double> table(const Json& j) {
    std::map<std::string, double> m;
    for (auto& kv : j.members()) m[kv.first] = kv.second.as_double();
    return m;
  }
  static CostConstants from_json(const Json& j) {
    CostConstants c;
    c.raw = j;
    try {
      c.launch_us_per_kernel = j.at("launch_us_per_kernel").as_double();
      c.overshoot_us_per_gb = j.at("overshoot_us_per_gb").as_double();
      if (const Json* h = j.find("kernel_overhead_us")) c.kernel_overhead_us = h->as_double();
      if (const Json* h = j.find("collective_fixed_us")) c.collective_fixed_us = table(*h);
      if (const Json* h = j.find("pipeline")) {
        c.pipeline_micro_per_stage = (uint32_t)h->at("micro_batches_per_stage").as_int();
        if (h->has("drain_per_step")) c.pipeline_drain = h->at("drain_per_step").as_int() != 0;
      }
      for (auto& kv : j.at("peak_tflops").members()) c.peak_tflops[kv.first] = table(kv.second);
      for (auto& kv : j.at("efficiency").members()) c.efficiency[kv.first] = table(kv.second);
      c.collective_efficiency = table(j.at("collective_efficiency"));
      if (const Json* h = j.find("hbm_gbps")) c.hbm_gbps = table(*h);
      if (const Json* h = j.find("stream_efficiency")) c.stream_efficiency = table(*h);
      if (const Json* h = j.find("fused_overlap")) c.fused_overlap = table(*h);
      if (const Json* h = j.find("parity_tolerance_mse")) c.parity_tolerance_mse = table(*h);
      if (const Json* r = j.find("representative_workload")) {
        c.prefill_tokens = (uint32_t)r->at("prefill_tokens").as_int();
        c.decode_kv_tokens = (uint32_t)r->at("decode_kv_tokens").as_int();
      }
      if (const Json* d = j.find("dp")) {
        c.memory_buckets = (uint32_t)d->at("memory_buckets").as_int();
        c.drift_buckets = (uint32_t)d->at("drift_buckets").as_int();
      }
      if (const Json* r = j.find("runtime")) {
        if (r->has("metrics_buffer_capacity")) c.metrics_buffer_capacity = (uint32_t)r->at("metrics_buffer_capacity").as_int();
        if (r->has("drain_timeout_seconds")) c.drain_timeout_seconds = (uint32_t)r->at("drain_timeout_seconds").as_int();
        if (r->has("prometheus_port")) c.prometheus_port = (uint32_t)r->at("prometheus_port").as_int();
        if (r->has("radix_max_depth")) c.radix_max_depth = (uint32_t)r->at("radix_max_depth").as_int();
      }
      if (const Json* r = j.find("runtime_estimator")) {
        c.per_token_decode_us_at_b1 = r->at("per_token_decode_us_at_b1").as_double();
        c.batch_scaling_exponent = r->at("batch_scaling_exponent").as_double();
        c.prefill_per_token_us = r->at("prefill_per_token_us").as_double();
      }
    } catch (const JsonError& e) {
      throw CostError(std::string("cost constants: ") + e.what());
    }
    return c;
  }
  static CostConstants from_toml_str(const std::string& s) {
    try { return from_json(parse_toml(s)); } catch (const TomlError& e) { throw CostError(std::string("cost constants: ") + e.what()); }
  }
  double peak_tflops_for(const std::string& kind, Dtype d) const {
    auto it = peak_tflops.find(kind);
    if (it == peak_tflops.end()) throw CostError("no [peak_tflops." + kind + "] table in the cost constants");
    auto jt = it->second.find(dtype_name(d));
    if (jt == it->second.end()) throw CostError(std::string("no peak_tflops for dtype ") + dtype_name(d) + " on " + kind);
    return jt->second;
  }
  double efficiency_for(OpKind op, Dtype d) const {
    auto it = efficiency.find(op_kind_name(op));
    if (it == efficiency.end()) throw CostError(std::string("no [efficiency.") + op_kind_name(op) + "] table");
    auto jt = it->second.find(dtype_name(d));
    if (jt == it->second.end()) throw CostError(std::string("no efficiency for dtype ") + dtype_name(d));
    return jt->second;
  }
  double collective_eff(CollectiveKind k) const {
    auto it = collective_efficiency.find(collective_name(k));
    if (it == collective_efficiency.end()) throw CostError(std::string("no collective_efficiency.") + collective_name(k));
    return it->second;
  }
  double tolerance_mse(Dtype d) const {
    auto it = parity_tolerance_mse.find(dtype_name(d));
    return it == parity_tolerance_mse.end() ? 1e-3 : it->second;
  }
};

struct WorkloadCtx {
  uint32_t batch = 1, seq_len = 1, kv_len = 2048;
  static WorkloadCtx decode_step(const Plan& p, const CostConstants& c) { return {p.batching.max_batch, 1, c.decode_kv_tokens}; }
};

inline Dtype plan_weight_dtype(const Plan& p, std::optional<size_t> b) { return b && *b < p.dtype_map.size() ? p.dtype_map[*b].weight : Dtype::Bf16; }
inline Dtype plan_act_dtype(const Plan& p, std::optional<size_t> b) { return b && *b < p.dtype_map.size() ? p.dtype_map[*b].activation : Dtype::Bf16; }
inline Dtype plan_kv_dtype(const Plan& p, std::optional<size_t> b) { return b && *b < p.dtype_map.size() ? p.dtype_map[*b].kv_cache : Dtype::Bf16; }

inline uint64_t layer_flops(const Layer& l, const ModelMeta& meta, const WorkloadCtx& wl) {
  const uint64_t b = wl.batch, s = wl.seq_len, k = wl.kv_len;
  switch (l.kind) {
    case LayerKind::Embedding: return b * s * l.hidden;
    case LayerKind::RmsNorm: return 5 * b * s * l.hidden;
    case LayerKind::Attention: {
      const uint64_t hidden = meta.hidden, q = l.num_heads * l.head_dim, kv = l.num_kv_heads * l.head_dim;
      const uint64_t qkvo = 2 * b * s * (q + kv + kv + q) * hidden;
      const uint64_t scores = 2 * b * l.num_heads * s * k * l.head_dim;
      const uint64_t softmax = 3 * b * l.num_heads * s * k;
      return qkvo + scores + softmax + scores;
    }
    case LayerKind::Mlp: return 6 * b * s * l.hidden * l.intermediate;
    case LayerKind::Moe: return 2 * b * s * l.hidden * l.num_experts + 6 * b * s * l.top_k * l.hidden * l.intermediate;
    case LayerKind::Lmhead: return 2 * b * s * l.vocab * l.hidden;
  }
  return 0;
}

inline uint64_t compute_divisor(LayerKind k, const Placement& pl) {
  switch (k) {
    case LayerKind::Moe: return (uint64_t)pl.tp * pl.ep;
    case LayerKind::RmsNorm: return 1;
    default: return pl.tp;
  }
}

inline uint64_t layer_param_elems(const Layer& l) { uint64_t n = 0; for (auto& p : l.params) n += p.numel(); return n; }

// Bytes a decode step must stream for this layer on one device (weights touched + KV read).
// Pure expert parallelism runs attention data-parallel: every expert-parallel rank attends over its own 1/ep of the
// step's sequences with the whole (replicated) attention weights, and the MoE blocks exchange tokens. With tensor or
// pipeline parallelism beside it the attention is replicated across the expert-parallel ranks instead.
inline uint64_t attention_dp_ways(const Placement& pl) { return (pl.ep > 1 && pl.tp == 1 && pl.pp == 1) ? pl.ep : 1; }

inline double layer_stream_bytes(const Layer& l, const ModelMeta& meta, Dtype wd, Dtype kvd, const Placement& pl, const WorkloadCtx& wl) {
  const double div = (double)std::max<uint64_t>(1, compute_divisor(l.kind, pl));
  double elems = (double)layer_param_elems(l);
  if (l.kind == LayerKind::Embedding) elems = (double)wl.batch * wl.seq_len * l.hidden;  // only the gathered rows
  if (l.kind == LayerKind::Moe && l.num_experts > 0) {
    // experts actually touched by batch*top_k routed tokens (uniform routing): E * (1 - (1 - 1/E)^(b*k))
    const double E = (double)l.num_experts, draws = (double)wl.batch * wl.seq_len * l.top_k;
    const double touched = E * (1.0 - std::pow(1.0 - 1.0 / E, draws));
    elems *= touched / E;
  }
  double bytes = (double)dtype_bits(wd) / 8.0 * elems / div;
  if (l.kind == LayerKind::Attention)
    bytes += (double)dtype_bits(kvd) / 8.0 * 2.0 * l.num_kv_heads * l.head_dim * (double)wl.kv_len * wl.batch /
             (double)(pl.tp * attention_dp_ways(pl));
  (void)meta;
  return bytes;
}

inline double compute_time_with_dtype(const Layer& l, const ModelMeta& meta, Dtype wd, Dtype kvd, const Placement& pl,
                                      const Cluster& cl, const CostConstants& c, const WorkloadCtx& wl, size_t device) {
  const double flops = (double)layer_flops(l, meta, wl);
  const std::string& kind = cl.device_kind(device);
  const double peak = c.peak_tflops_for(kind, wd);
  const double eff = c.efficiency_for(op_kind_of(l.kind), wd);
  double div = (double)std::max<uint64_t>(1, compute_divisor(l.kind, pl));
  if (l.kind == LayerKind::Attention || l.kind == LayerKind::Lmhead) div *= (double)attention_dp_ways(pl);   // 1/ep of the rows
  double t = flops / (peak * 1e12 * eff * div) * 1e6;
  auto hb = c.hbm_gbps.find(kind);
  if (hb != c.hbm_gbps.end() && hb->second > 0) {
    // a narrower weight type moves fewer bytes but its kernel may reach a smaller share of the copy bandwidth (the e4m3
    // tiles are rescaled to bf16 on their way to the tensor cores): the measured share per weight dtype decides whether
    // the dtype map gains time or only memory
    auto share = [&](Dtype d) {
      auto se = c.stream_efficiency.find(dtype_name(d));
      return (se != c.stream_efficiency.end() && se->second > 0) ? se->second : 1.0;
    };
    // the share belongs to the kernel that streams the bytes: the weight dtype's for the weights, the attention kernel's
    // (bf16 rate) for the KV cache of an attention layer
    double kv_bytes = 0;
    if (l.kind == LayerKind::Attention)
      kv_bytes = (double)dtype_bits(kvd) / 8.0 * 2.0 * l.num_kv_heads * l.head_dim * (double)wl.kv_len * wl.batch /
                 (double)(pl.tp * attention_dp_ways(pl));
    const double w_bytes = layer_stream_bytes(l, meta, wd, kvd, pl, wl) - kv_bytes;
    t = std::max(t, (w_bytes / share(wd) + kv_bytes / share(Dtype::Bf16)) / (hb->second * 1e9) * 1e6);
  }
  return t;
}

inline bool layer_on_stage(const Layer& l, size_t num_blocks, const Placement& pl, uint32_t stage, bool final_norm_last) {
  if (l.block_idx) return block_to_stage(*l.block_idx, num_blocks, pl.pp) == stage;
  switch (l.kind) {
    case LayerKind::Embedding: return stage == 0;
    case LayerKind::Lmhead: return stage == pl.pp - 1;
    case LayerKind::RmsNorm: return final_norm_last ? stage == pl.pp - 1 : stage == 0;
    default: return stage == 0;
  }
}

inline double block_compute_time(size_t block, const Graph& ir, Dtype wd, Dtype kvd, const Placement& pl, const Cluster& cl,
                                 const CostConstants& c, const WorkloadCtx& wl, size_t device) {
  double t = 0;
  for (auto& l : ir.layers) if (l.block_idx && *l.block_idx == block) t += compute_time_with_dtype(l, ir.meta, wd, kvd, pl, cl, c, wl, device);
  return t;
}

// Kernels launched per layer by this runtime's fused decode path (the reference counts 7 / 3 / 3+top_k
// for its unfused graph: crates/skein_cost/src/compute.rs:232-242).
inline uint32_t kernels_per_layer(const Layer& l) {
  switch (l.kind) {
    case LayerKind::Attention: return 4;  // qkv GEMM, RoPE + KV append + attention, o_proj GEMM, reduce + norm (+ router)
    case LayerKind::Mlp: return 3;        // gate/up GEMM (SwiGLU epilogue), down GEMM, reduce+norm
    case LayerKind::Moe: return 3;        // grouped gate/up (gathers its rows), grouped down, combine + norm
    case LayerKind::RmsNorm: return 0;    // fused into the reduce kernels above
    default: return 1;
  }
}

inline uint32_t kernels_per_step_on_device(const Graph& ir, const Plan& plan, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  if (!pl.holds(device)) return 0;
  uint32_t total = 0;
  for (auto& l : ir.layers) if (layer_on_stage(l, ir.meta.num_layers, pl, pl.stage_of(device), false)) total += kernels_per_layer(l);
  return total + 3;  // first norm, sampling, state advance
}

inline double comm_time(const Collective& col, const Cluster& cl, const CostConstants& c) {
  if (col.participants.size() < 2) throw CostError(std::string("degenerate collective ") + collective_name(col.kind));
  const PathInfo path = cl.collective_path(col.participants);
  const double factor = collective_factor(col.kind, col.participants.size());
  const double eff = c.collective_eff(col.kind);
  double transfer = 0;
  if (std::isfinite(path.min_bandwidth_gbps)) transfer = factor * (double)col.bytes / (path.min_bandwidth_gbps * eff * 1e9) * 1e6;
  auto ov = c.fused_overlap.find(collective_name(col.kind));
  if (ov != c.fused_overlap.end()) transfer *= std::max(0.0, 1.0 - ov->second);
  auto fx = c.collective_fixed_us.find(collective_name(col.kind));
  return path.total_latency_us + transfer + (fx == c.collective_fixed_us.end() ? 0.0 : fx->second);
}

inline std::vector<Collective> collectives_on_device(const Plan& plan, const Graph& ir, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  std::vector<Collective> out;
  if (!pl.holds(device)) return out;
  const uint32_t stage = pl.stage_of(device);
  const size_t nb = ir.meta.num_layers;
  const uint64_t hidden = ir.meta.hidden, mb = plan.batching.max_batch;
  if (pl.tp > 1) {
    auto grp = pl.tp_group(device);
    for (auto& l : ir.layers) {
      if (!l.block_idx || block_to_stage(*l.block_idx, nb, pl.pp) != stage) continue;
      if (l.kind == LayerKind::Attention || l.kind == LayerKind::Mlp || l.kind == LayerKind::Moe)
        out.push_back({CollectiveKind::RingAllReduce, grp, dtype_bytes_for(plan_act_dtype(plan, l.block_idx), mb * hidden)});
    }
  }
  if (pl.ep > 1) {
    auto grp = pl.ep_group(device);
    for (auto& l : ir.layers) {
      if (!l.block_idx || block_to_stage(*l.block_idx, nb, pl.pp) != stage || l.kind != LayerKind::Moe) continue;
      // dispatch and combine; under data-parallel attention a rank sends only its own rows' copies
      const uint64_t bytes = dtype_bytes_for(plan_act_dtype(plan, l.block_idx), mb * l.top_k * hidden) / attention_dp_ways(pl);
      out.push_back({CollectiveKind::AllToAll, grp, bytes});
      out.push_back({CollectiveKind::AllToAll, grp, bytes});
    }
  }
  if (pl.pp > 1 && stage < pl.pp - 1) {
    auto grp = pl.pp_group(device);
    out.push_back({CollectiveKind::SendRecv, {device, grp[stage + 1]}, dtype_bytes_for(plan_act_dtype(plan, 0), mb * hidden)});
  }
  return out;
}

// ---- memory -------------------------------------------------------------------------------------------
inline uint64_t layer_weight_bytes(const Layer& l, Dtype wd, const Placement& pl) {
  uint64_t raw = 0;
  for (auto& p : l.params) raw += dtype_bytes_for(wd, p.numel());
  return raw / std::max<uint64_t>(1, compute_divisor(l.kind, pl));
}
inline uint64_t weight_bytes_on_device(const Plan& plan, const Graph& ir, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  if (!pl.holds(device)) return 0;
  uint64_t t = 0;
  for (auto& l : ir.layers)
    if (layer_on_stage(l, ir.meta.num_layers, pl, pl.stage_of(device), true)) t += layer_weight_bytes(l, plan_weight_dtype(plan, l.block_idx), pl);
  return t;
}
inline uint64_t kv_bytes_on_device(const Plan& plan, const Graph& ir, const CostConstants& c, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  if (!pl.holds(device)) return 0;
  const uint64_t per_seq = 2ull * ir.meta.num_kv_heads * ir.meta.head_dim * c.decode_kv_tokens;
  uint64_t t = 0;
  for (size_t b = 0; b < ir.meta.num_layers; ++b)
    if (block_to_stage(b, ir.meta.num_layers, pl.pp) == pl.stage_of(device)) t += dtype_bytes_for(plan_kv_dtype(plan, b), per_seq) * plan.batching.max_batch;
  return (plan.kv.kv_sharded && pl.tp > 1) ? t / pl.tp : t;
}
inline uint64_t activation_bytes_on_device(const Plan& plan, const Graph& ir, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  if (!pl.holds(device)) return 0;
  const Dtype dt = plan.dtype_map.empty() ? Dtype::Bf16 : plan.dtype_map[0].activation;
  return 4 * dtype_bytes_for(dt, (uint64_t)plan.batching.max_batch * ir.meta.hidden);
}
inline uint64_t peak_memory_bytes(const Plan& plan, const Graph& ir, const CostConstants& c, size_t device) {
  return weight_bytes_on_device(plan, ir, device) + kv_bytes_on_device(plan, ir, c, device) + activation_bytes_on_device(plan, ir, device);
}
inline uint64_t block_weight_bytes(size_t block, const Graph& ir, Dtype wd, const Placement& pl) {
  uint64_t t = 0;
  for (auto& l : ir.layers) if (l.block_idx && *l.block_idx == block) t += layer_weight_bytes(l, wd, pl);
  return t;
}
inline uint64_t block_kv_bytes(const Graph& ir, Dtype kvd, const Placement& pl, const WorkloadCtx& wl, bool kv_sharded) {
  const uint64_t bytes = dtype_bytes_for(kvd, 2ull * ir.meta.num_kv_heads * ir.meta.head_dim * wl.kv_len * wl.batch);
  return (kv_sharded && pl.tp > 1) ? bytes / pl.tp : bytes;
}
inline uint64_t non_decoder_weight_bytes(const Graph& ir, const Placement& pl) {
  uint64_t t = 0;
  for (auto& l : ir.layers) if (!l.block_idx) t += layer_weight_bytes(l, Dtype::Bf16, pl);
  return t;
}
inline double memory_penalty(const Plan& plan, const Graph& ir, const Cluster& cl, const CostConstants& c, size_t device) {
  const uint64_t peak = peak_memory_bytes(plan, ir, c, device), cap = cl.device_memory_bytes(device);
  return peak <= cap ? 0.0 : (double)(peak - cap) / 1e9 * c.overshoot_us_per_gb;
}

// ---- bubble, launch ---------------------------------------------------------------------------------------
inline double bubble_time(const Plan& plan, double stage_compute_us) {
  const double pp = std::max(1u, plan.parallelism.pp);
  return pp <= 1.0 ? 0.0 : (pp - 1.0) / pp * stage_compute_us;
}
inline double cuda_graph_coverage(const Plan& plan) {
  if (!plan.execution.cuda_graphs) return 0.0;
  switch (plan.batching.kind) {
    case BatchKind::Static: return 1.0;
    case BatchKind::Continuous: return plan.execution.capture_classes.size() >= 4 ? 0.95 : 0.7;
    case BatchKind::ContinuousChunked: return 0.4;
  }
  return 0.0;
}
inline double launch_overhead(const Plan& plan, const CostConstants& c, uint32_t kernels) {
  return kernels * (c.launch_us_per_kernel * (1.0 - cuda_graph_coverage(plan)) + c.kernel_overhead_us);
}

// ---- the model ------------------------------------------------------------------------------------------------
struct CostBreakdown { double compute = 0, comm = 0, memory = 0, bubble = 0, launch = 0; double total() const { return compute + comm + memory + bubble + launch; } };

class CostModel {
 public:
  explicit CostModel(CostConstants c) : c_(std::move(c)) {}
  const CostConstants& constants() const { return c_; }

  double compute_on_device(const Plan& plan, const Graph& ir, const Cluster& cl, const WorkloadCtx& wl, size_t device) const {
    const Placement pl = Placement::from_plan(plan);
    if (!pl.holds(device)) return 0;
    double t = 0;
    for (auto& l : ir.layers)
      if (layer_on_stage(l, ir.meta.num_layers, pl, pl.stage_of(device), false))
        t += compute_time_with_dtype(l, ir.meta, plan_weight_dtype(plan, l.block_idx), plan_kv_dtype(plan, l.block_idx), pl, cl, c_, wl, device);
    return t;
  }
  CostBreakdown per_device(const Plan& plan, const Graph& ir, const Cluster& cl, const WorkloadCtx& wl, size_t device) const {
    CostBreakdown b;
    if (!Placement::from_plan(plan).holds(device)) return b;
    const uint32_t pp = std::max(1u, plan.parallelism.pp);
    if (pp > 1 && c_.pipeline_micro_per_stage > 0) {
      // M micro-batches of batch / M rows each cross this stage one after the other; a step that drains ends pp - 1
      // stage times after the first stage has sent its last one
      const uint32_t M = std::max(1u, std::min(pp * c_.pipeline_micro_per_stage, wl.batch));
      Plan mp = plan;
      mp.batching.max_batch = (wl.batch + M - 1) / M;
      WorkloadCtx mwl = wl;
      mwl.batch = mp.batching.max_batch;
      const double stage = compute_on_device(mp, ir, cl, mwl, device);
      double comm = 0;
      for (auto& col : collectives_on_device(mp, ir, device)) comm += comm_time(col, cl, c_);
      const double launch = launch_overhead(plan, c_, kernels_per_step_on_device(ir, plan, device));
      b.compute = M * stage;
      b.comm = M * comm;
      b.launch = M * launch;
      b.bubble = c_.pipeline_drain ? (pp - 1.0) * (stage + comm + launch) : 0.0;
      b.memory = memory_penalty(plan, ir, cl, c_, device);
      return b;
    }
    b.compute = compute_on_device(plan, ir, cl, wl, device);
    for (auto& col : collectives_on_device(plan, ir, device)) b.comm += comm_time(col, cl, c_);
    b.memory = memory_penalty(plan, ir, cl, c_, device);
    b.bubble = bubble_time(plan, b.compute);
    b.launch = launch_overhead(plan, c_, kernels_per_step_on_device(ir, plan, device));
    return b;
  }
  double total_cost(const Plan& plan, const Graph& ir, const Cluster& cl) const {
    if (plan.dtype_map.size() != ir.meta.num_layers)
      throw CostError("dtype_map has " + std::to_string(plan.dtype_map.size()) + " entries, model has " + std::to_string(ir.meta.num_layers) + " layers");
    if (Placement::from_plan(plan).devices() > cl.num_devices()) throw CostError("plan uses more devices than the cluster has");
    const WorkloadCtx wl = WorkloadCtx::decode_step(plan, c_);
    double mx = 0;
    for (size_t d = 0; d < cl.num_devices(); ++d) mx = std::max(mx, per_device(plan, ir, cl, wl, d).total());
    return mx;
  }

 private:
  CostConstants c_;
};

}  // namespace skein
