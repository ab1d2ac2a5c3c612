// Lowering of a plan to per-device structure: shard roles of every parameter, the ordered list of
// collectives (topology.json), per-device segments (the regions between collectives, each of which
// the runtime captures into its CUDA graph) with named hand-off tensors, the per-device schedule, and
// the weight manifest (io.json).
//
// Mirrors the reference's emit crate (crates/skein_emit/src/shard_role.rs:35-166, topology.rs:26-54,
// handoff.rs:23-211, segment.rs:55-87, io_manifest.rs:17-45, lib.rs:58-71), with the differences this
// runtime has: expert parallelism is token-routed (all-to-all dispatch and combine, as the
// reference's cost model and docs describe but its executor rejects), experts are owned in contiguous
// blocks, and sampling exchanges (value, index) candidates. The embedding table is vocabulary-parallel as in the
// reference (its lookups are summed by an all-reduce that the first RMSNorm carries).
#pragma once
#include "cost.hpp"

namespace skein {

// ---- shard roles ------------------------------------------------------------------------------------------
enum class ParamKind { Replicated, ColumnParallel, RowParallel, Expert };
struct ParamRole {
  ParamKind kind = ParamKind::Replicated;
  int expert_idx = -1;        // Expert
  bool expert_column = true;  // Expert: w1/w3 are column-parallel inside the expert, w2 row-parallel
};

inline ParamRole param_kind_for(const std::string& name) {
  auto has = [&](const char* s) { return name.find(s) != std::string::npos; };
  ParamRole r;
  const size_t ex = name.find(".experts.");
  if (ex != std::string::npos) {
    r.kind = ParamKind::Expert;
    r.expert_idx = std::atoi(name.c_str() + ex + 9);
    r.expert_column = !has(".w2.");
    return r;
  }
  if (has("q_proj") || has("k_proj") || has("v_proj") || has("gate_proj") || has("up_proj") || has("lm_head") || has("embed_tokens")) r.kind = ParamKind::ColumnParallel;
  else if (has("o_proj") || has("down_proj")) r.kind = ParamKind::RowParallel;
  return r;  // norms, router gate: replicated (the embedding table is split by vocabulary rows like lm_head)
}

struct ShardSlice {
  bool present = false;          // this device holds (part of) the parameter
  int axis = -1;                 // -1 whole tensor, 0 = rows (outer, contiguous), 1 = columns (row-strided)
  uint64_t start = 0, len = 0;   // along `axis`
  std::vector<uint64_t> shape;   // shape of the shard
};

// Priority: pipeline stage, then expert ownership, then tensor parallelism.
inline ShardSlice shard_of(const Param& p, const Layer& l, const ModelMeta& meta, const Placement& pl, size_t device) {
  ShardSlice s;
  if (!pl.holds(device)) return s;
  const uint32_t stage = pl.stage_of(device);
  if (!layer_on_stage(l, meta.num_layers, pl, stage, true)) return s;
  const ParamRole role = param_kind_for(p.name);
  s.shape = p.shape;
  const uint32_t tpi = pl.tp_idx(device);
  auto split = [&](int axis) {
    const uint64_t n = p.shape[axis];
    const uint64_t per = (n + pl.tp - 1) / pl.tp;
    s.axis = axis; s.start = std::min<uint64_t>(n, per * tpi); s.len = std::min<uint64_t>(per, n - s.start);
    s.shape[axis] = s.len;
  };
  s.present = true;
  switch (role.kind) {
    case ParamKind::Replicated: break;
    case ParamKind::ColumnParallel: if (pl.tp > 1) split(0); break;
    case ParamKind::RowParallel: if (pl.tp > 1) split(1); break;
    case ParamKind::Expert: {
      const uint32_t per_rank = (uint32_t)(*meta.num_experts / pl.ep);
      if ((uint32_t)role.expert_idx / per_rank != pl.ep_idx(device)) { s.present = false; return s; }
      if (pl.tp > 1) split(role.expert_column ? 0 : 1);
      break;
    }
  }
  return s;
}

// ---- topology ------------------------------------------------------------------------------------------------
struct TopologyEntry {
  uint64_t sequence_idx;
  std::string kind;                  // ring_allreduce | alltoall | send_recv | allgather
  std::vector<size_t> participants;
  std::string tensor_name, after_node, dtype;
  std::vector<uint64_t> shape;
  bool fused = false;                // carried inside the producing/consuming kernels (no stand-alone launch)
};

inline std::vector<size_t> tp_group_of_stage(uint32_t stage, uint32_t ep_idx, const Placement& pl) { return pl.tp_group(((size_t)stage * pl.ep + ep_idx) * pl.tp); }
inline std::vector<size_t> ep_group_of_stage(uint32_t stage, uint32_t tp_idx, const Placement& pl) { return pl.ep_group((size_t)stage * pl.ep * pl.tp + tp_idx); }

inline std::vector<TopologyEntry> emit_topology(const Plan& plan, const Graph& ir) {
  const Placement pl = Placement::from_plan(plan);
  const uint64_t H = ir.meta.hidden, B = plan.batching.max_batch;
  std::vector<TopologyEntry> out;
  uint64_t seq = 0;
  auto add = [&](const char* kind, std::vector<size_t> parts, std::string tensor, std::vector<uint64_t> shape, Dtype dt, std::string after, bool fused) {
    out.push_back({seq++, kind, std::move(parts), std::move(tensor), std::move(after), dtype_name(dt), std::move(shape), fused});
  };
  if (pl.tp > 1)
    for (uint32_t e = 0; e < pl.ep; ++e)
      add("ring_allreduce", tp_group_of_stage(0, e, pl), "embed_out", {B, 1, H}, plan_act_dtype(plan, 0), "embed_tokens", true);
  for (size_t b = 0; b < ir.meta.num_layers; ++b) {
    const uint32_t stage = block_to_stage(b, ir.meta.num_layers, pl.pp);
    const Dtype ad = plan_act_dtype(plan, b);
    if (pl.pp > 1 && stage > 0 && (b == 0 || block_to_stage(b - 1, ir.meta.num_layers, pl.pp) != stage))
      for (uint32_t i = 0; i < pl.tp * pl.ep; ++i)
        add("send_recv", {(size_t)(stage - 1) * pl.tp * pl.ep + i, (size_t)stage * pl.tp * pl.ep + i}, "block_" + std::to_string(b) + "_pp_boundary",
            {B, 1, H}, ad, "stage_" + std::to_string(stage - 1) + "_to_" + std::to_string(stage), false);
    bool moe = false, ffn = false;
    size_t topk = 1;
    for (auto& l : ir.layers) if (l.block_idx && *l.block_idx == b) { if (l.kind == LayerKind::Moe) { moe = ffn = true; topk = l.top_k; } if (l.kind == LayerKind::Mlp) ffn = true; }
    for (uint32_t e = 0; e < pl.ep; ++e)
      if (pl.tp > 1) add("ring_allreduce", tp_group_of_stage(stage, e, pl), "block_" + std::to_string(b) + "_attn_out", {B, 1, H}, ad, "block_" + std::to_string(b) + "_o_proj", true);
    if (pl.ep > 1 && moe)
      for (uint32_t t = 0; t < pl.tp; ++t) {
        add("alltoall", ep_group_of_stage(stage, t, pl), "block_" + std::to_string(b) + "_moe_dispatch", {B, topk, H}, ad, "block_" + std::to_string(b) + "_router", true);
        add("alltoall", ep_group_of_stage(stage, t, pl), "block_" + std::to_string(b) + "_moe_combine", {B, topk, H}, ad, "block_" + std::to_string(b) + "_expert_out", true);
      }
    if (pl.tp > 1 && ffn)
      for (uint32_t e = 0; e < pl.ep; ++e)
        add("ring_allreduce", tp_group_of_stage(stage, e, pl), "block_" + std::to_string(b) + "_ffn_out", {B, 1, H}, ad, "block_" + std::to_string(b) + "_down_proj", true);
  }
  if (pl.tp > 1)
    for (uint32_t e = 0; e < pl.ep; ++e)
      add("allgather", tp_group_of_stage(pl.pp - 1, e, pl), "logit_candidates", {B, 2}, Dtype::F32, "lm_head", true);
  return out;
}

inline Json topology_to_json(const std::vector<TopologyEntry>& t, const Plan& plan) {
  Json arr = Json::array();
  for (auto& e : t) {
    Json parts = Json::array(), shape = Json::array();
    for (auto p : e.participants) parts.push(p);
    for (auto s : e.shape) shape.push(s);
    arr.push(Json::object().set("sequence_idx", e.sequence_idx).set("kind", e.kind).set("participants", parts).set("tensor_name", e.tensor_name)
                 .set("shape", shape).set("dtype", e.dtype).set("after_node", e.after_node).set("fused", e.fused));
  }
  Json kvt = Json();
  if (plan.disaggregation) kvt = Json::object().set("kind", kv_transfer_name(plan.disaggregation->mode)).set("layer_overlap", plan.disaggregation->layer_overlap);
  return Json::object().set("collectives", arr).set("kv_transfer", kvt);
}

// ---- segments and per-device schedule ------------------------------------------------------------------------------
// Hand-off tensor names (crates/skein_emit/src/handoff.rs:23-66).
inline std::string handoff_input_tokens() { return "input_tokens"; }
inline std::string handoff_embed_out() { return "embed_out"; }
inline std::string handoff_logits() { return "logits"; }
inline std::string handoff_carry_pre_block(size_t b) { return "carry_pre_block_" + std::to_string(b); }
inline std::string handoff_carry_post_attn(size_t b) { return "carry_post_attn_" + std::to_string(b); }
inline std::string handoff_collective_attn_out(size_t b) { return "collective_attn_out_" + std::to_string(b); }
inline std::string handoff_collective_ffn_out(size_t b) { return "collective_ffn_out_" + std::to_string(b); }
inline std::string handoff_moe_dispatch(size_t b) { return "collective_moe_dispatch_" + std::to_string(b); }
inline std::string handoff_moe_combine(size_t b) { return "collective_moe_combine_" + std::to_string(b); }

struct Segment {
  size_t idx;
  std::string name;
  std::vector<std::string> inputs, outputs, ops;
};
struct SequenceStep {
  std::string kind;  // execute_segment | collective | moe_route
  size_t segment = 0;
  std::string collective_kind, tensor;
  std::vector<size_t> participants;
};
struct LoweredDevice {
  size_t device = 0;
  std::vector<Segment> segments;
  std::vector<SequenceStep> sequencing;
};

// One segment between every two collectives that involve this device (segments = collectives + 1).
inline LoweredDevice lower_device(const Plan& plan, const Graph& ir, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  LoweredDevice d;
  d.device = device;
  if (!pl.holds(device)) return d;
  const uint32_t stage = pl.stage_of(device);
  Segment cur{0, "segment_0", {}, {}, {}};
  auto cut = [&](const std::string& kind, const std::string& tensor, std::vector<size_t> parts) {
    cur.outputs.push_back(tensor);
    d.sequencing.push_back({"execute_segment", cur.idx, "", "", {}});
    d.sequencing.push_back({"collective", 0, kind, tensor, std::move(parts)});
    d.segments.push_back(cur);
    cur = Segment{d.segments.size(), "segment_" + std::to_string(d.segments.size()), {tensor}, {}, {}};
  };
  bool first_on_stage = true;
  if (stage == 0) {
    cur.inputs.push_back(handoff_input_tokens());
    cur.ops.push_back("embed_tokens");
    // vocabulary-parallel table: the ranks' lookups are summed before the first norm
    if (pl.tp > 1) cut("ring_allreduce", handoff_embed_out(), pl.tp_group(device));
  }
  for (size_t b = 0; b < ir.meta.num_layers; ++b) {
    if (block_to_stage(b, ir.meta.num_layers, pl.pp) != stage) continue;
    if (first_on_stage && stage > 0) {
      // the carry arrives from the previous stage before any compute of this stage
      d.sequencing.push_back({"collective", 0, "send_recv", handoff_carry_pre_block(b), {device - (size_t)pl.tp * pl.ep, device}});
      cur.inputs.push_back(handoff_carry_pre_block(b));
    }
    first_on_stage = false;
    bool moe = false;
    for (auto& l : ir.layers) if (l.block_idx && *l.block_idx == b && l.kind == LayerKind::Moe) moe = true;
    const std::string bs = "block_" + std::to_string(b);
    cur.ops.insert(cur.ops.end(), {bs + "_input_layernorm", bs + "_qkv_proj", bs + "_rope_kv_append", bs + "_attention", bs + "_o_proj"});
    if (pl.tp > 1) cut("ring_allreduce", handoff_collective_attn_out(b), pl.tp_group(device));
    cur.ops.push_back(bs + "_post_attention_layernorm");
    if (moe) {
      cur.ops.push_back(bs + "_router");
      d.sequencing.push_back({"moe_route", cur.idx, "", bs + "_router", {}});
      if (pl.ep > 1) cut("alltoall", handoff_moe_dispatch(b), pl.ep_group(device));
      cur.ops.insert(cur.ops.end(), {bs + "_experts_gate_up", bs + "_experts_down"});
      if (pl.ep > 1) cut("alltoall", handoff_moe_combine(b), pl.ep_group(device));
    } else {
      cur.ops.insert(cur.ops.end(), {bs + "_gate_up_proj", bs + "_down_proj"});
    }
    if (pl.tp > 1) cut("ring_allreduce", handoff_collective_ffn_out(b), pl.tp_group(device));
  }
  if (stage == pl.pp - 1) {
    cur.ops.insert(cur.ops.end(), {"norm", "lm_head", "sample"});
    if (pl.tp > 1) cut("allgather", "logit_candidates", pl.tp_group(device));
    cur.outputs.push_back(handoff_logits());
  } else {
    size_t next_first = 0;
    for (size_t b = 0; b < ir.meta.num_layers; ++b) if (block_to_stage(b, ir.meta.num_layers, pl.pp) == stage + 1) { next_first = b; break; }
    cur.outputs.push_back(handoff_carry_pre_block(next_first));
    d.sequencing.push_back({"execute_segment", cur.idx, "", "", {}});
    d.sequencing.push_back({"collective", 0, "send_recv", handoff_carry_pre_block(next_first), {device, device + (size_t)pl.tp * pl.ep}});
    d.segments.push_back(cur);
    return d;
  }
  d.sequencing.push_back({"execute_segment", cur.idx, "", "", {}});
  d.segments.push_back(cur);
  return d;
}

inline Json lowered_to_json(const LoweredDevice& d) {
  auto strs = [](const std::vector<std::string>& v) { Json a = Json::array(); for (auto& s : v) a.push(s); return a; };
  Json segs = Json::array(), seqj = Json::array();
  for (auto& s : d.segments)
    segs.push(Json::object().set("idx", s.idx).set("name", s.name).set("inputs", strs(s.inputs)).set("outputs", strs(s.outputs)).set("ops", strs(s.ops)));
  for (auto& st : d.sequencing) {
    Json parts = Json::array();
    for (auto p : st.participants) parts.push(p);
    Json o = Json::object().set("kind", st.kind);
    if (st.kind == "execute_segment") o.set("segment", st.segment);
    else if (st.kind == "collective") o.set("collective", st.collective_kind).set("tensor", st.tensor).set("participants", parts);
    else o.set("segment", st.segment).set("tensor", st.tensor);
    seqj.push(o);
  }
  return Json::object().set("device", d.device).set("segments", segs).set("sequencing", seqj);
}

// ---- weight manifest (io.json) -----------------------------------------------------------------------------------------
inline Json io_manifest(const Plan& plan, const Graph& ir, size_t device) {
  const Placement pl = Placement::from_plan(plan);
  Json ts = Json::array();
  for (auto& l : ir.layers)
    for (auto& p : l.params) {
      ShardSlice s = shard_of(p, l, ir.meta, pl, device);
      if (!s.present) continue;
      Json shape = Json::array();
      for (auto v : s.shape) shape.push(v);
      ts.push(Json::object().set("name", p.name).set("shape", shape).set("dtype", dtype_name(plan_weight_dtype(plan, l.block_idx) == Dtype::Bf16 || !l.block_idx ? Dtype::Bf16 : plan_weight_dtype(plan, l.block_idx)))
                  .set("kind", "weight").set("axis", s.axis).set("start", s.start).set("len", s.len));
    }
  return Json::object().set("tensors", ts);
}

}  // namespace skein
