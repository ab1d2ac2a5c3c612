// Core types: dtypes, the model IR (a flat list of typed layers with HuggingFace parameter names),
// the Plan (TP x PP x EP placement, KV layout, batch policy, per-layer dtype map, execution config)
// and their JSON forms. Field names and enum spellings follow the reference's serde output
// (crates/skein_ir/src/types.rs:25-266, ir.rs:22-183, plan.rs:20-140) so that a plan.json written by
// either implementation reads in the other.
#pragma once
#include "blake3.hpp"
#include "json.hpp"
#include <optional>

namespace skein {

struct PlanError : std::runtime_error { using std::runtime_error::runtime_error; };
struct ImportError : std::runtime_error { using std::runtime_error::runtime_error; };

// ---- dtypes ------------------------------------------------------------------------------------
enum class Dtype { F32, Bf16, Fp16, Fp8E4m3, Fp8E5m2, Int8, Int4 };
inline const char* dtype_name(Dtype d) {
  switch (d) {
    case Dtype::F32: return "f32"; case Dtype::Bf16: return "bf16"; case Dtype::Fp16: return "fp16";
    case Dtype::Fp8E4m3: return "fp8_e4m3"; case Dtype::Fp8E5m2: return "fp8_e5m2";
    case Dtype::Int8: return "int8"; case Dtype::Int4: return "int4";
  }
  return "?";
}
inline Dtype dtype_from(const std::string& s) {
  for (Dtype d : {Dtype::F32, Dtype::Bf16, Dtype::Fp16, Dtype::Fp8E4m3, Dtype::Fp8E5m2, Dtype::Int8, Dtype::Int4})
    if (s == dtype_name(d)) return d;
  throw PlanError("unknown dtype `" + s + "`");
}
inline uint32_t dtype_bits(Dtype d) {
  switch (d) {
    case Dtype::F32: return 32;
    case Dtype::Bf16: case Dtype::Fp16: return 16;
    case Dtype::Fp8E4m3: case Dtype::Fp8E5m2: case Dtype::Int8: return 8;
    case Dtype::Int4: return 4;
  }
  return 0;
}
inline uint64_t dtype_bytes_for(Dtype d, uint64_t n) { return (dtype_bits(d) * n + 7) / 8; }
inline bool dtype_is_float(Dtype d) { return d != Dtype::Int8 && d != Dtype::Int4; }

enum class Component { Weight, Activation, KvCache };
inline const char* component_name(Component c) {
  return c == Component::Weight ? "weight" : c == Component::Activation ? "activation" : "kv_cache";
}

// ---- model IR ------------------------------------------------------------------------------------
struct Param {
  std::string name;
  std::vector<uint64_t> shape;
  Dtype dtype = Dtype::Bf16;
  uint64_t numel() const { uint64_t n = 1; for (auto d : shape) n *= d; return n; }
};

enum class LayerKind { Embedding, RmsNorm, Attention, Mlp, Moe, Lmhead };
inline const char* layer_kind_name(LayerKind k) {
  switch (k) {
    case LayerKind::Embedding: return "embedding"; case LayerKind::RmsNorm: return "rms_norm";
    case LayerKind::Attention: return "attention"; case LayerKind::Mlp: return "mlp";
    case LayerKind::Moe: return "moe"; case LayerKind::Lmhead: return "lmhead";
  }
  return "?";
}

struct Layer {
  size_t idx = 0;
  std::optional<size_t> block_idx;
  LayerKind kind = LayerKind::RmsNorm;
  // the union of the per-kind configs; unused fields stay 0
  size_t hidden = 0, vocab = 0, intermediate = 0, num_heads = 0, num_kv_heads = 0, head_dim = 0;
  size_t num_experts = 0, top_k = 0;
  double eps = 0, rope_theta = 0;
  bool tied = false;
  std::string label;  // e.g. "input_layernorm", "self_attn"
  std::vector<Param> params;
};

struct ModelMeta {
  std::string architecture;
  size_t num_layers = 0, hidden = 0, vocab = 0, max_position = 0, num_attention_heads = 0, num_kv_heads = 0,
         head_dim = 0, intermediate = 0;
  std::optional<size_t> num_experts, top_k, sliding_window;
  double rope_theta = 1e4, rms_norm_eps = 1e-5;
  bool tied_embeddings = false;
  bool qkv_bias = false;       // the q / k / v projections carry a bias vector each (Qwen2)

  Json to_json() const {
    Json j = Json::object();
    auto opt = [](const std::optional<size_t>& o) { return o ? Json((long long)*o) : Json(); };
    j.set("architecture", architecture).set("num_layers", num_layers).set("hidden", hidden).set("vocab", vocab)
        .set("max_position", max_position).set("num_attention_heads", num_attention_heads)
        .set("num_kv_heads", num_kv_heads).set("head_dim", head_dim).set("num_experts", opt(num_experts))
        .set("top_k", opt(top_k)).set("intermediate", intermediate).set("rope_theta", rope_theta)
        .set("rms_norm_eps", rms_norm_eps).set("sliding_window", opt(sliding_window))
        .set("tied_embeddings", tied_embeddings);
    if (qkv_bias) j.set("qkv_bias", true);      // written only when set: plans of models without biases keep their hash
    return j;
  }
  static ModelMeta from_json(const Json& j) {
    ModelMeta m;
    auto opt = [&](const char* k) -> std::optional<size_t> {
      const Json* v = j.find(k);
      if (!v || v->is_null()) return std::nullopt;
      return (size_t)v->as_int();
    };
    m.architecture = j.at("architecture").as_string();
    m.num_layers = j.at("num_layers").as_int(); m.hidden = j.at("hidden").as_int(); m.vocab = j.at("vocab").as_int();
    m.max_position = j.at("max_position").as_int(); m.num_attention_heads = j.at("num_attention_heads").as_int();
    m.num_kv_heads = j.at("num_kv_heads").as_int(); m.head_dim = j.at("head_dim").as_int();
    m.num_experts = opt("num_experts"); m.top_k = opt("top_k"); m.intermediate = j.at("intermediate").as_int();
    m.rope_theta = j.at("rope_theta").as_double(); m.rms_norm_eps = j.at("rms_norm_eps").as_double();
    m.sliding_window = opt("sliding_window"); m.tied_embeddings = j.at("tied_embeddings").as_bool();
    if (const Json* qb = j.find("qkv_bias"); qb && !qb->is_null()) m.qkv_bias = qb->as_bool();
    return m;
  }
  bool is_moe() const { return num_experts && *num_experts > 0; }
};

struct Graph {
  ModelMeta meta;
  std::vector<Layer> layers;
  size_t num_decoder_blocks() const {
    size_t n = 0;
    for (auto& l : layers) if (l.block_idx) n = std::max(n, *l.block_idx + 1);
    return n;
  }
  uint64_t param_count() const {
    uint64_t t = 0;
    for (auto& l : layers) for (auto& p : l.params) t += p.numel();
    return t;
  }
  Json to_json() const;
};

inline Json param_to_json(const Param& p) {
  Json shape = Json::array();
  for (auto d : p.shape) shape.push(Json::object().set("fixed", d));
  return Json::object().set("name", p.name).set("shape", shape).set("dtype", dtype_name(p.dtype));
}

inline Json Graph::to_json() const {
  Json ls = Json::array();
  for (auto& l : layers) {
    Json k = Json::object();
    k.set("kind", layer_kind_name(l.kind));
    switch (l.kind) {
      case LayerKind::Embedding: k.set("vocab", l.vocab).set("hidden", l.hidden); break;
      case LayerKind::RmsNorm: k.set("eps", l.eps).set("hidden", l.hidden); break;
      case LayerKind::Attention:
        k.set("num_heads", l.num_heads).set("num_kv_heads", l.num_kv_heads).set("head_dim", l.head_dim)
            .set("position", Json::object().set("kind", "rope").set("theta", l.rope_theta)).set("sliding_window", Json());
        break;
      case LayerKind::Mlp: k.set("hidden", l.hidden).set("intermediate", l.intermediate).set("activation", "silu"); break;
      case LayerKind::Moe:
        k.set("num_experts", l.num_experts).set("top_k", l.top_k).set("hidden", l.hidden)
            .set("intermediate", l.intermediate).set("activation", "silu");
        break;
      case LayerKind::Lmhead: k.set("vocab", l.vocab).set("hidden", l.hidden).set("tied", l.tied); break;
    }
    Json ps = Json::array();
    for (auto& p : l.params) ps.push(param_to_json(p));
    ls.push(Json::object().set("idx", l.idx).set("block_idx", l.block_idx ? Json((long long)*l.block_idx) : Json())
                .set("kind", k).set("label", l.label).set("params", ps));
  }
  return Json::object().set("meta", meta.to_json()).set("layers", ls);
}

}  // namespace skein
