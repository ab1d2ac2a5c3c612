// HuggingFace config.json -> model IR. One IR layer per logical op, parameters named exactly as in
// the HF safetensors files so that the weight sharder can slice checkpoints by name:
//   0            Embedding
//   4i+1..4i+4   RmsNorm(input_layernorm), Attention(self_attn), RmsNorm(post_attention_layernorm),
//                Moe(block_sparse_moe) or Mlp(mlp)                    for block i
//   4N+1, 4N+2   RmsNorm(model.norm), Lmhead
// The reference builds the same list for Mixtral (crates/skein_ir/src/model/mixtral.rs:74-372) and
// rejects every other architecture (model/mod.rs:33-47); the Llama family (Llama, Mistral, Qwen2
// shapes) is imported here as well.
#pragma once
#include "ir.hpp"

namespace skein {

inline size_t cfg_usize(const Json& j, const char* k) {
  const Json* v = j.find(k);
  if (!v || v->is_null()) throw ImportError(std::string("config.json: missing `") + k + "`");
  long long x = v->as_int();
  if (x < 0) throw ImportError(std::string("config.json: `") + k + "` is negative");
  return (size_t)x;
}

inline Graph import_model(const Json& cfg) {
  const Json* archs = cfg.find("architectures");
  if (!archs || !archs->is_array() || archs->size() == 0) throw ImportError("config.json: `architectures` is missing or empty");
  const std::string arch = archs->items()[0].as_string();
  const bool moe = arch == "MixtralForCausalLM";
  const bool dense = arch == "LlamaForCausalLM" || arch == "MistralForCausalLM" || arch == "Qwen2ForCausalLM";
  if (!moe && !dense) throw ImportError("architecture `" + arch + "` is not supported");
  if (const Json* act = cfg.find("hidden_act"); act && !act->is_null() && act->as_string() != "silu")
    throw ImportError("hidden_act `" + act->as_string() + "` is not supported (only silu)");

  ModelMeta m;
  m.architecture = arch;
  m.hidden = cfg_usize(cfg, "hidden_size");
  m.intermediate = cfg_usize(cfg, "intermediate_size");
  m.num_layers = cfg_usize(cfg, "num_hidden_layers");
  m.num_attention_heads = cfg_usize(cfg, "num_attention_heads");
  m.num_kv_heads = cfg.has("num_key_value_heads") && !cfg.at("num_key_value_heads").is_null()
                       ? cfg_usize(cfg, "num_key_value_heads") : m.num_attention_heads;
  m.vocab = cfg_usize(cfg, "vocab_size");
  m.max_position = cfg.has("max_position_embeddings") ? cfg_usize(cfg, "max_position_embeddings") : 8192;
  if (m.num_attention_heads == 0 || m.num_kv_heads == 0) throw ImportError("head counts must be positive");
  if (const Json* hd = cfg.find("head_dim"); hd && !hd->is_null()) m.head_dim = (size_t)hd->as_int();
  else {
    if (m.hidden % m.num_attention_heads) throw ImportError("hidden_size is not divisible by num_attention_heads and head_dim is absent");
    m.head_dim = m.hidden / m.num_attention_heads;
  }
  if (m.num_attention_heads % m.num_kv_heads) throw ImportError("num_attention_heads must be a multiple of num_key_value_heads (GQA)");
  // newer checkpoints nest theta and the frequency-scaling scheme in `rope_parameters`
  const Json* rp = cfg.find("rope_parameters");
  if (rp && (rp->is_null() || !rp->is_object())) rp = nullptr;
  m.rope_theta = cfg.has("rope_theta") && !cfg.at("rope_theta").is_null() ? cfg.at("rope_theta").as_double()
                 : (rp && rp->has("rope_theta") ? rp->at("rope_theta").as_double() : 1e4);
  {
    const Json* sc = cfg.find("rope_scaling");
    if (!sc || sc->is_null()) sc = rp;
    if (sc && sc->is_object()) {
      std::string kind = "default";
      if (const Json* t = sc->find("rope_type"); t && !t->is_null()) kind = t->as_string();
      else if (const Json* t2 = sc->find("type"); t2 && !t2->is_null()) kind = t2->as_string();
      if (kind != "default" && kind != "linear" && kind != "llama3")
        throw ImportError("rope scaling `" + kind + "` is not supported (plain, linear and llama3 are)");
    }
  }
  if (const Json* mb = cfg.find("mlp_bias"); mb && !mb->is_null() && mb->as_bool()) throw ImportError("mlp_bias = true is not supported");
  m.rms_norm_eps = cfg.has("rms_norm_eps") ? cfg.at("rms_norm_eps").as_double() : 1e-5;
  if (const Json* sw = cfg.find("sliding_window"); sw && !sw->is_null()) {
    const Json* use = cfg.find("use_sliding_window");
    // Qwen2 lists a window but applies it only with use_sliding_window. Where a window applies it becomes the position limit:
    // the kernels attend over the whole context, the same function up to that length.
    if (arch != "Qwen2ForCausalLM" || (use && !use->is_null() && use->as_bool())) {
      m.sliding_window = (size_t)sw->as_int();
      if (*m.sliding_window > 0 && *m.sliding_window < m.max_position) m.max_position = *m.sliding_window;
    }
  }
  m.tied_embeddings = cfg.has("tie_word_embeddings") && cfg.at("tie_word_embeddings").as_bool();
  // Qwen2 adds a bias to the q / k / v projections (none on o_proj). The Llama-style `attention_bias` switch adds one to
  // o_proj as well, which the runtime does not carry.
  m.qkv_bias = arch == "Qwen2ForCausalLM";
  if (const Json* ab = cfg.find("attention_bias"); ab && !ab->is_null() && ab->as_bool() && !m.qkv_bias)
    throw ImportError("attention_bias = true (biases on q, k, v and o_proj) is not supported for " + arch);
  if (moe) {
    m.num_experts = cfg_usize(cfg, "num_local_experts");
    m.top_k = cfg_usize(cfg, "num_experts_per_tok");
    if (*m.num_experts == 0 || *m.top_k == 0 || *m.top_k > *m.num_experts)
      throw ImportError("num_experts_per_tok must be in [1, num_local_experts]");
  }

  Graph g;
  g.meta = m;
  const uint64_t H = m.hidden, I = m.intermediate, D = m.head_dim, V = m.vocab;
  const uint64_t QO = m.num_attention_heads * D, KV = m.num_kv_heads * D;
  size_t idx = 0;
  auto add = [&](LayerKind k, std::optional<size_t> block, const std::string& label) -> Layer& {
    Layer l;
    l.idx = idx++; l.block_idx = block; l.kind = k; l.label = label;
    g.layers.push_back(l);
    return g.layers.back();
  };
  {
    Layer& e = add(LayerKind::Embedding, std::nullopt, "embed_tokens");
    e.vocab = V; e.hidden = H;
    e.params.push_back({"model.embed_tokens.weight", {V, H}, Dtype::Bf16});
  }
  for (size_t b = 0; b < m.num_layers; ++b) {
    const std::string pre = "model.layers." + std::to_string(b) + ".";
    Layer& n1 = add(LayerKind::RmsNorm, b, "input_layernorm");
    n1.hidden = H; n1.eps = m.rms_norm_eps;
    n1.params.push_back({pre + "input_layernorm.weight", {H}, Dtype::Bf16});
    Layer& a = add(LayerKind::Attention, b, "self_attn");
    a.num_heads = m.num_attention_heads; a.num_kv_heads = m.num_kv_heads; a.head_dim = D; a.hidden = H; a.rope_theta = m.rope_theta;
    a.params.push_back({pre + "self_attn.q_proj.weight", {QO, H}, Dtype::Bf16});
    a.params.push_back({pre + "self_attn.k_proj.weight", {KV, H}, Dtype::Bf16});
    a.params.push_back({pre + "self_attn.v_proj.weight", {KV, H}, Dtype::Bf16});
    a.params.push_back({pre + "self_attn.o_proj.weight", {H, QO}, Dtype::Bf16});
    if (m.qkv_bias) {
      a.params.push_back({pre + "self_attn.q_proj.bias", {QO}, Dtype::Bf16});
      a.params.push_back({pre + "self_attn.k_proj.bias", {KV}, Dtype::Bf16});
      a.params.push_back({pre + "self_attn.v_proj.bias", {KV}, Dtype::Bf16});
    }
    Layer& n2 = add(LayerKind::RmsNorm, b, "post_attention_layernorm");
    n2.hidden = H; n2.eps = m.rms_norm_eps;
    n2.params.push_back({pre + "post_attention_layernorm.weight", {H}, Dtype::Bf16});
    if (moe) {
      Layer& f = add(LayerKind::Moe, b, "block_sparse_moe");
      f.num_experts = *m.num_experts; f.top_k = *m.top_k; f.hidden = H; f.intermediate = I;
      f.params.push_back({pre + "block_sparse_moe.gate.weight", {(uint64_t)*m.num_experts, H}, Dtype::Bf16});
      for (size_t e = 0; e < *m.num_experts; ++e) {
        const std::string ep = pre + "block_sparse_moe.experts." + std::to_string(e) + ".";
        f.params.push_back({ep + "w1.weight", {I, H}, Dtype::Bf16});
        f.params.push_back({ep + "w2.weight", {H, I}, Dtype::Bf16});
        f.params.push_back({ep + "w3.weight", {I, H}, Dtype::Bf16});
      }
    } else {
      Layer& f = add(LayerKind::Mlp, b, "mlp");
      f.hidden = H; f.intermediate = I;
      f.params.push_back({pre + "mlp.gate_proj.weight", {I, H}, Dtype::Bf16});
      f.params.push_back({pre + "mlp.up_proj.weight", {I, H}, Dtype::Bf16});
      f.params.push_back({pre + "mlp.down_proj.weight", {H, I}, Dtype::Bf16});
    }
  }
  {
    Layer& n = add(LayerKind::RmsNorm, std::nullopt, "norm");
    n.hidden = H; n.eps = m.rms_norm_eps;
    n.params.push_back({"model.norm.weight", {H}, Dtype::Bf16});
    Layer& l = add(LayerKind::Lmhead, std::nullopt, "lm_head");
    l.vocab = V; l.hidden = H; l.tied = m.tied_embeddings;
    if (!m.tied_embeddings) l.params.push_back({"lm_head.weight", {V, H}, Dtype::Bf16});
  }
  return g;
}

inline Graph import_model_str(const std::string& text) {
  try {
    return import_model(Json::parse(text));
  } catch (const JsonError& e) {
    throw ImportError(std::string("config.json: ") + e.what());
  }
}

}  // namespace skein
