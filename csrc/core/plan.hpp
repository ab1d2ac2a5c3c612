// Plan: what `skein extract` decides and every later stage consumes. JSON layout follows the
// reference (crates/skein_ir/src/plan.rs:20-140, types.rs:149-266); the content hash is BLAKE3 of the
// compact JSON bytes and names the artifact directory.
#pragma once
#include "ir.hpp"

namespace skein {

struct ParallelismPlacement {
  uint32_t tp = 1, pp = 1, ep = 1;
  uint32_t devices_used() const { return tp * pp * ep; }
};

struct PerLayerDtype {
  Dtype weight = Dtype::Bf16, activation = Dtype::Bf16, kv_cache = Dtype::Bf16;
  static PerLayerDtype uniform(Dtype d) { return {d, d, d}; }
  bool operator==(const PerLayerDtype& o) const { return weight == o.weight && activation == o.activation && kv_cache == o.kv_cache; }
};

struct KVCacheSpec {
  bool paged = true;
  uint32_t page_size = 16;
  bool kv_sharded = true;
};

enum class BatchKind { Static, Continuous, ContinuousChunked };
struct BatchPolicy {
  BatchKind kind = BatchKind::Continuous;
  uint32_t max_batch = 1, chunk_tokens = 0;
};

struct CaptureClass { uint32_t batch_size = 1, kv_class = 0; };
struct ExecutionConfig {
  bool cuda_graphs = false;
  std::vector<CaptureClass> capture_classes;
  bool spec_decode = false;
  std::string draft_model_path;
  uint32_t speculation_depth = 0;
  bool prefix_cache = true;
  std::string reuse_policy = "lru_by_last_access";
};

enum class KvTransferMode { RdmaWrite, NcclByLayer, NvlinkP2p };
inline const char* kv_transfer_name(KvTransferMode m) {
  return m == KvTransferMode::RdmaWrite ? "rdma_write" : m == KvTransferMode::NcclByLayer ? "nccl_by_layer" : "nvlink_p2p";
}

struct Plan;
struct Disaggregation {
  std::shared_ptr<Plan> prefill, decode;
  KvTransferMode mode = KvTransferMode::NvlinkP2p;
  bool layer_overlap = true;
};

struct Plan {
  ParallelismPlacement parallelism;
  KVCacheSpec kv;
  BatchPolicy batching;
  std::vector<PerLayerDtype> dtype_map;
  ExecutionConfig execution;
  std::optional<Disaggregation> disaggregation;
  ModelMeta model_meta;

  void validate() const {
    if (dtype_map.size() != model_meta.num_layers)
      throw PlanError("dtype_map has " + std::to_string(dtype_map.size()) + " entries but the model has " +
                      std::to_string(model_meta.num_layers) + " layers");
    if (parallelism.tp == 0 || parallelism.pp == 0 || parallelism.ep == 0) throw PlanError("parallel degrees must be >= 1");
    if (disaggregation) { disaggregation->prefill->validate(); disaggregation->decode->validate(); }
  }

  Json to_json() const {
    Json j = Json::object();
    j.set("parallelism", Json::object().set("tp", parallelism.tp).set("pp", parallelism.pp).set("ep", parallelism.ep));
    Json layout = Json::object();
    if (kv.paged) layout.set("kind", "paged").set("page_size", kv.page_size); else layout.set("kind", "contiguous");
    j.set("kv", Json::object().set("layout", layout).set("kv_sharded", kv.kv_sharded));
    Json b = Json::object();
    switch (batching.kind) {
      case BatchKind::Static: b.set("kind", "static").set("max_batch", batching.max_batch); break;
      case BatchKind::Continuous: b.set("kind", "continuous").set("max_batch", batching.max_batch); break;
      case BatchKind::ContinuousChunked:
        b.set("kind", "continuous_chunked").set("max_batch", batching.max_batch).set("chunk_tokens", batching.chunk_tokens);
        break;
    }
    j.set("batching", b);
    Json per = Json::array();
    for (auto& d : dtype_map)
      per.push(Json::object().set("weight", dtype_name(d.weight)).set("activation", dtype_name(d.activation))
                   .set("kv_cache", dtype_name(d.kv_cache)));
    j.set("dtype_map", Json::object().set("per_layer", per));
    Json cc = Json::array();
    for (auto& c : execution.capture_classes) cc.push(Json::object().set("batch_size", c.batch_size).set("kv_class", c.kv_class));
    Json draft = execution.draft_model_path.empty()
                     ? Json()
                     : Json::object().set("model_path", execution.draft_model_path).set("speculation_depth", execution.speculation_depth);
    j.set("execution", Json::object()
                           .set("cuda_graphs", Json::object().set("enable", execution.cuda_graphs).set("capture_classes", cc))
                           .set("spec_decode", Json::object().set("enable", execution.spec_decode).set("draft", draft))
                           .set("prefix_cache", Json::object().set("enable", execution.prefix_cache).set("reuse_policy", execution.reuse_policy)));
    if (disaggregation) {
      j.set("disaggregation", Json::object()
                                  .set("prefill", disaggregation->prefill->to_json())
                                  .set("decode", disaggregation->decode->to_json())
                                  .set("transfer", Json::object().set("mode", kv_transfer_name(disaggregation->mode))
                                                       .set("layer_overlap", disaggregation->layer_overlap)));
    } else {
      j.set("disaggregation", Json());
    }
    j.set("model_meta", model_meta.to_json());
    return j;
  }

  static Plan from_json(const Json& j) {
    Plan p;
    const Json& par = j.at("parallelism");
    p.parallelism = {(uint32_t)par.at("tp").as_int(), (uint32_t)par.at("pp").as_int(), (uint32_t)par.at("ep").as_int()};
    const Json& kvj = j.at("kv");
    const std::string lk = kvj.at("layout").at("kind").as_string();
    if (lk == "paged") { p.kv.paged = true; p.kv.page_size = (uint32_t)kvj.at("layout").at("page_size").as_int(); }
    else if (lk == "contiguous") p.kv.paged = false;
    else throw PlanError("unknown kv layout `" + lk + "`");
    p.kv.kv_sharded = kvj.at("kv_sharded").as_bool();
    const Json& b = j.at("batching");
    const std::string bk = b.at("kind").as_string();
    p.batching.max_batch = (uint32_t)b.at("max_batch").as_int();
    if (bk == "static") p.batching.kind = BatchKind::Static;
    else if (bk == "continuous") p.batching.kind = BatchKind::Continuous;
    else if (bk == "continuous_chunked") { p.batching.kind = BatchKind::ContinuousChunked; p.batching.chunk_tokens = (uint32_t)b.at("chunk_tokens").as_int(); }
    else throw PlanError("unknown batch policy `" + bk + "`");
    for (auto& d : j.at("dtype_map").at("per_layer").items())
      p.dtype_map.push_back({dtype_from(d.at("weight").as_string()), dtype_from(d.at("activation").as_string()),
                             dtype_from(d.at("kv_cache").as_string())});
    const Json& ex = j.at("execution");
    p.execution.cuda_graphs = ex.at("cuda_graphs").at("enable").as_bool();
    for (auto& c : ex.at("cuda_graphs").at("capture_classes").items())
      p.execution.capture_classes.push_back({(uint32_t)c.at("batch_size").as_int(), (uint32_t)c.at("kv_class").as_int()});
    p.execution.spec_decode = ex.at("spec_decode").at("enable").as_bool();
    const Json& dr = ex.at("spec_decode").at("draft");
    if (!dr.is_null()) {
      p.execution.draft_model_path = dr.at("model_path").as_string();
      p.execution.speculation_depth = (uint32_t)dr.at("speculation_depth").as_int();
    }
    p.execution.prefix_cache = ex.at("prefix_cache").at("enable").as_bool();
    p.execution.reuse_policy = ex.at("prefix_cache").at("reuse_policy").as_string();
    const Json* dis = j.find("disaggregation");
    if (dis && !dis->is_null()) {
      Disaggregation d;
      d.prefill = std::make_shared<Plan>(Plan::from_json(dis->at("prefill")));
      d.decode = std::make_shared<Plan>(Plan::from_json(dis->at("decode")));
      const std::string m = dis->at("transfer").at("mode").as_string();
      d.mode = m == "rdma_write" ? KvTransferMode::RdmaWrite : m == "nccl_by_layer" ? KvTransferMode::NcclByLayer : KvTransferMode::NvlinkP2p;
      d.layer_overlap = dis->at("transfer").at("layer_overlap").as_bool();
      p.disaggregation = d;
    }
    p.model_meta = ModelMeta::from_json(j.at("model_meta"));
    return p;
  }

  std::string content_hash() const { return blake3_hex(to_json().dump()); }
};

}  // namespace skein
