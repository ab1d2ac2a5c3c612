"""C++ core: IR import, plan round-trip and hashing, cluster/workload validation, cost model ordering,
planner (enumeration, constraints, dtype DP, end-to-end extract), lowering.

Mirrors the reference's CPU tests: crates/skein_ir/tests/round_trip.rs, skein_ir/src/{cluster,workload,plan}.rs
unit tests, crates/skein_cost/tests/{cost_ordering,known_mixtral,topology_walks}.rs,
crates/skein_extract/tests/{dp_correctness,enumeration,mixtral_2xh100}.rs,
crates/skein_emit/tests/{segmentation,shard_role_correctness,topology_emission}.rs.
"""
import json
import time
from pathlib import Path

import pytest

from skein_b200 import core

ROOT = Path(__file__).resolve().parent.parent
CFG = (ROOT / "configs/mixtral_8x7b_config.json").read_text()
LLAMA = (ROOT / "configs/llama3_70b_config.json").read_text()
H100_2 = (ROOT / "cluster/h100_2x.toml").read_text()
B200_8 = (ROOT / "cluster/b200_8x.toml").read_text()
TRACE = (ROOT / "cluster/sample_trace.jsonl").read_text()
DRIFT = (ROOT / "models/mixtral_8x7b_drift.toml").read_text()
CONST = (ROOT / "cluster/cost_constants.toml").read_text()
REF_CONST = CONST.split("[hbm_gbps]")[0].replace("kernel_overhead_us = 6.5", "kernel_overhead_us = 0.0") + "[efficiency.gemm]" + CONST.split("[efficiency.gemm]")[1].split("[fused_overlap]")[0] + \
    "[representative_workload]" + CONST.split("[representative_workload]")[1]


def make_plan(tp=1, pp=1, ep=1, max_batch=16, dtype="bf16", layers=32, cuda_graphs=False, classes=0, kind="continuous", cfg=CFG):
    meta = json.loads(core.model_meta(cfg))
    meta["num_layers"] = layers if layers else meta["num_layers"]
    batching = {"kind": kind, "max_batch": max_batch}
    if kind == "continuous_chunked":
        batching["chunk_tokens"] = 1024
    return json.dumps({
        "parallelism": {"tp": tp, "pp": pp, "ep": ep},
        "kv": {"layout": {"kind": "paged", "page_size": 16}, "kv_sharded": True},
        "batching": batching,
        "dtype_map": {"per_layer": [{"weight": dtype, "activation": "bf16", "kv_cache": "bf16"}] * meta["num_layers"]},
        "execution": {"cuda_graphs": {"enable": cuda_graphs, "capture_classes": [{"batch_size": 1 + i, "kv_class": 0} for i in range(classes)]},
                      "spec_decode": {"enable": False, "draft": None},
                      "prefix_cache": {"enable": True, "reuse_policy": "lru_by_last_access"}},
        "disaggregation": None, "model_meta": meta})


# ---- IR -------------------------------------------------------------------------------------------------------
def test_mixtral_param_count_matches_known_value():
    assert core.model_param_count(CFG) == 46_702_792_704


def test_shipped_configs_have_their_known_parameter_counts_and_plan():
    from skein_b200.models.config import ModelConfig
    known = {"mixtral_8x7b": 46_702_792_704, "llama3_70b": 70_553_706_496, "qwen2_5_7b": 7_615_616_512, "mistral_7b": 7_248_023_552}
    for name, n in known.items():
        cfg = (ROOT / f"configs/{name}_config.json").read_text()
        assert core.model_param_count(cfg) == n == ModelConfig.from_file(ROOT / f"configs/{name}_config.json").param_count(), name
        r = core.extract_plan(cfg, (ROOT / "cluster/b200_4x.toml").read_text(), TRACE, (ROOT / f"models/{name}_drift.toml").read_text(), CONST,
                              {"objective": "throughput"})
        par = json.loads(r["plan_json"])["parallelism"]
        assert par["tp"] * par["pp"] * par["ep"] <= 4 and r["cost_us"] > 0
    q = ModelConfig.from_file(ROOT / "configs/qwen2_5_7b_config.json")
    assert q.qkv_bias and q.eos_token_id == 151645 and q.head_dim == 128 and q.max_position_embeddings == 32768


def test_importer_layer_order_and_names():
    g = json.loads(core.import_model(CFG))
    kinds = [l["kind"]["kind"] for l in g["layers"]]
    assert kinds[0] == "embedding" and kinds[1:5] == ["rms_norm", "attention", "rms_norm", "moe"]
    assert kinds[-2:] == ["rms_norm", "lmhead"] and len(kinds) == 4 * 32 + 3
    names = [p["name"] for l in g["layers"] for p in l["params"]]
    assert "model.layers.3.block_sparse_moe.experts.7.w2.weight" in names and "lm_head.weight" in names
    gl = json.loads(core.import_model(LLAMA))
    assert gl["layers"][4]["kind"]["kind"] == "mlp" and gl["meta"]["num_experts"] is None
    assert "model.layers.0.mlp.gate_proj.weight" in [p["name"] for p in gl["layers"][4]["params"]]


@pytest.mark.parametrize("mutate,msg", [
    (lambda c: c.update(architectures=["GPT2LMHeadModel"]), "not supported"),
    (lambda c: c.update(architectures=[]), "architectures"),
    (lambda c: c.update(hidden_act="gelu"), "hidden_act"),
    (lambda c: c.update(num_key_value_heads=5), "multiple"),
    (lambda c: c.update(num_experts_per_tok=9), "num_experts_per_tok"),
    (lambda c: c.pop("hidden_size"), "hidden_size"),
    (lambda c: c.update(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope scaling"),
    (lambda c: c.update(rope_parameters={"rope_type": "dynamic", "factor": 2.0, "rope_theta": 1e6}), "rope scaling"),
    (lambda c: c.update(architectures=["LlamaForCausalLM"], attention_bias=True), "attention_bias"),
    (lambda c: c.update(architectures=["LlamaForCausalLM"], mlp_bias=True), "mlp_bias"),
])
def test_importer_rejections(mutate, msg):
    """What the runtime would compute differently from the checkpoint's own modelling code is refused, by the C++ importer
    and by its Python mirror alike, instead of being served wrong."""
    from skein_b200.models.config import ModelConfig
    c = json.loads(CFG)
    mutate(c)
    with pytest.raises(Exception, match=msg):
        core.import_model(json.dumps(c))
    with pytest.raises(Exception, match=msg):
        ModelConfig.from_hf_dict(c)


def test_importers_agree_on_family_details():
    from skein_b200.models.config import ModelConfig
    base = json.loads(LLAMA)
    # Qwen2: q / k / v biases are parameters; its listed window applies only with use_sliding_window
    q = dict(base, architectures=["Qwen2ForCausalLM"], sliding_window=4096, use_sliding_window=False, max_position_embeddings=32768)
    g = json.loads(core.import_model(json.dumps(q)))
    names = [p["name"] for l in g["layers"] for p in l["params"]]
    assert "model.layers.0.self_attn.q_proj.bias" in names and "model.layers.0.self_attn.o_proj.bias" not in names
    assert g["meta"]["qkv_bias"] is True and g["meta"]["max_position"] == 32768
    cq = ModelConfig.from_hf_dict(q)
    assert cq.qkv_bias and cq.max_position_embeddings == 32768 and cq.param_count() == core.model_param_count(json.dumps(q))
    assert "qkv_bias" not in json.loads(core.import_model(LLAMA))["meta"]          # plans of bias-free models keep their hash
    # a window that applies becomes the position limit (Mistral v0.1)
    m = dict(base, architectures=["MistralForCausalLM"], sliding_window=4096, max_position_embeddings=32768)
    assert json.loads(core.model_meta(json.dumps(m)))["max_position"] == 4096 and ModelConfig.from_hf_dict(m).max_position_embeddings == 4096
    # theta nested in rope_parameters (recent checkpoints), llama3 scaling accepted
    n = {k: v for k, v in base.items() if k != "rope_theta"}
    n["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}
    assert json.loads(core.model_meta(json.dumps(n)))["rope_theta"] == 5e5
    cn = ModelConfig.from_hf_dict(n)
    assert cn.rope_theta == 5e5 and cn.rope_scaling["rope_type"] == "llama3" and cn.to_hf_dict()["rope_scaling"]["factor"] == 8.0


def test_plan_round_trip_and_hash_stability():
    p = make_plan(tp=2, max_batch=16)
    rt = core.plan_roundtrip(p)
    assert json.loads(rt) == json.loads(p)
    assert core.plan_roundtrip(rt) == rt                      # byte-stable once canonical
    assert core.plan_hash(p) == core.plan_hash(rt) and len(core.plan_hash(p)) == 64
    assert core.plan_hash(make_plan(tp=4)) != core.plan_hash(p)
    bad = json.loads(p)
    bad["dtype_map"]["per_layer"].pop()
    with pytest.raises(Exception, match="dtype_map"):
        core.plan_validate(json.dumps(bad))


def test_blake3_known_vectors():
    assert core.blake3_hex(b"") == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    data = bytes(i % 251 for i in range(1025))
    assert core.blake3_hex(data) == "d00278ae47eb27b34faecf67b4fe263f82d5412916c1ffd97c8cb7fb814b8444"
    try:
        import blake3
        big = bytes(i % 251 for i in range(70000))
        assert core.blake3_hex(big) == blake3.blake3(big).hexdigest()
    except ImportError:
        pass


def test_dtype_bytes():
    assert core.dtype_bytes_for("int4", 3) == 2 and core.dtype_bytes_for("int4", 1024) == 512
    assert core.dtype_bytes_for("bf16", 1024) == 2048 and core.dtype_bits("fp8_e4m3") == 8


# ---- cluster / workload -------------------------------------------------------------------------------------------
def test_cluster_parses_and_rejects():
    c = json.loads(core.cluster_validate(H100_2))
    assert c["num_devices"] == 2 and c["link"][0]["kind"] == "nvlink_gen4"
    assert len(json.loads(core.cluster_validate(B200_8))["link"]) == 28
    with pytest.raises(Exception, match="num_devices"):
        core.cluster_validate(H100_2.replace("num_devices = 2", "num_devices = 3"))
    with pytest.raises(Exception, match="duplicate device"):
        core.cluster_validate(H100_2.replace('["d0", "d1"]', '["d0", "d0"]', 1))
    with pytest.raises(Exception, match="itself"):
        core.cluster_validate(H100_2.replace('endpoints      = ["d0", "d1"]', 'endpoints      = ["d0", "d0"]'))
    with pytest.raises(Exception, match="unknown device"):
        core.cluster_validate(H100_2.replace('endpoints      = ["d0", "d1"]', 'endpoints      = ["d0", "d9"]'))
    with pytest.raises(Exception, match="link kind"):
        core.cluster_validate(H100_2.replace("nvlink_gen4", "carrier_pigeon"))


def test_workload_parses_and_rejects():
    w = core.workload_parse(TRACE)
    assert w["n"] == 5 and w["ttft_p95_ms"] == 500 and abs(w["max_accuracy_drift"] - 0.01) < 1e-12
    with pytest.raises(Exception, match="empty"):
        core.workload_parse("\n  \n")
    with pytest.raises(Exception, match="slo"):
        core.workload_parse('{"prompt_tokens": 1, "output_tokens": 1, "arrival_ms": 0}\n')
    lines = TRACE.strip().split("\n")
    with pytest.raises(Exception, match="earlier"):
        core.workload_parse("\n".join([lines[0], lines[2], lines[1]]))


def test_synthetic_traces_are_deterministic_and_valid():
    a = core.synth_uniform_trace(256, 0, 128, 2048, 64, 512, 4.0)
    assert a == core.synth_uniform_trace(256, 0, 128, 2048, 64, 512, 4.0)
    assert a != core.synth_uniform_trace(256, 1, 128, 2048, 64, 512, 4.0)
    w = core.workload_parse(a)
    assert w["n"] == 256 and 128 <= w["mean_prompt"] <= 2048
    b = core.synth_burst_trace(2000, 0, 50.0, 2.0, 10.0, 600.0, 8192, 32, 1024)
    assert core.workload_parse(b)["n"] == 2000


# ---- topology / placement ------------------------------------------------------------------------------------------
def test_paths_and_placement():
    bw, lat, hops = core.pair_path(B200_8, 0, 7)
    assert (bw, lat, hops) == (770.0, 2.0, 1)
    chain = """num_devices = 3
[[node]]
id = "n"
devices = ["a", "b", "c"]
device_kind = "h100_sxm5"
device_memory_gb = 80
[[link]]
endpoints = ["a", "b"]
kind = "nvlink_gen4"
bandwidth_gbps = 900.0
latency_us = 1.0
[[link]]
endpoints = ["b", "c"]
kind = "pcie5"
bandwidth_gbps = 64.0
latency_us = 1.5
"""
    assert core.pair_path(chain, 0, 2) == (64.0, 2.5, 2)          # bottleneck bandwidth, summed latency
    assert core.collective_path(chain, [0, 1, 2])[0] == 64.0      # worst pair decides
    g = core.placement_groups(2, 2, 2, 5)                          # device 5 = stage 1, ep 0, tp 1
    assert g["stage"] == 1 and g["tp_group"] == [4, 5] and g["ep_group"] == [5, 7] and g["pp_group"] == [1, 5]
    assert [core.block_to_stage(b, 10, 4) for b in range(10)] == [0, 0, 0, 1, 1, 1, 2, 2, 3, 3]
    assert core.collective_factor("ring_allreduce", 8) == 1.75 and core.collective_factor("allgather", 4) == 0.75
    assert core.collective_factor("send_recv", 2) == 1.0


# ---- cost model ------------------------------------------------------------------------------------------------------
def test_cost_ordering_invariants():
    cost = lambda p, cl=H100_2, c=REF_CONST: core.total_cost(p, CFG, cl, c)
    # bf16 TP=1 does not fit one 80 GB card: the memory penalty dominates everything else
    a = cost(make_plan(tp=1))
    b = cost(make_plan(tp=2))
    c = cost(make_plan(tp=2, dtype="fp8_e4m3"))
    assert a > 1e6 and b < 1e5 and c < 1e5
    assert 1.05 < b / c < 2.5                                     # fp8 speed-up band of the reference's known_mixtral test
    # compute shrinks with TP; comm appears with TP
    b1 = core.cost_breakdown(make_plan(tp=1), CFG, H100_2, REF_CONST, 0)
    b2 = core.cost_breakdown(make_plan(tp=2), CFG, H100_2, REF_CONST, 0)
    assert b2["compute"] < b1["compute"] and b1["comm"] == 0 and b2["comm"] > 0
    assert b2["collectives"] == 64                                # 2 all-reduces per block at tp=2
    # bubble = (pp-1)/pp * stage compute
    p2 = make_plan(pp=2)
    bp = core.cost_breakdown(p2, CFG, H100_2, REF_CONST, 0)
    assert abs(bp["bubble"] - 0.5 * bp["compute"]) < 1e-6 and core.bubble_time(make_plan(pp=1), 100.0) == 0
    # CUDA graphs reduce the launch term
    assert cost(make_plan(tp=2, cuda_graphs=True, classes=4)) < cost(make_plan(tp=2))
    assert core.cuda_graph_coverage(make_plan(cuda_graphs=False)) == 0.0
    assert core.cuda_graph_coverage(make_plan(cuda_graphs=True, classes=4)) == 0.95
    assert core.cuda_graph_coverage(make_plan(cuda_graphs=True, classes=2)) == 0.7
    assert core.cuda_graph_coverage(make_plan(cuda_graphs=True, classes=4, kind="continuous_chunked")) == 0.4
    assert core.cuda_graph_coverage(make_plan(cuda_graphs=True, kind="static")) == 1.0
    # a fused (one-launch) all-reduce of 2x bytes beats two separate ones by exactly one latency
    one = core.comm_time("ring_allreduce", [0, 1], 2 << 20, H100_2, REF_CONST)
    two = 2 * core.comm_time("ring_allreduce", [0, 1], 1 << 20, H100_2, REF_CONST)
    assert abs((two - one) - 1.0) < 1e-9


def test_b200_roofline_and_overlap_terms():
    p = make_plan(tp=8, max_batch=64)
    with_roof = core.cost_breakdown(p, CFG, B200_8, CONST, 0)
    no_roof = core.cost_breakdown(p, CFG, B200_8, CONST.replace("b200      = 6552.0", "b200      = 0.0"), 0)
    assert with_roof["compute"] > no_roof["compute"]              # decode is bandwidth-bound on B200
    no_overlap = core.cost_breakdown(p, CFG, B200_8, CONST.replace("ring_allreduce = 0.5", "ring_allreduce = 0.0"), 0)
    assert with_roof["comm"] < no_overlap["comm"]
    # narrower weights move fewer bytes and win the roofline term with the measured share of the copy bandwidth ...
    p8 = make_plan(tp=8, max_batch=64, dtype="fp8_e4m3")
    assert "fp8_e4m3 = 0.70" in CONST
    assert core.cost_breakdown(p8, CFG, B200_8, CONST, 0)["compute"] < with_roof["compute"]
    # ... and would not if the fp8 kernel reached less than half of the share of the bf16 one (fp8 then buys memory only)
    slow8 = CONST.replace("fp8_e4m3 = 0.70", "fp8_e4m3 = 0.42")
    assert core.cost_breakdown(p8, CFG, B200_8, slow8, 0)["compute"] >= with_roof["compute"]


def test_b200_constants_reproduce_measured_decode_steps():
    """The constants file carries fits to decode steps measured on B200s (Mixtral-8x7B, CUDA graphs, context about 600 for
    the tensor-parallel runs of 64 sequences and about 1040 for the expert-parallel runs of 256 with e4m3 weights): the
    model must land within 10 % of each of them, so that a change of a term or a constant that breaks the fit shows."""
    def predict(n, kv, **kw):
        cl = (ROOT / f"cluster/b200_{n}x.toml").read_text()
        c = CONST.replace("decode_kv_tokens = 2048", f"decode_kv_tokens = {kv}")
        b = core.cost_breakdown(make_plan(cuda_graphs=True, classes=4, **kw), CFG, cl, c, 0)
        return b
    for n, ms in ((1, 16.99), (2, 9.95), (4, 5.79), (8, 4.44)):
        b = predict(n, 608, tp=n, max_batch=64)
        assert b["kernels"] == 229                                 # 7 launches per block + embedding, lm_head, 3 per step
        assert abs(b["total"] / 1e3 - ms) / ms < 0.10, (n, b)
    for n, ms in ((8, 7.66), (4, 10.28)):
        b = predict(n, 1040, ep=n, max_batch=256, dtype="fp8_e4m3")
        assert abs(b["total"] / 1e3 - ms) / ms < 0.10, (n, b)
    # pure expert parallelism attends data-parallel: a rank streams the KV of its own 1/ep of the sequences, while with
    # tensor parallelism beside it every expert-parallel group attends over the whole batch
    one = predict(8, 1040, tp=8, max_batch=256)
    ep8 = predict(8, 1040, ep=8, max_batch=256)
    mix = predict(8, 1040, tp=2, ep=4, max_batch=256)
    kv_full = 256 * 1040 * 2 * 8 * 128 * 2 * 32 / 6552e9 * 1e6      # us to stream the whole batch's KV on one GPU
    assert ep8["compute"] < one["compute"] + kv_full               # nowhere near a replicated read of the KV
    assert mix["compute"] > kv_full / 2                            # tp2 x ep4: half of the KV per GPU
    # pipeline parallelism as the runtime runs it: Llama-3-70B on TP4 x PP2, 32 sequences, measured 18.3 ms per drained step
    # (12.0 ms with the pipeline kept full); a stage streams its weights once per micro-batch, so PP buys memory, not time
    cl8 = (ROOT / "cluster/b200_8x.toml").read_text()
    c = CONST.replace("decode_kv_tokens = 2048", "decode_kv_tokens = 1100")
    pl = make_plan(tp=4, pp=2, max_batch=32, cuda_graphs=True, classes=4, cfg=LLAMA, layers=80)
    b = core.cost_breakdown(pl, LLAMA, cl8, c, 0)
    assert abs(b["total"] / 1e3 - 18.3) / 18.3 < 0.12, b
    full = core.cost_breakdown(pl, LLAMA, cl8, c.replace("drain_per_step = 1", "drain_per_step = 0"), 0)
    assert full["bubble"] == 0 and abs(full["total"] / 1e3 - 12.0) / 12.0 < 0.12, full
    assert abs(b["bubble"] - (b["compute"] + b["comm"] + b["launch"]) / 2) < 1e-6        # (pp - 1) of the M = 2 stage passes
    for n in (2, 4, 8):                                            # on one NVSwitch domain the latency planner shards, never pipelines
        r = core.extract_plan(CFG, (ROOT / f"cluster/b200_{n}x.toml").read_text(), TRACE, DRIFT, CONST)
        assert json.loads(r["plan_json"])["parallelism"] == {"tp": n, "pp": 1, "ep": 1}
    # the fixed cost per kernel is not hidden by CUDA graphs, the host launch cost is
    g, e = predict(1, 608, tp=1, max_batch=64), core.cost_breakdown(make_plan(tp=1, max_batch=64), CFG, (ROOT / "cluster/b200_1x.toml").read_text(), CONST, 0)
    assert 229 * 6.5 <= g["launch"] < 229 * 6.5 + 40 and e["launch"] > g["launch"] + 229 * 2.0


# ---- planner ----------------------------------------------------------------------------------------------------------
def test_enumeration_and_constraints():
    assert core.enumerate_parallelism(CFG, 2) == [(1, 1, 1), (1, 1, 2), (1, 2, 1), (2, 1, 1)]
    assert core.enumerate_parallelism(LLAMA, 4) == [(1, 1, 1), (1, 2, 1), (1, 4, 1), (2, 1, 1), (2, 2, 1), (4, 1, 1)]
    assert core.enumerate_count(CFG, H100_2) == 4 * 10 * 14
    assert core.reject_reason(CFG, H100_2, REF_CONST, 2, 1, 1, 16, True) == "none"
    assert core.reject_reason(CFG, H100_2, REF_CONST, 4, 1, 1, 16, True) == "device_count"
    assert core.reject_reason(LLAMA, B200_8, CONST, 1, 1, 2, 16, True) == "ep_divisibility"
    c3 = json.loads(CFG); c3["num_attention_heads"] = 36; c3["num_key_value_heads"] = 6; c3["head_dim"] = 128
    assert core.reject_reason(json.dumps(c3), B200_8, CONST, 8, 1, 1, 16, True) == "tp_divisibility"
    tiny_mem = H100_2.replace("device_memory_gb = 80", "device_memory_gb = 4")
    assert core.reject_reason(CFG, tiny_mem, REF_CONST, 2, 1, 1, 16, True) == "global_memory"


def test_throughput_objective_respects_both_latency_targets():
    """The throughput objective keeps plans whose decode step meets the TPOT target and whose prefill of the trace's
    95th-percentile prompt meets the TTFT target; long prompts therefore need more tensor-parallel ranks. When nothing meets
    both, the best plan that meets the TPOT target is returned, and when nothing meets that either, the shortest step."""
    def trace(prompt, ttft, tpot=50):
        hdr = {"slo": {"ttft_p95_ms": ttft, "tpot_p95_ms": tpot, "max_accuracy_drift": 0.01, "recompile_drift_threshold_kl": 0.05}}
        return json.dumps(hdr) + "\n" + "".join(json.dumps({"prompt_tokens": prompt, "output_tokens": 64, "arrival_ms": 10 * i}) + "\n" for i in range(20))

    def pick(n, prompt, ttft, tpot=50):
        r = core.extract_plan(CFG, (ROOT / f"cluster/b200_{n}x.toml").read_text(), trace(prompt, ttft, tpot), DRIFT, CONST, {"objective": "throughput"})
        p = json.loads(r["plan_json"])
        return p["parallelism"]["tp"], p["batching"]["max_batch"]
    assert pick(4, 2000, 300) == (4, 64)
    # 32k-token prompts at about 20 us per token and rank: 650 ms on one rank, within 300 ms only on four
    assert pick(4, 32000, 300) == (4, 64) and pick(2, 32000, 400)[0] == 2
    # one GPU cannot meet 300 ms for such prompts: the plan that meets the TPOT target is kept, not a batch of one
    assert pick(1, 32000, 300) == (1, 64)
    # a TPOT target below any step: the shortest step
    assert pick(1, 2000, 300, tpot=1) == (1, 1)
    # on 8 GPUs a prompt-heavy trace with a tight TTFT keeps tensor parallelism at 8 where a lax one could choose fewer ranks' worth
    assert pick(8, 32000, 150)[0] == 8


def test_dtype_dp_behaviour():
    dp = lambda mem, drift: core.layer_dtype_dp(CFG, H100_2, REF_CONST, DRIFT, 2, 1, 1, 16, True, mem, drift)
    cost, dm = dp(70 * 10**9, 1e-9)                               # tight drift: everything stays bf16
    assert all(d == ("bf16", "bf16", "bf16") for d in dm)
    cost_q, dm_q = dp(16 * 10**9, 100.0)                          # tight memory: aggressive quantisation
    assert sum(d[0] == "int4" for d in dm_q) > 16
    assert dp(10**6, 100.0) is None                               # infeasible
    cost_loose, dm_loose = dp(70 * 10**9, 100.0)
    assert cost_loose <= cost


def test_extract_end_to_end_fast_and_deterministic():
    t0 = time.time()
    r = core.extract_plan(CFG, H100_2, TRACE, DRIFT, REF_CONST)
    assert time.time() - t0 < 5.0
    plan = json.loads(r["plan_json"])
    assert plan["parallelism"]["tp"] * plan["parallelism"]["pp"] * plan["parallelism"]["ep"] <= 2
    assert len(plan["dtype_map"]["per_layer"]) == 32
    # never worse than the all-bf16 TP=2 baseline
    assert r["cost_us"] <= core.total_cost(make_plan(tp=2, max_batch=plan["batching"]["max_batch"]), CFG, H100_2, REF_CONST) + 1e-6
    r2 = core.extract_plan(CFG, H100_2, TRACE, DRIFT, REF_CONST)
    assert r2["plan_json"] == r["plan_json"] and r2["content_hash"] == r["content_hash"]
    counters = json.loads(r["counters_json"])
    assert counters["raw"] == 560 and counters["scored"] > 0
    # forced placement and throughput objective
    f = json.loads(core.extract_plan(CFG, B200_8, TRACE, DRIFT, CONST, {"force_tp": 2, "force_ep": 4, "force_pp": 1})["plan_json"])
    assert f["parallelism"] == {"tp": 2, "pp": 1, "ep": 4}
    thr = json.loads(core.extract_plan(CFG, B200_8, TRACE, DRIFT, CONST, {"objective": "throughput"})["plan_json"])
    assert thr["batching"]["max_batch"] == 64 and thr["kv"]["layout"] == {"kind": "paged", "page_size": 16}
    # restricting the dtype combos to what the kernels implement
    only = core.extract_plan(CFG, B200_8, TRACE, DRIFT, CONST, {}, [["bf16", "bf16", "bf16"], ["fp8_e4m3", "fp8_e4m3", "bf16"]])
    assert {tuple(d.values()) for d in json.loads(only["plan_json"])["dtype_map"]["per_layer"]} <= {("bf16", "bf16", "bf16"), ("fp8_e4m3", "fp8_e4m3", "bf16")}
    with pytest.raises(Exception, match="no feasible plan"):
        core.extract_plan(CFG, H100_2.replace("device_memory_gb = 80", "device_memory_gb = 1"), TRACE, DRIFT, REF_CONST)


def test_disaggregated_plan_splits_the_cluster():
    r = core.extract_disaggregated_plan(CFG, (ROOT / "cluster/b200_4x.toml").read_text(), TRACE, DRIFT, CONST, 2)
    plan = json.loads(r["plan_json"])
    d = plan["disaggregation"]
    assert d["transfer"]["mode"] == "nvlink_p2p" and d["prefill"]["disaggregation"] is None
    assert d["decode"]["parallelism"]["tp"] * d["decode"]["parallelism"]["ep"] * d["decode"]["parallelism"]["pp"] <= 2
    with pytest.raises(Exception, match="invalid disaggregation"):
        core.extract_disaggregated_plan(CFG, H100_2, TRACE, DRIFT, REF_CONST, 2)


def test_drift_table_lookup_update_and_byte_stability():
    t = core.DriftTable.from_toml(DRIFT)
    assert t.lookup(5, "weight", "fp8_e4m3") == 0.008 and t.lookup(5, "kv_cache", "bf16") == 0.0
    assert abs(t.block_contribution(0, "fp8_e4m3", "fp8_e4m3", "int8") - (0.008 + 0.005 + 0.018)) < 1e-12
    assert t.raise_layer_override(10, "weight", "fp8_e4m3", 0.05) is True
    assert t.raise_layer_override(10, "weight", "fp8_e4m3", 0.01) is False      # monotonic
    assert t.lookup(10, "weight", "fp8_e4m3") == 0.05 and t.lookup(11, "weight", "fp8_e4m3") == 0.008
    text = t.to_toml()
    assert "[layer.10.weight]\nfp8_e4m3 = 0.05" in text
    assert core.DriftTable.from_toml(text).to_toml() == text
    with pytest.raises(Exception, match="default"):
        core.DriftTable.from_toml("[default.weight]\nbf16 = 0.0\n")


# ---- lowering ------------------------------------------------------------------------------------------------------------
def test_topology_and_segments():
    p = make_plan(tp=2)
    topo = json.loads(core.emit_topology(p, CFG))["collectives"]
    # the vocabulary-parallel embedding's sum, two all-reduces per block, the candidate exchange of the sampler
    assert len(topo) == 1 + 2 * 32 + 1 and topo[0]["tensor_name"] == "embed_out" and topo[1]["tensor_name"] == "block_0_attn_out"
    assert topo[-1]["kind"] == "allgather"
    assert [e["sequence_idx"] for e in topo] == list(range(len(topo)))
    low = json.loads(core.lower_device(p, CFG, 0))
    n_coll = sum(1 for s in low["sequencing"] if s["kind"] == "collective")
    assert len(low["segments"]) == n_coll + 1                      # one segment between every two collectives
    # hand-off names agree between the producer and the consumer segment
    for a, b in zip(low["segments"], low["segments"][1:]):
        assert a["outputs"][-1] == b["inputs"][0]
    assert core.lower_device(p, CFG, 0) == core.lower_device(p, CFG, 0)   # byte-stable
    # tp2 x ep2: dispatch/combine all-to-all per MoE block, token-routed
    p22 = make_plan(tp=2, ep=2)
    topo22 = json.loads(core.emit_topology(p22, CFG))["collectives"]
    assert sum(e["kind"] == "alltoall" for e in topo22) == 2 * 32 * 2
    low22 = json.loads(core.lower_device(p22, CFG, 3))
    assert len(low22["segments"]) == sum(1 for s in low22["sequencing"] if s["kind"] == "collective") + 1
    # pipeline stages: recv before the first segment, send after the last
    lowpp = json.loads(core.lower_device(make_plan(pp=2), CFG, 1))
    assert lowpp["sequencing"][0]["collective"] == "send_recv" and lowpp["segments"][0]["inputs"] == ["carry_pre_block_16"]


def test_shard_roles_and_io_manifest():
    assert core.param_kind_for("model.layers.0.self_attn.q_proj.weight")[0] == "column"
    assert core.param_kind_for("model.layers.0.self_attn.o_proj.weight")[0] == "row"
    assert core.param_kind_for("model.layers.0.block_sparse_moe.experts.5.w2.weight") == ("expert", 5, False)
    assert core.param_kind_for("model.layers.0.block_sparse_moe.gate.weight")[0] == "replicated"
    assert core.param_kind_for("model.norm.weight")[0] == "replicated"
    io = {t["name"]: t for t in json.loads(core.io_manifest(make_plan(tp=2, ep=2, pp=2), CFG, 7))["tensors"]}   # stage 1, ep 1, tp 1
    io0 = {t["name"]: t for t in json.loads(core.io_manifest(make_plan(tp=2, ep=2, pp=2), CFG, 1))["tensors"]}      # stage 0, ep 0, tp 1
    assert io0["model.embed_tokens.weight"]["shape"] == [16000, 4096] and io0["model.embed_tokens.weight"]["start"] == 16000
    assert "model.embed_tokens.weight" not in io and "lm_head.weight" in io and "model.layers.0.input_layernorm.weight" not in io
    assert io["lm_head.weight"]["shape"] == [16000, 4096] and io["lm_head.weight"]["start"] == 16000
    assert io["model.layers.20.self_attn.o_proj.weight"]["shape"] == [4096, 2048] and io["model.layers.20.self_attn.o_proj.weight"]["axis"] == 1
    assert "model.layers.20.block_sparse_moe.experts.5.w1.weight" in io and "model.layers.20.block_sparse_moe.experts.2.w1.weight" not in io
    assert io["model.layers.20.block_sparse_moe.experts.5.w1.weight"]["shape"] == [7168, 4096]
    assert io["model.layers.20.block_sparse_moe.experts.5.w2.weight"]["shape"] == [4096, 7168]
