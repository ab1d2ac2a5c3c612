"""`skein compile`: plan -> artifact -> bf16 reference artifact -> parity gate -> (on failure) drift-table
update and re-plan -> LATEST symlink.

Follows the reference's compile command (crates/skein_cli/src/cmd/compile.rs:23-256) minus its clamp of
every sub-bf16 dtype to bf16 (:57-77): the dtype map is honoured, so the gate really sees fp8 weights.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from .. import core
from ..models.config import ModelConfig
from . import parity
from .artifact import Artifact, WeightSource, build_artifact, update_latest_symlink

# (weight, activation, kv_cache) combinations the runtime's kernels implement today.
SUPPORTED_COMBOS = [["bf16", "bf16", "bf16"], ["fp8_e4m3", "bf16", "bf16"]]


@dataclass
class CompileResult:
    artifact_dir: Path
    plan: dict
    report: parity.ParityReport | None
    replans: int
    drift_toml: str


def all_bf16(plan: dict) -> dict:
    p = json.loads(json.dumps(plan))
    for d in p["dtype_map"]["per_layer"]:
        d["weight"] = d["activation"] = d["kv_cache"] = "bf16"
    return p


def default_parity_prompts(cfg: ModelConfig, n: int, length: int = 24, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]


def estimate_runtime(plan_json: str, config_json: str, cluster_toml: str, constants_toml: str) -> dict:
    """The batcher's latency estimator for this plan on this cluster, taken from the placement cost model instead of the
    constants file's machine-independent defaults: the decode step at batch 1, the exponent of the power law through the
    steps at batch 1 and at the plan's batch, and the prefill time per prompt token (2 FLOPs per active parameter at the
    measured GEMM rate, divided among the tensor-parallel ranks). The admission rule (predicted TPOT against the SLO) is only
    as good as these numbers: with the defaults (8 ms x batch^0.7) a B200 that steps 64 sequences in 17 ms is predicted to need
    147 ms and admits a fifth of what it can serve."""
    import math
    import re
    plan = json.loads(plan_json)
    B = int(plan["batching"]["max_batch"])

    def step_us(batch):
        p = json.loads(plan_json)
        p["batching"]["max_batch"] = batch
        return float(core.cost_breakdown(json.dumps(p), config_json, cluster_toml, constants_toml, 0)["total"])
    c1 = step_us(1)
    # through the steps at batch 1 and at the plan's batch, or at 64 for a plan of fewer sequences (a server may be started
    # with a larger --max-batch than the plan's)
    Bref = max(B, 64)
    exponent = min(1.0, max(0.0, math.log(max(step_us(Bref), c1) / c1) / math.log(Bref)))
    cfg = ModelConfig.from_hf_dict(json.loads(config_json))
    consts = json.loads(core.cost_constants_json(constants_toml))
    m = re.search(r'device_kind\s*=\s*"([^"]+)"', cluster_toml)
    kind = m.group(1) if m else "b200"
    peak = consts["peak_tflops"].get(kind, {}).get("bf16", 1000.0) * consts["efficiency"]["gemm"].get("bf16", 0.7)
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    active = cfg.num_layers * (2 * H * D * (cfg.num_heads + cfg.num_kv_heads) + 3 * H * I * (cfg.top_k if cfg.is_moe else 1)) + cfg.vocab_size * H
    tp = max(1, int(plan["parallelism"]["tp"]))
    prefill_us = 2.0 * active / (peak * 1e12) * 1e6 / tp + float(consts.get("runtime_estimator", {}).get("prefill_overhead_us_per_token", 0.0))
    return {"per_token_decode_us_at_b1": round(c1, 1), "batch_scaling_exponent": round(exponent, 4),
            "prefill_per_token_us": round(prefill_us, 3), "source": "placement cost model"}


def compile_model(config_json: str, cluster_toml: str, trace_jsonl: str, drift_toml: str, constants_toml: str, out_root,
                  weights: str | None = None, options: dict | None = None, n_parity_prompts: int = 8, prompts=None,
                  enforce_parity: bool = False, max_replans: int = 2, parity_device: str = "cpu", seed: int = 0,
                  run_parity: bool = True, tokenizer_json=None, search_budget: int = 0) -> CompileResult:
    """`search_budget` > 0 on a machine with a GPU: time up to that many launch configurations for every GEMM shape
    of the plan's decode step and store the winners in the artifact's cache/kernel_configs.json, which `serve`
    loads (the role of the reference's kernel search at compile time, crates/skein_compile/src/search_cache.rs:73)."""
    cfg = ModelConfig.from_hf_dict(json.loads(config_json))
    source = WeightSource(cfg, weights, seed=seed)
    consts = json.loads(core.cost_constants_json(constants_toml))
    tolerances = consts.get("parity_tolerance_mse", {})
    slo_drift = core.workload_parse(trace_jsonl)["max_accuracy_drift"]
    out_root = Path(out_root)
    out_root.mkdir(parents=True, exist_ok=True)
    replans = 0
    report = None
    while True:
        res = core.extract_plan(config_json, cluster_toml, trace_jsonl, drift_toml, constants_toml, options or {}, SUPPORTED_COMBOS)
        plan_json = res["plan_json"]
        plan = json.loads(plan_json)
        art_dir = build_artifact(plan_json, config_json, out_root, source, tokenizer_json=tokenizer_json)
        if not run_parity:
            break
        ref_plan = all_bf16(plan)
        ref_dir = art_dir / "reference_bf16"
        tmp_root = art_dir / ".ref_tmp"
        built = build_artifact(json.dumps(ref_plan), config_json, tmp_root, source)
        if ref_dir.exists():
            import shutil
            shutil.rmtree(ref_dir)
        built.rename(ref_dir)
        tmp_root.rmdir()
        cand = parity.ArtifactForward(Artifact(art_dir), parity_device)
        refc = parity.ArtifactForward(Artifact(ref_dir), parity_device)
        report = parity.verify(cand, refc, prompts or default_parity_prompts(cfg, n_parity_prompts), plan, slo_drift, tolerances)
        (art_dir / "parity_report.json").write_text(report.to_json())
        if report.passed or replans >= max_replans:
            break
        # feedback edge: make the failing (layer, component, dtype) look at least as bad as the whole budget
        t = core.DriftTable.from_toml(parity.update_drift_table_on_failure(drift_toml, report))
        for f in report.failing:
            if f.dtype != "bf16":
                t.raise_layer_override(f.layer, f.component, f.dtype, max(float(f.mse), slo_drift * 1.01))
        drift_toml = t.to_toml()
        replans += 1
    if enforce_parity and report is not None and not report.passed:
        raise RuntimeError(f"parity gate failed after {replans} re-plans: avg final KL {report.avg_final_kl:.3g}, "
                           f"{len(report.failing)} failing layers")
    if search_budget > 0 and torch.cuda.is_available():
        from ..calibrate import autotune_decode_gemms
        autotune_decode_gemms(cfg, int(plan["parallelism"]["tp"]), int(plan["batching"]["max_batch"]),
                              art_dir / "cache" / "kernel_configs.json", seed=seed, budget=search_budget)
    (art_dir / "runtime_estimator.json").write_text(json.dumps(estimate_runtime(plan_json, config_json, cluster_toml, constants_toml)))
    update_latest_symlink(out_root, art_dir)
    return CompileResult(art_dir, plan, report, replans, drift_toml)
