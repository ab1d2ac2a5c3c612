"""Parity gate: compare a candidate forward against a bf16 reference, per layer (MSE of the residual
stream after every block) and at the output (KL of the final-token distributions).

    pass  <=>  mean final KL <= slo.max_accuracy_drift  and  every layer's MSE <= tolerance(dtype of that layer)

A failing layer is reported as (layer, component, dtype) and raises that entry of the drift table
(monotonic maximum), so the next `extract` steers away from the dtype: the only upward data edge in
the pipeline.

Forwards are anything with `run(prompt_ids) -> (hidden_after_block list of [T, H] fp32, final_logits [V] fp32)`:
  ArtifactForward   a compiled artifact run through the runtime's decoder (candidate, or its reference_bf16)
  DenseForward      the cache-free straight-line model (the "HF-style" oracle)
  HFForward         HuggingFace transformers on the original checkpoint (the outside oracle)
  and the fakes used by the tests (offset / tilted forwards).

Counterpart of crates/skein_parity/src/verify.rs:46-315, comparison.rs:16-72, tolerance.rs:14-57, report.rs:10-36,
drift_update.rs:30, reference.rs:29-104 (there the oracle is a Python subprocess; here PyTorch is in process).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict

import torch

from .. import core
from ..models import dense_reference
from ..models.decoder import BatchInputs, Decoder
from .artifact import Artifact


@dataclass
class LayerReport:
    layer: int
    mse: float
    tolerance: float
    dtype: str
    passed: bool


@dataclass
class FailingLayer:
    layer: int
    component: str
    dtype: str
    mse: float


@dataclass
class ParityReport:
    passed: bool
    avg_final_kl: float
    max_accuracy_drift: float
    layers: list = field(default_factory=list)
    failing: list = field(default_factory=list)
    prompts: int = 0

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2)


def tolerance_for_layer(plan: dict, layer: int, tolerances: dict) -> tuple[float, str, str]:
    """(MSE tolerance, component, dtype) of a block: the loosest non-bf16 dtype among its components decides."""
    d = plan["dtype_map"]["per_layer"][layer]
    best = None
    for comp in ("weight", "activation", "kv_cache"):
        t = tolerances.get(d[comp], 1e-3)
        if d[comp] != "bf16" and (best is None or t > best[0]):
            best = (t, comp, d[comp])
    return best or (tolerances.get("bf16", 1e-3), "weight", "bf16")


class DenseForward:
    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights

    def run(self, prompt_ids):
        hid = []
        logits = dense_reference.forward_full(self.cfg, self.w, torch.tensor(prompt_ids), capture_hidden=hid)
        return [h.float().cpu() for h in hid], logits[-1].float().cpu()


class HFForward:
    """The HuggingFace `transformers` implementation of the model as the oracle: loads a checkpoint directory
    (config.json + safetensors) with AutoModelForCausalLM, runs the prompt in fp32 (or bf16) and returns the residual
    stream after every decoder layer and the last position's logits. This is the one reference that is not written
    by the same hand as the kernels: it pins the RoPE convention, the router's renormalisation and the GQA head
    order from outside. Role of the reference's verify_reference.py subprocess
    (crates/skein_parity/src/reference.rs:65-104, crates/skein_parity/reference/verify_reference.py)."""

    def __init__(self, checkpoint_dir, dtype: str = "float32"):
        try:
            import transformers
        except ImportError as e:     # the caller falls back to the in-process dense oracle
            raise RuntimeError("the `transformers` package is not installed") from e
        td = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        self.model = transformers.AutoModelForCausalLM.from_pretrained(str(checkpoint_dir), dtype=td).eval()

    @torch.no_grad()
    def run(self, prompt_ids):
        hid, hooks = [], []
        for layer in self.model.model.layers:
            hooks.append(layer.register_forward_hook(
                lambda _m, _i, out: hid.append((out[0] if isinstance(out, tuple) else out)[0].float().cpu())))
        try:
            out = self.model(input_ids=torch.tensor([list(prompt_ids)], dtype=torch.long), use_cache=False)
        finally:
            for h in hooks:
                h.remove()
        return hid, out.logits[0, -1].float().cpu()


class DecoderForward:
    """Runs a prompt through a (single-rank) runtime Decoder as one prefill chunk."""

    def __init__(self, decoder: Decoder):
        self.dec = decoder

    def run(self, prompt_ids):
        dec = self.dec
        dev = dec.device
        T = len(prompt_ids)
        n_blocks = (T + dec.page_size - 1) // dec.page_size
        if n_blocks > dec.num_pages:
            raise ValueError("prompt does not fit the decoder's KV pool")
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        bt = torch.arange(n_blocks, dtype=torch.int32, device=dev).unsqueeze(0)
        inp = BatchInputs(token_ids=i32(prompt_ids), positions=i32(list(range(T))), block_table=bt, seq_lens=i32([T]),
                          is_prefill=True, seq_of_token=i32([0] * T), q_start=i32([0]), q_len=i32([T]), max_q_len=T,
                          logit_rows=torch.tensor([T - 1], dtype=torch.int64, device=dev))
        dec.capture_hidden = []
        try:
            _, lg = dec.forward(inp)
            hid = dec.capture_hidden
        finally:
            dec.capture_hidden = None
        return hid, lg[0].float().cpu()


class ArtifactForward(DecoderForward):
    def __init__(self, artifact: Artifact, device="cpu", num_pages: int = 64):
        # the gate measures what the stored (possibly quantised) weights do to the numerics, so it runs the
        # model reassembled from all shards on one device; sharded execution is covered by the TP tests
        w = artifact.load_full_weights(device)
        super().__init__(Decoder(artifact.cfg, w, None, num_pages=num_pages, page_size=16,
                                 max_pos=min(artifact.cfg.max_position_embeddings, num_pages * 16)))


def verify(candidate, reference, prompts, plan: dict, max_accuracy_drift: float, tolerances: dict) -> ParityReport:
    n_layers = len(plan["dtype_map"]["per_layer"])
    layer_mse = [0.0] * n_layers
    kls = []
    for p in prompts:
        ch, cl = candidate.run(p)
        rh, rl = reference.run(p)
        if len(ch) != n_layers or len(rh) != n_layers:
            raise ValueError(f"forward returned {len(ch)}/{len(rh)} hidden states, the plan has {n_layers} layers")
        for i in range(n_layers):
            layer_mse[i] = max(layer_mse[i], core.mse(ch[i].flatten().tolist(), rh[i].flatten().tolist()))
        kls.append(core.kl_divergence(rl.tolist(), cl.tolist()))
    avg_kl = sum(kls) / max(1, len(kls))
    layers, failing = [], []
    for i in range(n_layers):
        tol, comp, dt = tolerance_for_layer(plan, i, tolerances)
        ok = layer_mse[i] <= tol
        layers.append(LayerReport(i, layer_mse[i], tol, dt, ok))
        if not ok:
            failing.append(FailingLayer(i, comp, dt, layer_mse[i]))
    passed = avg_kl <= max_accuracy_drift and not failing
    if avg_kl > max_accuracy_drift and not failing:
        # only the output drifted: blame the layer with the largest relative error among the quantised ones
        cands = [l for l in layers if l.dtype != "bf16"] or layers
        worst = max(cands, key=lambda l: l.mse / l.tolerance)
        _, comp, dt = tolerance_for_layer(plan, worst.layer, tolerances)
        failing.append(FailingLayer(worst.layer, comp, dt, worst.mse))
    return ParityReport(passed, avg_kl, max_accuracy_drift, layers, failing, len(prompts))


def update_drift_table_on_failure(drift_toml: str, report: ParityReport) -> str:
    """Returns the new drift-table text: each failing (layer, component, dtype) is raised to the measured MSE,
    never lowered."""
    t = core.DriftTable.from_toml(drift_toml)
    for f in report.failing:
        if f.dtype == "bf16":
            continue
        t.raise_layer_override(f.layer, f.component, f.dtype, float(f.mse))
    return t.to_toml()
