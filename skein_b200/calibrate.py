"""`skein calibrate`: measure kernel efficiencies, collective bandwidth and dtype drift on this machine and
rewrite `cost_constants.toml` and the drift table. Measured entries change, everything else (comments,
unmeasured keys, ordering) is preserved byte for byte.

    corpus TOML   workload_trace_path, n_drift_prompts, sampling_strategy (uniform_random | first_n |
                  stratified_by_length), sampling_seed, [[kernel_samples]] {op_kind, dtype, shape, repeats}
    kernel sample timed with CUDA events on the launching stream after warm-up (the reference times
                  `execute` with a host clock: crates/skein_calibrate/src/sampler/kernel_sample.rs:53-173);
                  efficiency = roofline time / measured time, median over samples of the same (op, dtype)
    drift sample  per-layer MSE of a candidate artifact against its bf16 reference, p95 over prompts,
                  attributed to the layer's non-bf16 components

Counterpart of crates/skein_calibrate/src/{lib.rs:51-83, corpus.rs:27-81, measurement.rs:22-99,
prompt_sampling.rs:26-108, cost_writer.rs:28-224, drift_writer.rs:21-42, hardware.rs:14-77}.
"""
from __future__ import annotations

import json
import math
import random
import re
from dataclasses import dataclass, field

from . import core

OP_KINDS = ("gemm", "attention", "elementwise")
DTYPES = ("bf16", "fp16", "fp8_e4m3", "fp8_e5m2", "int8", "int4")
STRATEGIES = ("uniform_random", "first_n", "stratified_by_length")
COLLECTIVES = ("ring_allreduce", "allgather", "reducescatter", "alltoall", "broadcast", "send_recv")


class CalibrationError(ValueError):
    pass


@dataclass
class KernelSample:
    op_kind: str
    dtype: str
    shape: list
    repeats: int = 100


@dataclass
class Corpus:
    workload_trace_path: str
    n_drift_prompts: int
    sampling_strategy: str
    sampling_seed: int
    kernel_samples: list = field(default_factory=list)

    @staticmethod
    def from_toml(text: str) -> "Corpus":
        try:
            j = json.loads(core.toml_to_json(text))
        except Exception as e:
            raise CalibrationError(f"corpus: {e}") from e
        for k in ("workload_trace_path", "n_drift_prompts", "sampling_strategy"):
            if k not in j:
                raise CalibrationError(f"corpus: missing `{k}`")
        c = Corpus(j["workload_trace_path"], int(j["n_drift_prompts"]), j["sampling_strategy"], int(j.get("sampling_seed", 0)))
        for s in j.get("kernel_samples", []):
            for k in ("op_kind", "dtype", "shape"):
                if k not in s:
                    raise CalibrationError(f"corpus: a kernel sample lacks `{k}`")
            c.kernel_samples.append(KernelSample(s["op_kind"], s["dtype"], list(s["shape"]), int(s.get("repeats", 100))))
        c.validate()
        return c

    def validate(self):
        if self.n_drift_prompts <= 0:
            raise CalibrationError("corpus: n_drift_prompts must be positive")
        if self.sampling_strategy not in STRATEGIES:
            raise CalibrationError(f"corpus: unknown sampling_strategy `{self.sampling_strategy}`")
        if not self.workload_trace_path:
            raise CalibrationError("corpus: empty workload_trace_path")
        if not self.kernel_samples:
            raise CalibrationError("corpus: no [[kernel_samples]]")
        for s in self.kernel_samples:
            if s.op_kind not in OP_KINDS:
                raise CalibrationError(f"corpus: unknown op_kind `{s.op_kind}`")
            if s.dtype not in DTYPES:
                raise CalibrationError(f"corpus: unknown dtype `{s.dtype}`")
            if not s.shape or any(int(d) <= 0 for d in s.shape):
                raise CalibrationError(f"corpus: bad shape {s.shape}")
            if s.repeats <= 0:
                raise CalibrationError("corpus: repeats must be positive")


# ---- statistics -----------------------------------------------------------------------------------------------
def median(values):
    if not values:
        return 0.0
    v = sorted(values)
    return v[len(v) // 2]


def p95(values):
    """Linear interpolation between order statistics (type 7)."""
    if not values:
        return 0.0
    v = sorted(values)
    if len(v) == 1:
        return v[0]
    pos = 0.95 * (len(v) - 1)
    lo = int(math.floor(pos))
    hi = min(lo + 1, len(v) - 1)
    return v[lo] * (1 - (pos - lo)) + v[hi] * (pos - lo)


# ---- prompt sampling ------------------------------------------------------------------------------------------------
def sample_prompts(lengths: list[int], n: int, strategy: str, seed: int) -> list[int]:
    """Indices of the trace entries to use as drift prompts. Deterministic in (strategy, seed)."""
    idx = list(range(len(lengths)))
    n = min(n, len(idx))
    if strategy == "first_n":
        return idx[:n]
    rng = random.Random(seed)
    if strategy == "uniform_random":
        return sorted(rng.sample(idx, n))
    if strategy == "stratified_by_length":
        order = sorted(idx, key=lambda i: (lengths[i], i))
        strata = [order[k * len(order) // n:(k + 1) * len(order) // n] for k in range(n)]
        return sorted(rng.choice(s) for s in strata if s)
    raise CalibrationError(f"unknown sampling strategy `{strategy}`")


# ---- byte-stable writers ---------------------------------------------------------------------------------------------
def _fmt(v) -> str:
    return repr(v) if isinstance(v, int) and not isinstance(v, bool) else repr(float(v))


def rewrite_toml_values(text: str, updates: dict) -> str:
    """updates: {(section, key): value}. Rewrites only the value token of matching `key = value` lines, keeping
    alignment, comments and every other byte. A key that is absent from its section is appended to the section."""
    lines = text.split("\n")
    section = ""
    seen = set()
    last_line_of = {}
    for i, line in enumerate(lines):
        m = re.match(r"\s*\[([^\]]+)\]\s*(#.*)?$", line)
        if m:
            section = m.group(1).strip()
            last_line_of[section] = i
            continue
        m = re.match(r"^(\s*)([A-Za-z0-9_]+)(\s*=\s*)([^#\n]*?)(\s*(#.*)?)$", line)
        if not m:
            continue
        last_line_of[section] = i
        key = (section, m.group(2))
        if key in updates:
            lines[i] = f"{m.group(1)}{m.group(2)}{m.group(3)}{_fmt(updates[key])}{m.group(5)}"
            seen.add(key)
    for (sec, k), v in sorted(updates.items()):
        if (sec, k) in seen:
            continue
        if sec in last_line_of:
            at = last_line_of[sec] + 1
            lines.insert(at, f"{k} = {_fmt(v)}")
            last_line_of = {s: (j + 1 if j >= at else j) for s, j in last_line_of.items()}
            last_line_of[sec] = at
        else:
            if lines and lines[-1] != "":
                lines.append("")
            lines += [f"[{sec}]", f"{k} = {_fmt(v)}"]
            last_line_of[sec] = len(lines) - 1
    return "\n".join(lines)


def write_cost_constants(text: str, efficiencies: dict, collective_eff: dict | None = None, hbm_gbps: dict | None = None,
                         peak_tflops: dict | None = None, launch_us: float | None = None,
                         stream_efficiency: dict | None = None) -> str:
    """efficiencies: {(op_kind, dtype): fraction}; collective_eff: {name: fraction}; hbm_gbps: {device_kind: GB/s};
    peak_tflops: {(device_kind, dtype): TFLOP/s}; stream_efficiency: {weight dtype: share of hbm_gbps}."""
    upd = {(f"efficiency.{op}", dt): v for (op, dt), v in efficiencies.items()}
    for k, v in (stream_efficiency or {}).items():
        upd[("stream_efficiency", k)] = v
    for k, v in (collective_eff or {}).items():
        upd[("collective_efficiency", k)] = v
    for k, v in (hbm_gbps or {}).items():
        upd[("hbm_gbps", k)] = v
    for (kind, dt), v in (peak_tflops or {}).items():
        upd[(f"peak_tflops.{kind}", dt)] = v
    if launch_us is not None:
        upd[("", "launch_us_per_kernel")] = launch_us
    return rewrite_toml_values(text, upd)


def fit_fixed_costs(plan_json: str, model_config_json: str, cluster_toml: str, cost_text: str, measured_step_ms: float,
                    kv_tokens: int | None = None) -> dict:
    """Fits the fixed-cost entry of the cost constants that a measured decode step of `plan_json` identifies, so that the
    model reproduces the measurement: `kernel_overhead_us` from a one-GPU plan (everything else in its step is streaming
    time), `collective_fixed_us.ring_allreduce` from a tensor-parallel plan, `collective_fixed_us.alltoall` from a purely
    expert-parallel one. `kv_tokens` is the context length of the measured step (default: the file's decode_kv_tokens).
    Returns {(section, key): value} for rewrite_toml_values."""
    plan = json.loads(plan_json)
    par = plan["parallelism"]
    tp, pp, ep = int(par["tp"]), int(par["pp"]), int(par["ep"])
    if pp > 1 or (tp > 1 and ep > 1):
        raise CalibrationError("a fixed cost is fitted from a step of one GPU, of tensor parallelism or of expert parallelism alone")
    key = ("", "kernel_overhead_us") if tp == ep == 1 else ("collective_fixed_us", "ring_allreduce" if tp > 1 else "alltoall")
    text = rewrite_toml_values(cost_text, {key: 0.0})
    if kv_tokens is not None:
        text = rewrite_toml_values(text, {("representative_workload", "decode_kv_tokens"): int(kv_tokens)})
    b = core.cost_breakdown(plan_json, model_config_json, cluster_toml, text, 0)
    n = b["kernels"] if key[1] == "kernel_overhead_us" else b["collectives"]
    if n <= 0:
        raise CalibrationError("the plan has nothing to attach the fixed cost to")
    return {key: round(max(0.0, measured_step_ms * 1e3 - b["total"]) / n, 2)}


def write_drift_table(text: str, measured: dict) -> str:
    """measured: {(layer, component, dtype): value}; entries are raised monotonically."""
    t = core.DriftTable.from_toml(text)
    for (layer, comp, dt), v in sorted(measured.items()):
        t.raise_layer_override(layer, comp, dt, float(v))
    return t.to_toml()


# ---- measurement ------------------------------------------------------------------------------------------------------
def time_cuda(fn, repeats: int, warmup: int = 3, flush_mb: int = 256) -> float:
    """Median device time of fn() in microseconds: CUDA events on the current stream, L2 flushed between runs."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(repeats):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    return median(ts)


def measure_kernel(sample: KernelSample, peak_tflops: float, hbm_gbps: float):
    """Returns (measured_us, roofline_us). Only dtypes with a kernel in this runtime are measured (bf16 today);
    others return None so that their constants stay untouched."""
    import torch

    from . import ops
    if sample.dtype != "bf16":
        return None
    reps = min(sample.repeats, 30)
    if sample.op_kind == "gemm":
        n_out, k = int(sample.shape[0]), int(sample.shape[1])
        tokens = int(sample.shape[2]) if len(sample.shape) > 2 else 1024
        x = torch.randn(tokens, k, device="cuda").bfloat16()
        w = torch.randn(n_out, k, device="cuda").bfloat16()
        out = torch.empty(tokens, n_out, device="cuda", dtype=torch.bfloat16)
        us = time_cuda(lambda: ops.linear(x, w, out=out), reps)
        roof = max(2.0 * tokens * n_out * k / (peak_tflops * 1e12), (w.numel() + x.numel() + out.numel()) * 2 / (hbm_gbps * 1e9)) * 1e6
        return us, roof
    if sample.op_kind == "elementwise":
        rows, h = int(sample.shape[0]), int(sample.shape[1])
        x = torch.randn(rows, h, device="cuda").bfloat16()
        g = torch.ones(h, device="cuda").bfloat16()
        us = time_cuda(lambda: ops.rmsnorm(x, g, 1e-5), reps)
        return us, 3 * x.numel() * 2 / (hbm_gbps * 1e9) * 1e6
    if sample.op_kind == "attention":
        batch, ctx = int(sample.shape[0]), int(sample.shape[1])
        hq, hkv, d, ps = 32, 8, 128, 16
        blocks = (ctx + ps - 1) // ps
        kv = torch.randn(batch * blocks, 2, hkv, ps, d, device="cuda").bfloat16()
        bt = torch.arange(batch * blocks, device="cuda", dtype=torch.int32).view(batch, blocks)
        q = torch.randn(batch, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        sl = torch.full((batch,), ctx, device="cuda", dtype=torch.int32)
        us = time_cuda(lambda: ops.attn_decode(q, kv, bt, sl, hq, hkv, d, ctx_hint=ctx), reps)
        return us, kv.numel() * 2 / (hbm_gbps * 1e9) * 1e6
    return None


def measure_stream_efficiency(hbm_gbps: float, tokens: int = 64, hidden: int = 4096, inter: int = 14336, experts: int = 8,
                              repeats: int = 10) -> dict:
    """Share of the copy bandwidth the weight-streaming expert GEMMs reach at decode size, per weight dtype the runtime has
    a kernel for: {"bf16": f, "fp8_e4m3": f}. Bytes-weighted over the gate/up and the down projection (the weights of
    `experts` experts of a Mixtral-sized block, `tokens` tokens routed top-2)."""
    import torch

    from . import ops
    from .ops import fp8
    per = max(1, tokens * 2 // experts)
    rows = experts * per
    cnt = torch.full((experts,), per, dtype=torch.int32, device="cuda")
    off = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
    off[1:] = torch.cumsum(cnt, 0)
    out = {}
    for dt in ("bf16", "fp8_e4m3"):
        t_us, n_bytes = 0.0, 0
        for swiglu, (f_out, k_in) in ((True, (inter, hidden)), (False, (hidden, inter))):
            xs = torch.randn(rows, k_in, device="cuda").bfloat16()
            w = (torch.randn(experts, 2 * f_out if swiglu else f_out, k_in, device="cuda") * 0.02).bfloat16()
            y = torch.empty(rows, f_out, dtype=torch.bfloat16, device="cuda")
            if dt == "bf16":
                fn = lambda: ops.grouped_linear(xs, w, cnt, off, swiglu=swiglu, out=y)
                nb = w.numel() * 2
            else:
                wq = fp8.quantize_weight(w)
                del w
                fn = lambda: fp8.grouped_linear_a16(xs, wq, cnt, off, swiglu=swiglu, out=y)
                nb = wq.nbytes()
            t_us += time_cuda(fn, repeats)
            n_bytes += nb
        out[dt] = round(min(1.0, n_bytes / (t_us * 1e-6) / (hbm_gbps * 1e9)), 3)
    return out


def calibrate_kernels(corpus: Corpus, peak_tflops: float, hbm_gbps: float) -> dict:
    """{(op_kind, dtype): median efficiency} over the corpus' kernel samples."""
    by_key: dict = {}
    for s in corpus.kernel_samples:
        r = measure_kernel(s, peak_tflops, hbm_gbps)
        if r is None:
            continue
        us, roof = r
        by_key.setdefault((s.op_kind, s.dtype), []).append(min(1.0, roof / us) if us > 0 else 0.0)
    return {k: round(median(v), 4) for k, v in by_key.items()}


def calibrate_drift(report_layers, plan: dict) -> dict:
    """Per-layer MSEs of a parity run -> {(layer, component, dtype): value} for the non-bf16 components."""
    out = {}
    for l in report_layers:
        d = plan["dtype_map"]["per_layer"][l["layer"]]
        for comp in ("weight", "activation", "kv_cache"):
            if d[comp] != "bf16":
                out[(l["layer"], comp, d[comp])] = l["mse"]
    return out


def autotune_decode_gemms(cfg, tp: int, batch: int, out_path, seed: int = 0, budget: int = 0):
    """Measure launch configurations for the GEMM shapes of one decode step of `cfg` at tensor-parallel degree
    `tp` and `batch` sequences, and write them to `out_path` (the artifact's cache/kernel_configs.json).

    Random weights of the shard shapes and an even routing are used: the winner depends on shapes, not values.
    `budget` > 0 caps the launch configurations timed per shape (the compile command's --search-budget).
    Returns {shape name: best config}. The reference memoises its kernel search the same way
    (crates/skein_compile/src/search_cache.rs:71-150)."""
    import torch

    from . import ops
    from .ops import tuning

    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    bf = lambda *s, std=0.02: (torch.randn(*s, device=dev, generator=g) * std).bfloat16()
    H, D = cfg.hidden_size, cfg.head_dim
    hq, hkv = cfg.num_heads // tp, max(1, cfg.num_kv_heads // tp)
    inter = cfg.intermediate_size // tp
    cache = tuning.KernelConfigCache(out_path)
    x = bf(batch, H, std=1.0)
    found = {}
    found["qkv"] = ops.tune_linear(x, bf((hq + 2 * hkv) * D, H), cache=cache, budget=budget)[0]
    found["o_proj"] = ops.tune_linear(bf(batch, hq * D, std=1.0), bf(H, hq * D), cache=cache, budget=budget)[0]
    found["lm_head"] = ops.tune_linear(x, bf(cfg.vocab_size // tp, H), cache=cache, budget=budget)[0]
    if cfg.is_moe:
        E, k = cfg.num_experts, cfg.top_k
        per = max(1, batch * k // E)
        cnt = torch.full((E,), per, dtype=torch.int32, device=dev)
        off = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        off[1:] = torch.cumsum(cnt, 0)
        found["moe_gate_up"] = ops.tune_grouped(bf(E * per, H, std=1.0), bf(E, 2 * inter, H), cnt, off, True, cache, budget)[0]
        found["moe_down"] = ops.tune_grouped(bf(E * per, inter, std=1.0), bf(E, H, inter), cnt, off, False, cache, budget)[0]
    else:
        found["gate_up"] = ops.tune_linear(x, bf(2 * inter, H), swiglu=True, cache=cache, budget=budget)[0]
        found["down"] = ops.tune_linear(bf(batch, inter, std=1.0), bf(H, inter), cache=cache, budget=budget)[0]
    ops.workspace().check_status()
    cache.save()
    return found
