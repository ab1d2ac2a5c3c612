"""Per-operator timing of a served step.

`OpProfiler` wraps every operator of `skein_b200.ops` (and the communicator's fused collectives) with a pair of
CUDA events on the launching stream, runs whatever the caller runs inside the `with` block EAGERLY (kernels inside
a captured graph cannot be timed one by one, so the profiled step is launched kernel by kernel, which also exposes
each launch's host cost), and reports a table: calls, total and mean device time, share of the step.

    with OpProfiler() as prof:
        runner._decode_body(bucket, feedback=False)          # one decode step, eager
    print(prof.table())

`skein bench --artifact ... --op-profile` prints the table for one decode step of the served batch, and
SKEIN_OP_PROFILE=1 makes the engine profile its first full decode step and log the table.

Counterpart of the reference's SKEIN_OP_PROFILE per-op table and its compute/communication split
(vendor/luminal/crates/luminal_cuda_lite/src/runtime.rs:2364-2500, crates/skein_runtime/src/perf_timing.rs:22-171).
"""
from __future__ import annotations

import functools
import time
from collections import OrderedDict

import torch

# operators whose device time is communication (waiting for and pulling peers' data) rather than local compute
COMM_OPS = ("publish", "pull", "all_gather", "all_reduce", "reduce_scatter", "all_to_all", "vocab_parallel_argmax")


class OpProfiler:
    def __init__(self, extra_objects=()):
        """extra_objects: communicators (parallel.tp.TPComm) whose collective methods should be timed as well."""
        self.records = []          # (name, start event, end event, host seconds)
        self._patched = []
        self.extra_objects = list(extra_objects)
        self._depth = 0

    def _wrap(self, name, fn):
        @functools.wraps(fn)
        def timed(*a, **k):
            if self._depth > 0 or not torch.cuda.is_available():      # only the outermost operator is recorded
                return fn(*a, **k)
            self._depth += 1
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            s.record()
            try:
                return fn(*a, **k)
            finally:
                e.record()
                self.records.append((name, s, e, time.perf_counter() - t0))
                self._depth -= 1
        return timed

    def __enter__(self):
        from .. import ops
        from ..ops import fp8, functional
        names = ("linear", "swiglu_linear", "grouped_linear", "linear_push", "reduce_residual_rmsnorm", "reduce_norm_route",
                 "rmsnorm", "rope_kv_append", "attn_decode", "attn_decode_rope", "attn_prefill", "router_topk", "route",
                 "router_plan", "gather_rows", "embed", "sample_argmax", "sample", "quant_fp8_block128", "advance_decode_state")
        for mod in (functional, ops):
            for n in names:
                if hasattr(mod, n):
                    self._patch(mod, n, n)
        for n in ("linear", "grouped_linear", "linear_publish"):
            self._patch(fp8, n, "fp8." + n)
        for obj in self.extra_objects:
            for n in ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "vocab_parallel_argmax", "embed_reduce",
                      "reduce_scatter_norm", "gather_rows"):
                if hasattr(obj, n):
                    self._patch(obj, n, "comm." + n)
        return self

    def _patch(self, owner, attr, label):
        orig = getattr(owner, attr)
        if getattr(orig, "_skein_timed", False):
            return
        w = self._wrap(label, orig)
        w._skein_timed = True
        setattr(owner, attr, w)
        self._patched.append((owner, attr, orig))

    def __exit__(self, *exc):
        for owner, attr, orig in reversed(self._patched):
            setattr(owner, attr, orig)
        self._patched = []
        return False

    def summary(self) -> "OrderedDict[str, dict]":
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out: "OrderedDict[str, dict]" = OrderedDict()
        for name, s, e, host in self.records:
            d = out.setdefault(name, {"calls": 0, "device_us": 0.0, "host_us": 0.0})
            d["calls"] += 1
            d["device_us"] += s.elapsed_time(e) * 1e3
            d["host_us"] += host * 1e6
        total = sum(d["device_us"] for d in out.values()) or 1.0
        for name, d in out.items():
            d["mean_us"] = d["device_us"] / d["calls"]
            d["share"] = d["device_us"] / total
            d["comm"] = any(k in name for k in COMM_OPS)
        return out

    def table(self) -> str:
        sm = self.summary()
        rows = sorted(sm.items(), key=lambda kv: -kv[1]["device_us"])
        lines = [f"{'operator':34s} {'calls':>6s} {'device us':>11s} {'mean us':>9s} {'share':>7s} {'host us':>9s}"]
        for name, d in rows:
            lines.append(f"{name:34s} {d['calls']:6d} {d['device_us']:11.1f} {d['mean_us']:9.2f} {100 * d['share']:6.1f}% {d['host_us']:9.1f}")
        tot = sum(d["device_us"] for d in sm.values())
        comm = sum(d["device_us"] for d in sm.values() if d["comm"])
        lines.append(f"{'total (eager, serialised)':34s} {sum(d['calls'] for d in sm.values()):6d} {tot:11.1f} {'':9s} {'':7s}")
        lines.append(f"{'  of which collectives':34s} {'':6s} {comm:11.1f}")
        return "\n".join(lines)
