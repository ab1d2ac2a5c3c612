"""Profiling switches: one environment variable instead of the reference's family of flags.

    SKEIN_PROFILE=0   nothing (default)
    SKEIN_PROFILE=1   CUDA-event timers around named regions (`region("prefill")`), summary via `report()`
    SKEIN_PROFILE=2   additionally NVTX ranges around every region (visible in Nsight tools)
    SKEIN_PROFILE=3   additionally a Chrome trace through torch.profiler (`trace_to(path)`)

Regions are timed on the current stream with CUDA events and read without stalling the step: events are
resolved lazily when `report()` is called. Counterpart of SKEIN_OP_PROFILE / SKEIN_KERNEL_TIMING /
SKEIN_GRAPH_KERNEL_TIMING and the perf-trace SegTimer/StepTimer (vendor/luminal/crates/luminal_cuda_lite/src/
runtime.rs:2364-2500, crates/skein_runtime/src/perf_timing.rs:22-171).
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict

import torch

LEVEL = int(os.environ.get("SKEIN_PROFILE", "0") or 0)
_events = defaultdict(list)
_host_bytes = {"h2d": 0, "d2h": 0}


def count_h2d(nbytes: int) -> None:
    _host_bytes["h2d"] += nbytes


def count_d2h(nbytes: int) -> None:
    _host_bytes["d2h"] += nbytes


def host_bytes() -> dict:
    return dict(_host_bytes)


@contextlib.contextmanager
def region(name: str):
    if LEVEL <= 0 or not torch.cuda.is_available():
        yield
        return
    if LEVEL >= 2:
        torch.cuda.nvtx.range_push(name)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    try:
        yield
    finally:
        e.record()
        _events[name].append((s, e))
        if LEVEL >= 2:
            torch.cuda.nvtx.range_pop()


def report(reset: bool = True) -> dict:
    """{region: {"calls", "total_us", "mean_us"}} from the recorded events (synchronises once)."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    out = {}
    for name, evs in _events.items():
        us = [s.elapsed_time(e) * 1e3 for s, e in evs]
        out[name] = {"calls": len(us), "total_us": sum(us), "mean_us": sum(us) / max(1, len(us))}
    if reset:
        _events.clear()
    return out


@contextlib.contextmanager
def trace_to(path: str):
    """Chrome trace of everything inside the block (torch.profiler / Kineto)."""
    if LEVEL < 3:
        yield
        return
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        yield
    prof.export_chrome_trace(path)
