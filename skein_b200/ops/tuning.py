"""Kernel-configuration cache: measured launch parameters per (operator, shape, dtype, device arch, kernel build).

The kernels are compiled ahead of time, so what is left to search at run time is their launch configuration: for the
weight-streaming GEMM the token-tile width, the grid (whole tiles per CTA or an equal K share per CTA) and the way
split tiles are cut. `tune_gemm` times the candidates on the device (cold launches inside a CUDA graph, median)
and records the winner; `_gemm_launch` (functional.py) consults the active cache before it falls back to its
heuristics. Entries are keyed by a hash of the kernel library, so a rebuilt library never reuses stale winners. The
compile pipeline stores the file as `cache/kernel_configs.json` inside the artifact and `serve` loads it.

Counterpart of the reference's search cache, which memoises the result of its e-graph kernel search per graph and
device (crates/skein_compile/src/search_cache.rs:36-55, 71-150): same role (do the expensive search once, key it by
everything that can invalidate it), different search space.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
from pathlib import Path

_LOCK = threading.Lock()
_ACTIVE: "KernelConfigCache | None" = None
_LIB_HASH: str | None = None


def kernel_build_hash() -> str:
    """First 16 hex digits of the SHA-256 of the kernel library ('nolib' when it has not been built)."""
    global _LIB_HASH
    if _LIB_HASH is None:
        from . import _lib
        p = _lib.lib_path()
        if not p.exists():
            _LIB_HASH = "nolib"
        else:
            h = hashlib.sha256()
            with open(p, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            _LIB_HASH = h.hexdigest()[:16]
    return _LIB_HASH


def device_arch() -> str:
    try:
        import torch
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability()
            return f"sm_{major}{minor}"
    except Exception:
        pass
    return "cpu"


def make_key(op: str, shape, dtype: str = "bf16", arch: str | None = None, build: str | None = None) -> str:
    shape_s = "x".join(str(int(v)) for v in shape)
    return f"{op}|{shape_s}|{dtype}|{arch or device_arch()}|{build or kernel_build_hash()}"


class KernelConfigCache:
    def __init__(self, path: str | os.PathLike | None = None, strict: bool = True):
        """strict=False: an unreadable or corrupt file counts as an empty cache (`load_error` says why) instead of
        raising, so that a damaged cache can never keep a server from starting."""
        self.path = Path(path) if path else None
        self.entries: dict[str, dict] = {}
        self.hits = 0
        self.misses = 0
        self.load_error: str | None = None
        if self.path is not None and self.path.exists():
            try:
                self.load()
            except (OSError, ValueError) as e:   # json.JSONDecodeError is a ValueError
                if strict:
                    raise
                self.entries, self.load_error = {}, f"{type(e).__name__}: {e}"

    def load(self) -> None:
        with open(self.path) as f:
            doc = json.load(f)
        if doc.get("version") != 1:
            raise ValueError(f"{self.path}: unknown kernel-config cache version {doc.get('version')!r}")
        self.entries = dict(doc.get("entries", {}))

    def save(self, path: str | os.PathLike | None = None) -> Path:
        dst = Path(path) if path else self.path
        if dst is None:
            raise ValueError("no path to save the kernel-config cache to")
        dst.parent.mkdir(parents=True, exist_ok=True)
        tmp = dst.with_suffix(dst.suffix + ".tmp")
        with open(tmp, "w") as f:
            json.dump({"version": 1, "entries": self.entries}, f, indent=1, sort_keys=True)
        os.replace(tmp, dst)   # readers never see a half-written file
        return dst

    def get(self, op: str, shape, dtype: str = "bf16", arch=None, build=None) -> dict | None:
        e = self.entries.get(make_key(op, shape, dtype, arch, build))
        if e is None:
            self.misses += 1
        else:
            self.hits += 1
        return e

    def put(self, op: str, shape, config: dict, dtype: str = "bf16", arch=None, build=None) -> None:
        self.entries[make_key(op, shape, dtype, arch, build)] = dict(config)

    def prune_stale(self, build: str | None = None) -> int:
        """Drop entries measured with another kernel build. Returns how many were dropped."""
        b = build or kernel_build_hash()
        stale = [k for k in self.entries if not k.endswith("|" + b)]
        for k in stale:
            del self.entries[k]
        return len(stale)


def active() -> KernelConfigCache | None:
    """The cache the launch paths consult (None: heuristics only). SKEIN_TUNE_CACHE names a file to load at first use."""
    global _ACTIVE
    with _LOCK:
        if _ACTIVE is None and os.environ.get("SKEIN_TUNE_CACHE"):
            _ACTIVE = KernelConfigCache(os.environ["SKEIN_TUNE_CACHE"], strict=False)
        return _ACTIVE


def activate(cache: KernelConfigCache | None) -> None:
    global _ACTIVE
    with _LOCK:
        _ACTIVE = cache


def gemm_shape_key(mode: int, G: int, F: int, K: int, rows: int):
    """Shape part of a GEMM entry: epilogue mode, groups, features per group, K, activation rows (rounded up to 16)."""
    return (mode, G, F, K, (max(rows, 1) + 15) // 16 * 16)


WHOLE_TILE_WASTE_LIMIT = 24   # K-blocks a CTA may idle before equal K shares (and their fix-up) are the better deal


def heuristic_grid(units: int, k_blocks: int, sm_count: int, dual: bool = False) -> int:
    """Grid for a GEMM of `units` output tiles of `k_blocks` K-blocks each when nothing was measured for its shape:
    a whole number of tiles per CTA (fewer CTAs than SMs) when there are between one and two tiles per SM and the
    idle time that costs is below the price of splitting tiles; else 0 (one CTA per SM, equal K shares).
    dual: the gate/up kernel with two accumulators per tile, whose split-tile repair costs twice as much: whole tiles
    measured faster for it at every shape in that range (80.4 vs 84.7 us at Mixtral's 4-rank shard)."""
    if not (sm_count < units <= 2 * sm_count):
        return 0
    per_cta = (units + sm_count - 1) // sm_count
    if not dual and k_blocks * (per_cta - units / sm_count) > WHOLE_TILE_WASTE_LIMIT:
        return 0
    return (units + per_cta - 1) // per_cta


def gemm_candidates(mode: int, G: int, F: int, rows: int, sm_count: int):
    """Launch configurations worth timing for one GEMM shape."""
    per_group = max(1, rows // max(G, 1))
    cap = 128 if mode == 1 else 256
    tiles = sorted({t for t in (16, 32, 64, 128, 256) if t <= cap and t >= min(16, cap) and t < 4 * max(per_group, 16)})
    out = []
    for nt in tiles:
        units = G * ((F + 127) // 128) * max(1, (per_group + nt - 1) // nt)
        grids = {0}
        if units > sm_count:
            per_cta = (units + sm_count - 1) // sm_count
            grids.add((units + per_cta - 1) // per_cta)      # whole tiles per CTA
        for g in sorted(grids):
            for line_cut in (0, 1):
                out.append({"n_tile": nt, "grid": g, "line_cut_only": line_cut})
    return out


def tune_gemm(run, mode: int, G: int, F: int, K: int, rows: int, cache: KernelConfigCache | None = None, iters: int = 9,
              budget: int = 0):
    """Time `run(config)` (one launch of the GEMM with that configuration) for every candidate and record the fastest.

    run: callable taking a dict {"n_tile", "grid", "line_cut_only"}; it must launch on the current stream. Returns
    (best_config, {config_json: median_us}). `budget` > 0 caps the number of candidates that are timed."""
    import torch
    from .functional import workspace
    cache = cache if cache is not None else (active() or KernelConfigCache())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    results = {}
    best, best_us = None, float("inf")
    candidates = gemm_candidates(mode, G, F, rows, workspace().sm_count)
    if budget > 0:
        candidates = candidates[:budget]
    for cfg in candidates:
        try:
            run(cfg)
            torch.cuda.synchronize()
        except RuntimeError:
            continue   # a configuration the kernel refuses (tile width for this epilogue, ...)
        # `reps` cold launches (an L2 flush before each) captured into one CUDA graph: the event timer's resolution
        # (~2 us here) is spread over the whole graph, and the flush costs every candidate the same
        reps = 8
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                flush.zero_()
                run(cfg)
        graph.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3 / reps)
        ts.sort()
        us = ts[len(ts) // 2]       # includes the (constant) flush: only differences between candidates matter
        results[json.dumps(cfg, sort_keys=True)] = us
        if us < best_us:
            best, best_us = cfg, us
    if best is not None:
        cache.put("gemm", gemm_shape_key(mode, G, F, K, rows), dict(best, us_with_flush=round(best_us, 2)))
    return best, results
