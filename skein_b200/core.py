"""Python face of the C++ host core (skein_b200/_native/_skein_core*.so).

Everything here is implemented in C++ (csrc/core, csrc/runtime): IR and importers, plan, cluster and
workload parsing, the cost model, the placement search with its dtype DP, lowering (topology,
segments, shard roles, io manifest), the paged-KV block manager with radix prefix cache, the
continuous batcher, parity math, drift table / monitor, speculative acceptance, CPU reference
collectives and metrics. Build with `python -m skein_b200._build`.
"""
from __future__ import annotations

import importlib.util
import sys

from . import _build


def _load():
    path = _build.core_lib_path()
    if not path.exists():
        raise ImportError(f"{path} is missing: build it with `python -m skein_b200._build`")
    spec = importlib.util.spec_from_file_location("_skein_core", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_core = _load()
sys.modules.setdefault("skein_b200._skein_core", _core)

globals().update({k: getattr(_core, k) for k in dir(_core) if not k.startswith("__")})
