"""One typed place for the runtime switches.

The fast path is the default path, so there are few switches and all of them exist for comparisons and debugging.
Each is one field of `RuntimeConfig` with one environment variable behind it; the kernels' Python wrappers read the
variables, and this module is how a user sets them as a group: from a `[runtime]` table of a TOML file
(`skein serve --runtime-config file.toml`), from the environment, or in code, with unknown keys and bad values
rejected before anything is launched. `apply_to_env` exports the configuration, so the rank processes that the
launcher spawns inherit it.

The reference spreads about 95 `SKEIN_*` variables over its crates (planner overrides, kernel variants, device-resident
paths; e.g. crates/skein_runtime/src/distributed/gpu_rank.rs:466-555 reads ten of them for graph capture alone) and has
`[runtime]` keys in cluster/cost_constants.toml:140-160 for ports and buffer sizes.
"""
from __future__ import annotations

import dataclasses
import os
import tomllib
from dataclasses import dataclass


class RuntimeConfigError(ValueError):
    pass


def _bool(v) -> bool:
    if isinstance(v, bool):
        return v
    if isinstance(v, int) and v in (0, 1):
        return bool(v)
    if isinstance(v, str) and v.strip().lower() in ("0", "1", "true", "false", "on", "off"):
        return v.strip().lower() in ("1", "true", "on")
    raise RuntimeConfigError(f"expected a boolean, got {v!r}")


# field -> (environment variable, parser, allowed values or None)
_FIELDS = {
    "comm": ("SKEIN_COMM", str, ("fused", "unfused", "nccl")),
    "multimem": ("SKEIN_MULTIMEM", _bool, None),
    "profile": ("SKEIN_PROFILE", int, (0, 1, 2, 3)),
    "attn_decode": ("SKEIN_ATTN_DECODE", str, ("auto", "tc", "mma", "scalar")),
    "attn_splits": ("SKEIN_ATTN_SPLITS", int, None),
    "ep_dp_attention": ("SKEIN_EP_DP_ATTENTION", _bool, None),
    "fuse_route": ("SKEIN_FUSE_ROUTE", _bool, None),
    "fuse_rope": ("SKEIN_FUSE_ROPE", _bool, None),
    "gemm_aligned": ("SKEIN_GEMM_ALIGNED", _bool, None),
    "gemm_autogrid": ("SKEIN_GEMM_AUTOGRID", _bool, None),
    "pack_moe": ("SKEIN_PACK_MOE", _bool, None),
    "pdl": ("SKEIN_PDL", _bool, None),
    "pp_continuous": ("SKEIN_PP_CONTINUOUS", _bool, None),
    "tune_cache": ("SKEIN_TUNE_CACHE", str, None),
    "grid_barrier_ms": ("SKEIN_GRID_BARRIER_MS", int, None),
    "gemm_wait_ms": ("SKEIN_GEMM_WAIT_MS", int, None),
    "peer_wait_ms": ("SKEIN_PEER_WAIT_MS", int, None),
}


@dataclass(frozen=True)
class RuntimeConfig:
    comm: str = "fused"            # tensor-parallel all-reduce: fused into the GEMM / reduce kernels, or a library call
    multimem: bool = False         # sum the tensor-parallel partials inside the NVSwitch (multicast-bound heap)
    profile: int = 0               # 0 off, 1 CUDA-event region timers, 2 + NVTX ranges, 3 + Chrome trace
    attn_decode: str = "auto"      # decode attention kernel: tcgen05 / mma.sync chosen per launch, or one of them forced
    attn_splits: int = 0           # split-KV factor (0: chosen per launch)
    ep_dp_attention: bool = True   # pure expert parallelism: each rank attends over its own share of the sequences
    fuse_route: bool = True        # router inside the post-attention reduce kernel
    fuse_rope: bool = True         # RoPE + KV append inside the decode attention kernel
    gemm_aligned: bool = True      # tile-aligned K pieces when there are fewer tiles than SMs
    gemm_autogrid: bool = True     # whole tiles per CTA when that wastes little
    pack_moe: bool = True          # tile-packed expert weights
    pdl: bool = False              # programmatic dependent launch between the per-layer kernels
    pp_continuous: bool = False    # pipeline parallelism: one group of sequences per stage in flight across engine steps
    tune_cache: str = ""           # kernel-configuration cache to load ("" = the artifact's own, if any)
    grid_barrier_ms: int = 2000    # budget of the grid-wide arrival counter in the fused reduce + router kernel
    gemm_wait_ms: int = 2000       # budget of the GEMM's pipeline waits and of its wait for the other pieces of a split tile
    peer_wait_ms: int = 10000      # budget of a reduce kernel's wait for a tensor-parallel peer's flag

    def __post_init__(self):
        for name, (_, _, allowed) in _FIELDS.items():
            v = getattr(self, name)
            if allowed is not None and v not in allowed:
                raise RuntimeConfigError(f"runtime.{name} = {v!r}: expected one of {list(allowed)}")
        if not 0 <= self.attn_splits <= 16:
            raise RuntimeConfigError(f"runtime.attn_splits = {self.attn_splits}: expected 0..16")
        for name in ("grid_barrier_ms", "gemm_wait_ms", "peer_wait_ms"):
            if not 1 <= getattr(self, name) <= 3600000:
                raise RuntimeConfigError(f"runtime.{name} = {getattr(self, name)}: expected 1..3600000 milliseconds")
        if self.multimem and self.comm == "nccl":
            raise RuntimeConfigError("runtime.multimem needs runtime.comm = \"fused\" (or \"unfused\")")

    # ---- sources -----------------------------------------------------------------------------------------------
    @classmethod
    def from_mapping(cls, table: dict, base: "RuntimeConfig | None" = None) -> "RuntimeConfig":
        unknown = sorted(set(table) - set(_FIELDS))
        if unknown:
            raise RuntimeConfigError(f"unknown runtime key(s) {unknown}; known: {sorted(_FIELDS)}")
        values = dataclasses.asdict(base) if base is not None else {}
        for name, raw in table.items():
            _, parse, _ = _FIELDS[name]
            try:
                if parse is int and isinstance(raw, bool):
                    raise ValueError("a boolean is not a number")
                values[name] = parse(raw)
            except (TypeError, ValueError) as e:
                if isinstance(e, RuntimeConfigError):
                    raise RuntimeConfigError(f"runtime.{name}: {e}") from e
                raise RuntimeConfigError(f"runtime.{name} = {raw!r}: not a valid {parse.__name__}") from e
        return cls(**values)

    @classmethod
    def from_toml(cls, text: str, base: "RuntimeConfig | None" = None) -> "RuntimeConfig":
        try:
            doc = tomllib.loads(text)
        except tomllib.TOMLDecodeError as e:
            raise RuntimeConfigError(f"runtime config: {e}") from e
        table = doc.get("runtime", {})
        if not isinstance(table, dict):
            raise RuntimeConfigError("runtime config: [runtime] must be a table")
        return cls.from_mapping(table, base)

    @classmethod
    def from_env(cls, env: dict | None = None, base: "RuntimeConfig | None" = None) -> "RuntimeConfig":
        env = os.environ if env is None else env
        table = {name: env[var] for name, (var, _, _) in _FIELDS.items() if var in env and env[var] != ""}
        return cls.from_mapping(table, base)

    @classmethod
    def resolve(cls, toml_text: str | None = None, env: dict | None = None, overrides: dict | None = None) -> "RuntimeConfig":
        """Defaults, then the file, then the environment, then explicit overrides (the command line)."""
        cfg = cls()
        if toml_text is not None:
            cfg = cls.from_toml(toml_text, cfg)
        cfg = cls.from_env(env, cfg)
        if overrides:
            cfg = cls.from_mapping({k: v for k, v in overrides.items() if v is not None}, cfg)
        return cfg

    # ---- sinks -------------------------------------------------------------------------------------------------
    def to_env(self) -> dict:
        """The environment variables that express this configuration (booleans as 0/1; an empty path is left out)."""
        out = {}
        for name, (var, _, _) in _FIELDS.items():
            v = getattr(self, name)
            if isinstance(v, bool):
                out[var] = "1" if v else "0"
            elif v != "":
                out[var] = str(v)
        if self.attn_splits == 0:
            out.pop("SKEIN_ATTN_SPLITS", None)      # 0 means "chosen per launch", which is what an unset variable says
        return out

    def apply_to_env(self, env: dict | None = None) -> dict:
        env = os.environ if env is None else env
        env.update(self.to_env())
        if self.tune_cache == "":
            env.pop("SKEIN_TUNE_CACHE", None)
        if self.attn_splits == 0:
            env.pop("SKEIN_ATTN_SPLITS", None)
        return env

    def describe(self) -> dict:
        return dataclasses.asdict(self)
