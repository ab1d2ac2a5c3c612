"""ctypes binding of libskein_kernels.so (the hand-written sm_100a kernels).

The library is plain C ABI: raw device pointers plus a CUDA stream handle. It is loaded lazily;
on a machine with a GPU a missing library is an error (there is no silent fallback to PyTorch on
the device path), on a CPU-only machine the operators in this package use their PyTorch reference
implementations instead.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

MAX_PEERS = 8
MAX_GROUPS = 64

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_native" / "libskein_kernels.so"


class GemmParams(C.Structure):
    """Mirror of SkeinGemmParams in csrc/kernels/gemm_ws.cuh (same field order)."""

    _fields_ = [
        ("W", C.c_void_p), ("X", C.c_void_p), ("out", C.c_void_p), ("residual", C.c_void_p),
        ("group_off", C.c_void_p), ("group_cnt", C.c_void_p),
        ("workspace", C.c_void_p), ("counters", C.c_void_p), ("status", C.c_void_p),
        ("w_scale", C.c_void_p), ("x_scale", C.c_void_p),
        ("peer_flag", C.c_void_p * MAX_PEERS),
        ("epoch", C.c_void_p), ("done_counter", C.c_void_p),
        ("n_peers", C.c_int32), ("G", C.c_int32), ("F", C.c_int32), ("K", C.c_int32),
        ("w_rows_per_group", C.c_int32), ("up_row_off", C.c_int32), ("x_rows", C.c_int32),
        ("t_static", C.c_int32), ("n_tile", C.c_int32), ("ldo", C.c_int32), ("out_col0", C.c_int32),
        ("mode", C.c_int32), ("fp8", C.c_int32), ("stages", C.c_int32), ("grid", C.c_int32),
        ("wait_budget_ms", C.c_int32), ("w_packed", C.c_int32), ("line_cut_only", C.c_int32),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def _sig(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def lib():
    """Load the kernel library (once). Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m skein_b200._build` "
            "(the CUDA path has no PyTorch fallback)")
    L = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    _sig(L, "skein_gemm_ws", i32, [C.POINTER(GemmParams), vp])
    _sig(L, "skein_gemm_ws_workspace_bytes", i64, [C.POINTER(GemmParams)])
    _sig(L, "skein_sm_count", i32, [])
    _sig(L, "skein_reduce_residual_rmsnorm", i32,
         [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, f32, i32, vp, i32, i32, vp, vp, vp])
    _sig(L, "skein_reduce_norm_route", i32,
         [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, f32, i32, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp,
          vp, vp, i32, vp, vp, vp])
    _sig(L, "skein_rope_kv_append", i32,
         [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp])
    _sig(L, "skein_embed_gather", i32, [vp, vp, vp, i32, i32, i32, i32, vp])
    _sig(L, "skein_gather_rows", i32, [vp, vp, vp, i32, i32, vp, vp])
    _sig(L, "skein_attn_decode_workspace_floats", i64, [i32, i32, i32])
    _sig(L, "skein_attn_decode", i32,
         [vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_attn_decode_mma", i32,
         [vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_attn_decode_rope_mma", i32,
         [vp, i64, vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_attn_prefill", i32,
         [vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_attn_decode_tc", i32,
         [vp, i64, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_attn_prefill_tc", i32,
         [vp, i64, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp])
    _sig(L, "skein_router_topk", i32, [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, vp])
    _sig(L, "skein_router_plan", i32, [vp, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp])
    _sig(L, "skein_sample_argmax", i32, [vp, i64, i32, i32, i32, vp, vp, vp])
    _sig(L, "skein_merge_candidates", i32, [vp, vp, i32, i32, i32, vp, vp, vp, i32, vp, vp])
    _sig(L, "skein_sample_topk_topp", i32, [vp, i64, i32, i32, vp, vp, vp, vp, vp, i32, vp, vp])
    _sig(L, "skein_quant_fp8_block128", i32, [vp, vp, vp, i64, i32, vp])
    _sig(L, "skein_dequant_fp8_block128_t", i32, [vp, vp, vp, i64, i32, vp])
    _sig(L, "skein_advance_decode_state", i32, [vp, vp, vp, vp, i32, vp, vp])
    pvp = C.POINTER(C.c_void_p)
    _sig(L, "skein_ep_dispatch_pull", i32, [pvp, pvp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp])
    _sig(L, "skein_ipc_alloc", i32, [pvp, i64])
    _sig(L, "skein_ipc_free", i32, [vp])
    _sig(L, "skein_ipc_get_handle", i32, [vp, C.c_char_p])
    _sig(L, "skein_ipc_open", i32, [C.c_char_p, pvp])
    _sig(L, "skein_ipc_close", i32, [vp])
    _sig(L, "skein_ipc_handle_bytes", i32, [])
    _sig(L, "skein_publish_rows", i32, [vp, i64, vp, pvp, i32, vp, vp, vp])
    _sig(L, "skein_pull_collective", i32, [i32, pvp, i32, i32, i64, vp, vp, vp, vp, i32, vp])
    _sig(L, "skein_argmax_push", i32, [vp, i64, i32, i32, i32, pvp, pvp, pvp, i32, vp, vp, vp])
    _sig(L, "skein_copy_pages", i32, [vp, vp, vp, vp, i32, i64, vp])
    _sig(L, "skein_wait_flag", i32, [vp, i32, i32, vp, vp])
    for name, rt, at in _OPTIONAL:
        if hasattr(L, name):
            _sig(L, name, rt, at)
    _LIB = L
    return L


# Entry points that newer builds add; bound when present.
_OPTIONAL: list = []


def register_optional(name, restype, argtypes):
    _OPTIONAL.append((name, restype, argtypes))
    if _LIB is not None and hasattr(_LIB, name):
        _sig(_LIB, name, restype, argtypes)


def ptr(t) -> int | None:
    """Device (or host) address of a tensor, None for None."""
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


# launch counter: every kernel launched through this package increments it (bench.py reports it)
_launches = 0


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches
