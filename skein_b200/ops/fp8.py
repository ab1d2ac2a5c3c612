"""Block-scaled fp8 (e4m3, one fp32 scale per 1 x 128 block along K) linear operators.

Two forms:
  * weights fp8, activations bf16 (`linear_a16`, `grouped_linear_a16`, `linear_publish_a16`): what the plan's dtype
    map selects (weight fp8_e4m3, activation bf16). The weight-streaming GEMM (csrc/kernels/gemm_ws.cu) moves the
    e4m3 tiles, turns them into scaled bf16 in shared memory and keeps one accumulator for the whole K range, so
    the bytes of a decode step halve and nothing else changes. This is the form the decoder uses.
  * both operands fp8 (`linear`, `grouped_linear`, `linear_publish`; csrc/kernels/gemm_ws_fp8.cu): activations
    quantised on the fly (`ops.quant_fp8_block128`), e4m3 x e4m3 on the tensor cores, both scales applied per K-block.
Weights are quantised once (`quantize_weight`). On CPU the same math runs through the fp32 reference (dequantise,
matmul).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib, functional as F, reference as ref

_lib.register_optional("skein_gemm_ws_fp8", C.c_int, [C.POINTER(_lib.GemmParams), C.c_void_p])


class Fp8Weight:
    """q: e4m3 [rows, K] (or [G, rows, K]); scale_t: fp32 [K/128, rows_total] (K-block major, the layout the
    kernel reads with coalesced loads). `shape` is the logical shape."""

    def __init__(self, q: torch.Tensor, scale_t: torch.Tensor, shape):
        self.q, self.scale_t, self.shape = q, scale_t, tuple(shape)
        self.device = q.device

    @property
    def is_cuda(self):
        return self.q.is_cuda

    def dequant(self) -> torch.Tensor:
        """The weight as bf16, in its logical shape. On a GPU one kernel pass (csrc/kernels/quant.cu)."""
        rows_total = self.scale_t.shape[1]
        K = self.shape[-1]
        if self.q.is_cuda:
            out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.q.device)
            _lib.check(_lib.lib().skein_dequant_fp8_block128_t(self.q.data_ptr(), self.scale_t.data_ptr(), out.data_ptr(),
                                                               rows_total, K, _lib.stream_ptr()), "dequant_fp8_block128")
            _lib.count_launch()
            return out
        w = ref.dequant_fp8_block128(self.q.reshape(rows_total, K), self.scale_t.t().contiguous())
        return w.view(*self.shape).to(torch.bfloat16)

    def nbytes(self) -> int:
        return self.q.numel() + self.scale_t.numel() * 4

    def copy_(self, src: "Fp8Weight"):
        """In-place update (hot swap keeps the storage that captured CUDA graphs point at)."""
        if tuple(src.shape) != self.shape:
            raise ValueError(f"fp8 weight shape {tuple(src.shape)} does not match {self.shape}")
        self.q.copy_(src.q)
        self.scale_t.copy_(src.scale_t)
        return self


def quantize_weight(w: torch.Tensor, pow2_scales: bool = True) -> Fp8Weight:
    """e4m3 with one fp32 scale per 1 x 128 block along K. With `pow2_scales` (the default for weights) every scale is
    the smallest power of two that brings the block's largest magnitude inside the e4m3 range: e4m3 is a floating-point
    format, so this costs no relative precision, and the GEMM's in-kernel rescaling of the tile to bf16 is then exact."""
    shape = tuple(w.shape)
    K = shape[-1]
    w2 = w.reshape(-1, K).contiguous()
    if not pow2_scales:
        q, s = F.quant_fp8_block128(w2) if w2.is_cuda else ref.quant_fp8_block128(w2)
    else:
        q, s = ref.quant_fp8_block128(w2, pow2_scales=True)      # plain tensor ops: runs on the weight's device
    return Fp8Weight(q.view(*shape), s.t().contiguous(), shape)


def _launch(p, what):
    ws = F.workspace()
    p.workspace = ws.gemm_ws.data_ptr()
    p.counters = ws.gemm_counters.data_ptr()
    p.status = ws.status.data_ptr()
    L = _lib.lib()
    if not hasattr(L, "skein_gemm_ws_fp8"):
        raise RuntimeError("libskein_kernels.so was built without the fp8 GEMM; rebuild with `python -m skein_b200._build`")
    _lib.check(L.skein_gemm_ws_fp8(C.byref(p), _lib.stream_ptr()), what)
    _lib.count_launch()


def _n_tile(rows_hint: int, dual: bool) -> int:
    """Token-tile width the fp8 kernel is instantiated for: 16, 32 or (single accumulator only) 64."""
    for t in ((16, 32) if dual else (16, 32, 64)):
        if rows_hint <= t:
            return t
    return 32 if dual else 64


def _ref_linear(xq, xs, w: Fp8Weight, swiglu):
    x = ref.dequant_fp8_block128(xq, xs)
    wd = w.dequant().float()
    if swiglu:
        I = wd.shape[-2] // 2
        return (torch.nn.functional.silu(x @ wd[:I].t()) * (x @ wd[I:].t())).to(torch.bfloat16)
    return (x @ wd.t()).to(torch.bfloat16)


def linear(xq, xs, w: Fp8Weight, swiglu: bool = False, out=None, n_tile=None):
    """xq e4m3 [T, K], xs fp32 [T, K/128] -> bf16 [T, F] (F = rows, or rows/2 with the SwiGLU pair epilogue)."""
    if not xq.is_cuda:
        return _ref_linear(xq, xs, w, swiglu)
    T, K = xq.shape
    rows = w.shape[-2]
    Fo = rows // 2 if swiglu else rows
    if out is None:
        out = torch.empty(T, Fo, dtype=torch.bfloat16, device=xq.device)
    if T == 0:
        return out
    p = _lib.GemmParams()
    p.W, p.X, p.out = w.q.data_ptr(), xq.data_ptr(), out.data_ptr()
    p.w_scale, p.x_scale = w.scale_t.data_ptr(), xs.data_ptr()
    p.G, p.F, p.K = 1, Fo, K
    p.w_rows_per_group, p.up_row_off = rows, (Fo if swiglu else 0)
    p.x_rows, p.t_static = T, T
    p.n_tile = n_tile or _n_tile(T, swiglu)
    p.ldo, p.mode, p.fp8 = out.stride(0), (1 if swiglu else 0), 1
    _launch(p, "fp8 linear")
    return out


def grouped_linear(xq, xs, w: Fp8Weight, counts, offsets, swiglu: bool = False, out=None, n_tile=None, rows_hint=None):
    """Per-expert fp8 linear over expert-sorted rows. w.shape = [E, rows, K]."""
    if not xq.is_cuda:
        x = ref.dequant_fp8_block128(xq, xs).to(torch.bfloat16)
        return ref.grouped_linear(x, w.dequant(), counts, offsets, swiglu)
    R, K = xq.shape
    E, rows = w.shape[0], w.shape[1]
    Fo = rows // 2 if swiglu else rows
    if out is None:
        out = torch.empty(R, Fo, dtype=torch.bfloat16, device=xq.device)
    if R == 0:
        return out
    if n_tile is None:
        avg = (rows_hint if rows_hint is not None else R) / E
        n_tile = _n_tile(int(math.ceil(avg * 1.5)), swiglu)
    p = _lib.GemmParams()
    p.W, p.X, p.out = w.q.data_ptr(), xq.data_ptr(), out.data_ptr()
    p.w_scale, p.x_scale = w.scale_t.data_ptr(), xs.data_ptr()
    p.G, p.F, p.K = E, Fo, K
    p.w_rows_per_group, p.up_row_off = rows, (Fo if swiglu else 0)
    p.x_rows, p.t_static = R, R
    p.group_off, p.group_cnt = offsets.data_ptr(), counts.data_ptr()
    p.n_tile = n_tile
    p.ldo, p.mode, p.fp8 = out.stride(0), (1 if swiglu else 0), 1
    _launch(p, "fp8 grouped_linear")
    return out


def linear_publish(xq, xs, w: Fp8Weight, out_local, peer_flag, epoch, done_counter, ldo, grouped=None, n_tile=None,
                   rows_hint=None):
    """Row-parallel fp8 projection that publishes its partial result to the tensor-parallel peers: the bf16 partial
    goes into `out_local` (peer-mapped), then this rank's flag on every peer is set (same contract as
    ops.linear_push; csrc/kernels/gemm_ws_fp8.cu mode 2)."""
    R, K = xq.shape
    p = _lib.GemmParams()
    p.W, p.X, p.out = w.q.data_ptr(), xq.data_ptr(), out_local.data_ptr()
    p.w_scale, p.x_scale = w.scale_t.data_ptr(), xs.data_ptr()
    if grouped is None:
        rows = w.shape[-2]
        p.G, p.F, p.K = 1, rows, K
        p.w_rows_per_group = rows
        p.n_tile = n_tile or _n_tile(R, False)
    else:
        counts, offsets = grouped
        E, rows = w.shape[0], w.shape[1]
        p.G, p.F, p.K = E, rows, K
        p.w_rows_per_group = rows
        p.group_off, p.group_cnt = offsets.data_ptr(), counts.data_ptr()
        avg = (rows_hint if rows_hint is not None else R) / E
        p.n_tile = n_tile or _n_tile(int(math.ceil(avg * 1.5)), False)
    p.up_row_off = 0
    p.x_rows, p.t_static = R, R
    p.ldo, p.mode, p.fp8 = ldo, 2, 1
    p.n_peers = len(peer_flag)
    for i, pf in enumerate(peer_flag):
        p.peer_flag[i] = pf
    p.epoch = epoch.data_ptr()
    p.done_counter = done_counter.data_ptr()
    _launch(p, "fp8 linear_publish")


# ---- fp8 weights, bf16 activations -----------------------------------------------------------------------------------
def _a16_n_tile(rows_hint: int, dual: bool) -> int:
    """Token-tile width of the e4m3-weight form: the converted weight tiles share the 512 tensor-memory columns with the
    two accumulators, which leaves room for 64 tokens per tile with the SwiGLU pair epilogue and 128 without."""
    return min(F.pick_n_tile(rows_hint, dual), 64 if dual else 128)


def _a16_params(x, w: Fp8Weight, out, F_out, n_tile, mode):
    w2d = w.q.view(-1, w.shape[-1])
    p = F._base_params(x, w2d, out, F_out, x.shape[1], n_tile, mode)
    p.w_scale = w.scale_t.data_ptr()
    p.fp8 = 2
    return p


def linear_a16(x, w: Fp8Weight, swiglu: bool = False, out=None, n_tile=None, _cfg=None):
    """bf16 x [T, K] times a block-scaled e4m3 weight -> bf16 [T, F] (F = rows, or rows / 2 with the SwiGLU pair epilogue)."""
    if not x.is_cuda:
        wd = w.dequant()
        return ref.swiglu_linear(x, wd) if swiglu else ref.linear(x, wd)
    F._check_act(x)
    T = x.shape[0]
    rows = w.shape[-2]
    Fo = rows // 2 if swiglu else rows
    if out is None:
        out = torch.empty(T, Fo, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    p = _a16_params(x, w, out, Fo, n_tile or _a16_n_tile(T, swiglu), 1 if swiglu else 0)
    p.w_rows_per_group, p.up_row_off = rows, (Fo if swiglu else 0)
    F._gemm_launch(p, "fp8-weight linear", _cfg)
    return out


def grouped_linear_a16(xs, w: Fp8Weight, counts, offsets, swiglu: bool = False, out=None, n_tile=None, rows_hint=None, _cfg=None):
    """Per-expert linear over expert-sorted bf16 rows with block-scaled e4m3 expert weights. w.shape = [E, rows, K]."""
    if not xs.is_cuda:
        return ref.grouped_linear(xs, w.dequant(), counts, offsets, swiglu)
    F._check_act(xs)
    R = xs.shape[0]
    E, rows = w.shape[0], w.shape[1]
    Fo = rows // 2 if swiglu else rows
    if out is None:
        out = torch.empty(R, Fo, dtype=torch.bfloat16, device=xs.device)
    if R == 0:
        return out
    if n_tile is None:
        avg = (rows_hint if rows_hint is not None else R) / E
        n_tile = _a16_n_tile(int(math.ceil(avg * 1.5)), swiglu)
    p = _a16_params(xs, w, out, Fo, n_tile, 1 if swiglu else 0)
    p.G, p.w_rows_per_group, p.up_row_off = E, rows, (Fo if swiglu else 0)
    p.group_off, p.group_cnt = offsets.data_ptr(), counts.data_ptr()
    F._gemm_launch(p, "fp8-weight grouped_linear", _cfg)
    return out


def linear_publish_a16(x, w: Fp8Weight, out_local, peer_flag, epoch, done_counter, ldo, grouped=None, n_tile=None, rows_hint=None):
    """Row-parallel projection with e4m3 weights and bf16 activations whose partial result is published to the
    tensor-parallel peers (the contract of ops.linear_push)."""
    F._check_act(x)
    R = x.shape[0]
    if grouped is None:
        rows = w.shape[-2]
        p = _a16_params(x, w, out_local, rows, n_tile or _a16_n_tile(R, False), 2)
        p.w_rows_per_group = rows
    else:
        counts, offsets = grouped
        E, rows = w.shape[0], w.shape[1]
        if n_tile is None:
            avg = (rows_hint if rows_hint is not None else R) / E
            n_tile = _a16_n_tile(int(math.ceil(avg * 1.5)), False)
        p = _a16_params(x, w, out_local, rows, n_tile, 2)
        p.G, p.w_rows_per_group = E, rows
        p.group_off, p.group_cnt = offsets.data_ptr(), counts.data_ptr()
    p.ldo = ldo
    p.n_peers = len(peer_flag)
    for i, pf in enumerate(peer_flag):
        p.peer_flag[i] = pf
    p.epoch = epoch.data_ptr()
    p.done_counter = done_counter.data_ptr()
    F._gemm_launch(p, "fp8-weight linear_publish")
