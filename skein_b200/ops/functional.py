"""Operator interface of the runtime.

Every operator has two implementations with identical semantics:

* CUDA tensors -> the hand-written sm_100a kernels in csrc/kernels (via skein_b200.ops._lib). There
  is no PyTorch fallback on this path: a missing or failing kernel raises.
* CPU tensors  -> the fp32 PyTorch reference in skein_b200.ops.reference (tests, planner-side
  tooling, parity oracle).

Conventions: activations are row-major [tokens, features] bf16; weights are [out_features,
in_features] bf16 (the HuggingFace layout), experts stacked on a leading dim.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from . import _lib, reference as ref, tuning

_WORKSPACES: dict = {}


class Workspace:
    """Per-device scratch shared by kernels that run one after another on a stream.

    Holds the stream-K partial-tile buffer and arrival counters of the GEMM, the split-KV buffers
    of decode attention, and the status word that kernels write an error code into when a
    bounded wait runs out or a debug bounds check trips (followed by a running total of the time the
    reduce kernels spent waiting for tensor-parallel peers).
    """

    GEMM_WS_BYTES = 148 * 2 * 128 * 256 * 4 + (1 << 20)

    def __init__(self, device):
        self.device = torch.device(device)
        L = _lib.lib()
        self.sm_count = L.skein_sm_count()
        self.gemm_ws = torch.empty(max(self.GEMM_WS_BYTES, self.sm_count * 2 * 128 * 256 * 4), dtype=torch.uint8,
                                   device=device)
        self.gemm_counters = torch.zeros(max(self.sm_count, 256), dtype=torch.int32, device=device)
        # [error code, detail, nanoseconds spent waiting for peers (64-bit total in words 2..3)]
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.router_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.route_barrier = torch.zeros(2, dtype=torch.int32, device=device)
        # Split-KV scratch of decode attention, sized ONCE for the worst case and never reallocated: captured CUDA
        # graphs keep its address, so growing it on demand would leave earlier graphs writing into freed memory.
        # Splits are only used while (sequences x kv heads x splits) <= SM count (pick_splits) with at most
        # MAX_GROUP query heads per kv head, which bounds B * Hq * splits; the counters are one per (sequence, kv head).
        self.attn_rows_cap = self.sm_count * self.MAX_GROUP
        self.attn_ws = torch.empty(int(L.skein_attn_decode_workspace_floats(self.attn_rows_cap, 1, 1)),
                                   dtype=torch.float32, device=device)
        self.attn_counters = torch.zeros(max(self.sm_count, 256), dtype=torch.int32, device=device)
        self.peer_state = []     # (epochs, done) tensors of live communicators, re-armed after a device error

    MAX_GROUP = 16   # query heads per kv head that the tensor-core decode attention accepts

    def attn_scratch(self, B, Hq, Hkv, splits):
        """The fixed split-KV scratch, or None when this launch would not fit it (the caller then runs unsplit)."""
        if B * Hq * splits > self.attn_rows_cap or B * Hkv > self.attn_counters.numel():
            return None
        return self.attn_ws, self.attn_counters

    def check_status(self):
        """Host read of the status word (synchronises). Raises on a recorded device-side error."""
        code, detail = self.status[:2].tolist()
        if code != 0:
            self.reset_after_error()
            names = {1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free stage",
                     3: "timeout waiting for an accumulator", 4: "timeout waiting for a drained accumulator",
                     5: "timeout waiting for a peer flag", 6: "timeout waiting for the other pieces of a split tile",
                     7: "index out of range", 8: "timeout at a grid-wide arrival counter"}
            raise RuntimeError(f"device status {code} ({names.get(code, 'unknown')}), detail {detail}")


    def reset_after_error(self):
        """A kernel that gave up leaves its arrival counters dirty: the split-K arrive/depart words of the GEMM, the
        grid barrier of the fused router, the last-arriver counters of split-KV attention and the "all CTAs done"
        counters of the publish epilogues. Clear them all together with the status word."""
        self.status[:2].zero_()
        self.route_barrier.zero_()
        self.gemm_counters.zero_()
        self.attn_counters.zero_()
        self.router_counter.zero_()
        for _, done in self.peer_state:
            done.zero_()


def workspace(device=None) -> Workspace:
    device = torch.device(device if device is not None else torch.cuda.current_device())
    if device.type != "cuda":
        raise ValueError("workspaces exist for CUDA devices only")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = _WORKSPACES.get(device)
    if ws is None:
        ws = _WORKSPACES[device] = Workspace(device)
    return ws


def _round_up(x, m):
    return (x + m - 1) // m * m


def pick_n_tile(rows_hint: int, dual: bool) -> int:
    cap = 128 if dual else 256
    return max(16, min(cap, _round_up(max(rows_hint, 1), 16)))


def _gemm_launch(p: "_lib.GemmParams", what: str, cfg: dict | None = None):
    """Launch with (in this order) an explicit configuration, the measured one from the kernel-configuration cache
    (tuning.py), or the heuristics below."""
    ws = workspace()
    p.workspace = ws.gemm_ws.data_ptr()
    p.counters = ws.gemm_counters.data_ptr()
    p.status = ws.status.data_ptr()
    p.line_cut_only = 1 if os.environ.get("SKEIN_GEMM_ALIGNED", "1") == "0" else 0
    if cfg is None:
        cache = tuning.active()
        if cache is not None:
            cfg = cache.get("gemm", tuning.gemm_shape_key(p.mode, p.G, p.F, p.K, p.x_rows))
    if cfg is not None:
        p.n_tile, p.grid, p.line_cut_only = int(cfg["n_tile"]), int(cfg["grid"]), int(cfg["line_cut_only"])
    elif p.grid == 0 and os.environ.get("SKEIN_GEMM_AUTOGRID", "1") == "1":
        # With between one and two tiles per SM there are two ways to deal the work. Whole tiles per CTA: no tile is
        # split, so there is no partial store / reduce, but the CTAs with two tiles set the time and the rest idle.
        # Equal K shares on every SM: balanced, at the price of the fix-up (~6 us measured, about 16 K-blocks of
        # streaming). Whole tiles win while the K-blocks they waste per CTA stay under that price: Mixtral's expert
        # down projection at 8 ranks (28 K-blocks per tile) 26.3 vs 29.7 us; the same projection on one GPU
        # (224 K-blocks per tile) 157.4 vs 143.6 us, so that one takes the equal shares.
        # (With fewer tiles than SMs the kernel itself cuts each tile into aligned pieces.)
        # The estimate assumes one token tile per group (decode); a wrong guess only changes the split.
        rows = p.t_static if not p.group_cnt else p.n_tile
        units = p.G * ((p.F + 127) // 128) * max(1, (rows + p.n_tile - 1) // p.n_tile)
        p.grid = tuning.heuristic_grid(units, p.K // (128 if p.fp8 else 64), ws.sm_count, dual=(p.mode == 1))
    _lib.check(_lib.lib().skein_gemm_ws(C.byref(p), _lib.stream_ptr()), what)
    _lib.count_launch()


def _base_params(x, w2d, out, F, K, n_tile, mode) -> "_lib.GemmParams":
    p = _lib.GemmParams()
    p.W = w2d.data_ptr()
    p.X = x.data_ptr()
    p.out = out.data_ptr() if out is not None else None
    p.G, p.F, p.K = 1, F, K
    p.w_rows_per_group = w2d.shape[0]
    p.up_row_off = 0
    p.x_rows = x.shape[0]
    p.t_static = x.shape[0]
    p.n_tile = n_tile
    p.ldo = out.stride(0) if out is not None else 0
    p.mode = mode
    return p


class PackedWeight:
    """A weight matrix re-laid for streaming: [groups, rows/128, K/64, 128, 64] bf16, so that each
    128 x 64 tile the GEMM loads is one contiguous 16 KB block and a CTA's K loop walks consecutive
    memory. `shape` keeps the logical [groups?, rows, K]."""

    def __init__(self, data: torch.Tensor, shape):
        self.data, self.shape = data, tuple(shape)
        self.device, self.dtype = data.device, data.dtype

    @property
    def is_cuda(self):
        return self.data.is_cuda

    def data_ptr(self):
        return self.data.data_ptr()

    def copy_(self, src):
        """In-place update from a plain [groups?, rows, K] tensor or another PackedWeight (hot swap keeps the storage
        that captured CUDA graphs point at)."""
        self.data.copy_(src.data if isinstance(src, PackedWeight) else pack_weight(src).data)
        return self

    def cpu(self) -> torch.Tensor:
        """The logical (row-major) tensor on the host."""
        return self.unpack().cpu()

    def unpack(self) -> torch.Tensor:
        *g, R, K = self.shape
        G = g[0] if g else 1
        t = self.data.view(G, R // 128, K // 64, 128, 64).permute(0, 1, 3, 2, 4).reshape(G, R, K)
        return t if g else t[0]


def pack_weight(w: torch.Tensor) -> PackedWeight:
    """[rows, K] or [G, rows, K] (rows % 128 == 0, K % 64 == 0) -> PackedWeight."""
    shape = tuple(w.shape)
    R, K = shape[-2], shape[-1]
    if R % 128 or K % 64:
        raise ValueError("pack_weight needs rows % 128 == 0 and K % 64 == 0")
    G = shape[0] if w.dim() == 3 else 1
    t = w.reshape(G, R // 128, 128, K // 64, 64).permute(0, 1, 3, 2, 4).contiguous()
    return PackedWeight(t, shape)


def _wview(w):
    """(2-D view or packed data, rows per group, packed flag)."""
    if isinstance(w, PackedWeight):
        return w.data, w.shape[-2], 1
    return (w.view(-1, w.shape[-1]) if w.dim() == 3 else w), w.shape[-2], 0


def _check_act(x):
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("activations must be contiguous bf16")


def linear(x, w, out=None, residual=None, n_tile=None, _cfg=None):
    """y[t, f] = sum_k x[t, k] w[f, k] (+ residual[t, f])."""
    if not x.is_cuda:
        y = ref.linear(x, w.unpack() if isinstance(w, PackedWeight) else w, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_act(x)
    T, K = x.shape
    F = w.shape[0]
    if out is None:
        out = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    wv, _, packed = _wview(w)
    p = _base_params(x, wv, out, F, K, n_tile or pick_n_tile(T, False), 0)
    p.w_rows_per_group, p.w_packed = F, packed
    if residual is not None:
        p.residual = residual.data_ptr()
    _gemm_launch(p, "linear", _cfg)
    return out


def swiglu_linear(x, w13, out=None, n_tile=None, _cfg=None):
    """silu(x @ w13[:I].T) * (x @ w13[I:].T) with both products from one pass over x."""
    if not x.is_cuda:
        return ref.swiglu_linear(x, w13.unpack() if isinstance(w13, PackedWeight) else w13)
    _check_act(x)
    T, K = x.shape
    inter = w13.shape[0] // 2
    if out is None:
        out = torch.empty(T, inter, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    wv, rows_pg, packed = _wview(w13)
    p = _base_params(x, wv, out, inter, K, n_tile or pick_n_tile(T, True), 1)
    p.w_rows_per_group, p.w_packed = rows_pg, packed
    p.up_row_off = inter
    _gemm_launch(p, "swiglu_linear", _cfg)
    return out


def grouped_linear(xs, w, counts, offsets, swiglu=False, out=None, n_tile=None, rows_hint=None, grid=0, _cfg=None):
    """Per-expert linear over an expert-sorted activation matrix.

    xs [rows, K]; w [E, F, K] (or [E, 2I, K] with gate rows first when swiglu); counts / offsets are
    int32 device tensors of E (offsets may have E+1) entries: rows of expert e are
    offsets[e] : offsets[e] + counts[e]. Rows not covered by any expert are left untouched.
    """
    if not xs.is_cuda:
        return ref.grouped_linear(xs, w.unpack() if isinstance(w, PackedWeight) else w, counts, offsets, swiglu)
    _check_act(xs)
    rows, K = xs.shape
    E = w.shape[0]
    F = w.shape[1] // 2 if swiglu else w.shape[1]
    if out is None:
        out = torch.empty(rows, F, dtype=torch.bfloat16, device=xs.device)
    if rows == 0:
        return out
    if n_tile is None:
        avg = (rows_hint if rows_hint is not None else rows) / E
        n_tile = pick_n_tile(int(math.ceil(avg * 1.5)), swiglu)
    wv, rows_pg, packed = _wview(w)
    p = _base_params(xs, wv, out, F, K, n_tile, 1 if swiglu else 0)
    p.G = E
    p.w_rows_per_group, p.w_packed = rows_pg, packed
    p.up_row_off = F if swiglu else 0
    p.group_off = offsets.data_ptr()
    p.group_cnt = counts.data_ptr()
    p.grid = grid
    _gemm_launch(p, "grouped_linear", _cfg)
    return out


def _partial_args(partial, flags, epoch):
    """(data pointer, source stride, n_src, per-source pointer array or None, multicast address or None, flags, epoch)
    of a partial-sum operand: a [n_src, rows, H] tensor, or peer partials (parallel/tp.py: one peer-mapped [rows, H]
    buffer per rank, pulled over NVLink by the kernel, through the multicast mapping when there is one)."""
    if partial is None:
        return None, 0, 0, None, None, flags, epoch
    if hasattr(partial, "ptrs"):
        return (partial.local.data_ptr(), 0, partial.n_src, partial.ptrs, getattr(partial, "mc", 0) or None, partial.flags,
                partial.epoch)
    return partial.data_ptr(), partial.stride(0), partial.shape[0], None, None, flags, epoch


def reduce_residual_rmsnorm(residual, partial, gamma, eps, row_idx=None, row_w=None, residual_out=None,
                            normed_out=None, flags=None, epoch=None, wait_budget_ms=0, owner_ids=None, experts_per_owner=1,
                            owner_span=1):
    """See csrc/kernels/norm.cu. partial: [n_src, rows, H], peer partials, or None. Returns (residual_out, normed_out)."""
    peer = hasattr(partial, "ptrs")
    src = residual if residual is not None else (partial.local if peer else partial)
    if not src.is_cuda:
        return ref.reduce_residual_rmsnorm(residual, partial, gamma, eps, row_idx, row_w, owner_ids, experts_per_owner, owner_span)
    H = src.shape[-1]
    B = residual.shape[0] if residual is not None else (row_idx.shape[0] if row_idx is not None else
                                                        (partial.rows if peer else partial.shape[1]))
    if residual_out is None:
        residual_out = torch.empty(B, H, dtype=torch.bfloat16, device=src.device)
    if normed_out is None and gamma is not None:
        normed_out = torch.empty(B, H, dtype=torch.bfloat16, device=src.device)
    pptr, src_stride, n_src, ptrs, mc, flags, epoch = _partial_args(partial, flags, epoch)
    if peer and wait_budget_ms == 0:
        wait_budget_ms = partial.wait_budget_ms
    topk = row_idx.shape[1] if row_idx is not None else 0
    ws = workspace()
    rc = _lib.lib().skein_reduce_residual_rmsnorm(
        _lib.ptr(residual), pptr, _lib.ptr(row_idx), _lib.ptr(row_w), _lib.ptr(gamma),
        _lib.ptr(residual_out), _lib.ptr(normed_out), _lib.ptr(flags), _lib.ptr(epoch), ws.status.data_ptr(),
        src_stride, B, H, n_src, topk, float(eps), wait_budget_ms, _lib.ptr(owner_ids), experts_per_owner, owner_span,
        ptrs, mc, _lib.stream_ptr())
    _lib.check(rc, "reduce_residual_rmsnorm")
    _lib.count_launch()
    return residual_out, normed_out


def can_fuse_route(T, topk, device=None) -> bool:
    """True when reduce_norm_route may be used: every token's CTA must be resident at once."""
    return 0 < T <= workspace(device).sm_count and T * topk <= 2048 and os.environ.get("SKEIN_FUSE_ROUTE", "1") != "0"


def reduce_norm_route(residual, partial, gamma, eps, wg, topk, e_first=0, e_count=None, flags=None, epoch=None,
                      wait_budget_ms=0, normed_out=None, ids_out=None, scatter=True):
    """Residual add + (all-reduce consumer) + RMSNorm + MoE router + scatter into expert-sorted order, one launch.

    Equals reduce_residual_rmsnorm followed by route and gather_rows (csrc/kernels/norm.cu). Returns
    (residual_out, normed_out, expert_ids [T,k], weights [T,k], counts [E], offsets [E+1], row_of [T*k],
    src_token [T*k], xs [T*k, H]). `normed_out` / `ids_out` let the caller have the normalised rows and the expert
    choices written somewhere else (a published buffer: expert-parallel dispatch); scatter=False skips the
    expert-sorted copy (xs is then None).
    """
    peer = hasattr(partial, "ptrs")
    src = residual if residual is not None else (partial.local if peer else partial)
    E = wg.shape[0]
    e_count = E if e_count is None else e_count
    if not src.is_cuda:
        res, normed = ref.reduce_residual_rmsnorm(residual, partial, gamma, eps, None, None, None, 1, 1)
        ids, w, _ = ref.router_topk(normed, wg, topk)
        counts, offsets, row_of, src_token = ref.router_plan(ids, E, e_first, e_count)
        return res, normed, ids, w, counts, offsets, row_of, src_token, normed[src_token.long()]
    H = src.shape[-1]
    T = residual.shape[0] if residual is not None else (partial.rows if peer else partial.shape[1])
    dev = src.device
    residual_out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    if normed_out is None:
        normed_out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    ids = ids_out if ids_out is not None else torch.empty(T, topk, dtype=torch.int32, device=dev)
    w = torch.empty(T, topk, dtype=torch.float32, device=dev)
    meta = torch.empty(2 * E + 1 + 2 * T * topk, dtype=torch.int32, device=dev)
    counts, offsets = meta[:E], meta[E:2 * E + 1]
    row_of, src_token = meta[2 * E + 1:2 * E + 1 + T * topk], meta[2 * E + 1 + T * topk:]
    xs = torch.empty(T * topk, H, dtype=torch.bfloat16, device=dev) if scatter else None
    pptr, src_stride, n_src, ptrs, mc, flags, epoch = _partial_args(partial, flags, epoch)
    if peer and wait_budget_ms == 0:
        wait_budget_ms = partial.wait_budget_ms
    ws = workspace()
    rc = _lib.lib().skein_reduce_norm_route(
        _lib.ptr(residual), pptr, gamma.data_ptr(), residual_out.data_ptr(), normed_out.data_ptr(),
        _lib.ptr(flags), _lib.ptr(epoch), ws.status.data_ptr(), src_stride, T, H, n_src, float(eps), wait_budget_ms,
        wg.data_ptr(), E, topk, e_first, e_count, ids.data_ptr(), w.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
        row_of.data_ptr(), src_token.data_ptr(), _lib.ptr(xs), ws.route_barrier.data_ptr(), ws.sm_count,
        ptrs, mc, _lib.stream_ptr())
    _lib.check(rc, "reduce_norm_route")
    _lib.count_launch()
    return residual_out, normed_out, ids, w, counts, offsets, row_of, src_token, xs


def rmsnorm(x, gamma, eps):
    return reduce_residual_rmsnorm(x, None, gamma, eps)[1]


def rope_kv_append(qkv, positions, seq_of_token, block_table, cos_sin, kv_cache, Hq, Hkv, D):
    """Rotate q (in place) and k, append k/v of every token into the paged cache."""
    if not qkv.is_cuda:
        return ref.rope_kv_append(qkv, positions, seq_of_token, block_table, cos_sin, kv_cache, Hq, Hkv, D)
    T = qkv.shape[0]
    ws = workspace()
    rc = _lib.lib().skein_rope_kv_append(
        qkv.data_ptr(), positions.data_ptr(), _lib.ptr(seq_of_token), block_table.data_ptr(), block_table.stride(0),
        cos_sin.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[3], T, Hq, Hkv, D, cos_sin.shape[0],
        kv_cache.shape[0], ws.status.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "rope_kv_append")
    _lib.count_launch()


def pick_splits(B, Hkv, ctx_hint, sm_count=148):
    """Split-KV factor of decode attention: only while there are fewer (sequence, kv head) pairs than SMs, never
    below 512 tokens per split, never more CTAs than SMs. Each split adds a workspace round trip and a last-arriver
    merge, which at 64 sequences costs more than the extra parallelism brings."""
    if os.environ.get("SKEIN_ATTN_SPLITS"):
        return int(os.environ["SKEIN_ATTN_SPLITS"])
    ctas = max(B * Hkv, 1)
    return max(1, min(sm_count // ctas, ctx_hint // 512, 16))


def _decode_tc_ok(kv_cache, B, Hq, Hkv, D, splits, impl) -> bool:
    """Whether the tcgen05 decode kernel (csrc/kernels/attn_decode_tc.cu) takes this launch: one split, head size 128,
    16-token pages, at most 8 query heads per kv head. "auto" (the default) picks it when the launch has at least 1.5
    (sequence, kv head) pairs per SM: there the kernel is bandwidth-bound and the tensor-memory form is the faster one
    (35.6 against 37.0 us at 512 pairs, 18.5 against 19.5 at 256); with fewer pairs a CTA's chain of per-tile latencies
    decides and the mma.sync kernel, whose four warps run independent pipelines, wins (13.2 against 15.9 us at 64 pairs).
    SKEIN_ATTN_DECODE=tc|mma|scalar (or impl) forces a kernel."""
    choice = impl or os.environ.get("SKEIN_ATTN_DECODE", _DECODE_DEFAULT)
    if choice == "auto":
        choice = "tc" if 2 * B * Hkv >= 3 * workspace().sm_count else "mma"
    return (choice == "tc" and splits == 1 and D == 128 and kv_cache.shape[3] == 16 and kv_cache.shape[4] == 128
            and Hq % Hkv == 0 and Hq // Hkv <= 8)


_DECODE_DEFAULT = "auto"


def attn_decode(q, kv_cache, block_table, seq_lens, Hq, Hkv, D, scale=None, out=None, splits=None, ctx_hint=1024,
                impl=None):
    """q: [B, row_stride] whose first Hq*D columns are the (rotated) query heads -> [B, Hq*D].

    impl "mma" (default where it applies: page size a multiple of 16, at most 16 query heads per kv head) is the
    tensor-core kernel with the asynchronous copy pipeline, "scalar" the FMA kernel; SKEIN_ATTN_DECODE overrides."""
    if not q.is_cuda:
        return ref.attn_decode(q, kv_cache, block_table, seq_lens, Hq, Hkv, D, scale)
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, Hq * D, dtype=torch.bfloat16, device=q.device)
    ws = workspace()
    if splits is None:
        splits = pick_splits(B, Hkv, ctx_hint, ws.sm_count)
    wsf, ctr = (None, None)
    if splits > 1:
        scratch = ws.attn_scratch(B, Hq, Hkv, splits)
        if scratch is None:
            splits = 1
        else:
            wsf, ctr = scratch
    if _decode_tc_ok(kv_cache, B, Hq, Hkv, D, splits, impl):
        rc = _lib.lib().skein_attn_decode_tc(
            q.data_ptr(), q.stride(0), kv_cache.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(), None, None, 0,
            out.data_ptr(), ws.status.data_ptr(), B, Hq, Hkv, D, kv_cache.shape[3], block_table.stride(0), kv_cache.shape[0],
            float(scale), _lib.stream_ptr())
        if rc != -1:
            _lib.check(rc, "attn_decode_tc")
            _lib.count_launch()
            return out
    impl = impl or os.environ.get("SKEIN_ATTN_DECODE", _DECODE_DEFAULT)
    if impl in ("tc", "auto"):
        impl = "mma"
    if kv_cache.shape[3] % 16 != 0 or Hq // Hkv > 16:
        impl = "scalar"
    fn = _lib.lib().skein_attn_decode_mma if impl == "mma" else _lib.lib().skein_attn_decode
    rc = fn(
        q.data_ptr(), q.stride(0), kv_cache.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
        _lib.ptr(wsf), _lib.ptr(ctr), ws.status.data_ptr(), B, Hq, Hkv, D, kv_cache.shape[3], block_table.stride(0),
        kv_cache.shape[0], splits, float(scale), _lib.stream_ptr())
    _lib.check(rc, "attn_decode")
    _lib.count_launch()
    return out


def can_fuse_rope(kv_cache, Hq, Hkv) -> bool:
    """True when attn_decode_rope runs as one kernel (else it falls back to rope_kv_append + attn_decode)."""
    return (kv_cache.is_cuda and kv_cache.shape[3] % 16 == 0 and Hq // Hkv <= 16 and kv_cache.shape[4] == 128
            and os.environ.get("SKEIN_ATTN_DECODE", _DECODE_DEFAULT) in ("auto", "mma", "tc") and os.environ.get("SKEIN_FUSE_ROPE", "1") != "0")


def attn_decode_rope(qkv, positions, block_table, cos_sin, kv_cache, seq_lens, Hq, Hkv, D, scale=None, out=None,
                     splits=None, ctx_hint=1024, impl=None):
    """Decode attention straight from the fused q/k/v projection: RoPE of q and k, append of the new token's k/v
    to the paged cache, attention; one launch (csrc/kernels/attn_decode_mma.cu). qkv: [B, (Hq + 2 Hkv) * D]."""
    if not can_fuse_rope(kv_cache, Hq, Hkv):
        rope_kv_append(qkv, positions, None, block_table, cos_sin, kv_cache, Hq, Hkv, D)
        return attn_decode(qkv, kv_cache, block_table, seq_lens, Hq, Hkv, D, scale, out, splits, ctx_hint)
    B = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, Hq * D, dtype=torch.bfloat16, device=qkv.device)
    ws = workspace()
    if splits is None:
        splits = pick_splits(B, Hkv, ctx_hint, ws.sm_count)
    wsf, ctr = (None, None)
    if splits > 1:
        scratch = ws.attn_scratch(B, Hq, Hkv, splits)
        if scratch is None:
            splits = 1
        else:
            wsf, ctr = scratch
    if _decode_tc_ok(kv_cache, B, Hq, Hkv, D, splits, impl):
        rc = _lib.lib().skein_attn_decode_tc(
            qkv.data_ptr(), qkv.stride(0), kv_cache.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(),
            positions.data_ptr(), cos_sin.data_ptr(), cos_sin.shape[0], out.data_ptr(), ws.status.data_ptr(), B, Hq, Hkv, D,
            kv_cache.shape[3], block_table.stride(0), kv_cache.shape[0], float(scale), _lib.stream_ptr())
        if rc != -1:
            _lib.check(rc, "attn_decode_tc")
            _lib.count_launch()
            return out
    rc = _lib.lib().skein_attn_decode_rope_mma(
        qkv.data_ptr(), qkv.stride(0), kv_cache.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(),
        positions.data_ptr(), cos_sin.data_ptr(), cos_sin.shape[0], out.data_ptr(), _lib.ptr(wsf), _lib.ptr(ctr),
        ws.status.data_ptr(), B, Hq, Hkv, D, kv_cache.shape[3], block_table.stride(0), kv_cache.shape[0], splits,
        float(scale), _lib.stream_ptr())
    _lib.check(rc, "attn_decode_rope")
    _lib.count_launch()
    return out


def attn_prefill(q, kv_cache, block_table, q_start, q_len, kv_len, max_q_len, Hq, Hkv, D, scale=None, out=None):
    if not q.is_cuda:
        return ref.attn_prefill(q, kv_cache, block_table, q_start, q_len, kv_len, Hq, Hkv, D, scale)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(q.shape[0], Hq * D, dtype=torch.bfloat16, device=q.device)
    ws = workspace()
    if D == 128 and kv_cache.shape[3] == 16 and os.environ.get("SKEIN_ATTN_PREFILL", "tc") != "mma":
        # tcgen05 kernel (csrc/kernels/attn_prefill_tc.cu): Q / K / V tiles by TMA, S, P and O in tensor memory
        rc = _lib.lib().skein_attn_prefill_tc(
            q.data_ptr(), q.stride(0), q.shape[0], kv_cache.data_ptr(), block_table.data_ptr(), q_start.data_ptr(),
            q_len.data_ptr(), kv_len.data_ptr(), out.data_ptr(), ws.status.data_ptr(), q_len.shape[0], int(max_q_len), Hq, Hkv, D,
            kv_cache.shape[3], block_table.stride(0), kv_cache.shape[0], float(scale), _lib.stream_ptr())
        if rc != -1:
            _lib.check(rc, "attn_prefill_tc")
            _lib.count_launch()
            return out
    rc = _lib.lib().skein_attn_prefill(
        q.data_ptr(), q.stride(0), kv_cache.data_ptr(), block_table.data_ptr(), q_start.data_ptr(), q_len.data_ptr(),
        kv_len.data_ptr(), out.data_ptr(), ws.status.data_ptr(), q_len.shape[0], int(max_q_len), Hq, Hkv, D,
        kv_cache.shape[3], block_table.stride(0), kv_cache.shape[0], float(scale), _lib.stream_ptr())
    _lib.check(rc, "attn_prefill")
    _lib.count_launch()
    return out


def router_topk(x, wg, topk, want_logits=False):
    """Returns (expert_ids int32 [T, k], weights fp32 [T, k], logits fp32 [T, E] or None)."""
    if not x.is_cuda:
        ids, w, lg = ref.router_topk(x, wg, topk)
        return ids, w, (lg if want_logits else None)
    T, H = x.shape
    E = wg.shape[0]
    ids = torch.empty(T, topk, dtype=torch.int32, device=x.device)
    w = torch.empty(T, topk, dtype=torch.float32, device=x.device)
    lg = torch.empty(T, E, dtype=torch.float32, device=x.device) if want_logits else None
    rc = _lib.lib().skein_router_topk(x.data_ptr(), wg.data_ptr(), T, H, E, topk, ids.data_ptr(), w.data_ptr(),
                                      _lib.ptr(lg), None, None, None, None, 0, E, None, _lib.stream_ptr())
    _lib.check(rc, "router_topk")
    _lib.count_launch()
    return ids, w, lg


def route(x, wg, topk, e_first=0, e_count=None):
    """Router and expert-sorted layout in one launch.

    Returns (expert_ids [T, k], weights [T, k], counts [E], offsets [E+1], row_of [T*k], src_token [T*k]);
    offsets[E] is the number of rows routed to this rank's experts, rows of src_token beyond it are unset.
    """
    E = wg.shape[0]
    if not x.is_cuda:
        ids, w, _ = ref.router_topk(x, wg, topk)
        return (ids, w) + tuple(ref.router_plan(ids, E, e_first, e_count))
    T, H = x.shape
    dev = x.device
    ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    w = torch.empty(T, topk, dtype=torch.float32, device=dev)
    meta = torch.empty(2 * E + 1 + 2 * T * topk, dtype=torch.int32, device=dev)
    counts, offsets = meta[:E], meta[E:2 * E + 1]
    row_of, src_token = meta[2 * E + 1:2 * E + 1 + T * topk], meta[2 * E + 1 + T * topk:]
    ws = workspace()
    rc = _lib.lib().skein_router_topk(x.data_ptr(), wg.data_ptr(), T, H, E, topk, ids.data_ptr(), w.data_ptr(), None,
                                      counts.data_ptr(), offsets.data_ptr(), row_of.data_ptr(), src_token.data_ptr(),
                                      e_first, E if e_count is None else e_count, ws.router_counter.data_ptr(),
                                      _lib.stream_ptr())
    _lib.check(rc, "route")
    _lib.count_launch()
    return ids, w, counts, offsets, row_of, src_token


def router_plan(expert_ids, E, e_first=0, e_count=None, bufs=None):
    """Expert-sorted layout of the (token, slot) pairs. Returns (counts[E], offsets[E+1], row_of[T*k], src_token[T*k])."""
    if not expert_ids.is_cuda:
        return ref.router_plan(expert_ids, E, e_first, e_count)
    T, topk = expert_ids.shape
    n = T * topk
    dev = expert_ids.device
    if bufs is None:
        counts = torch.empty(E, dtype=torch.int32, device=dev)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        row_of = torch.empty(n, dtype=torch.int32, device=dev)
        src_token = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    else:
        counts, offsets, row_of, src_token = bufs
    rc = _lib.lib().skein_router_plan(expert_ids.data_ptr(), n, E, topk, counts.data_ptr(), offsets.data_ptr(),
                                      row_of.data_ptr(), src_token.data_ptr(), e_first,
                                      E if e_count is None else e_count, _lib.stream_ptr())
    _lib.check(rc, "router_plan")
    _lib.count_launch()
    return counts, offsets, row_of, src_token


def gather_rows(x, src_row, n_rows_dev=None, out=None):
    """out[r] = x[src_row[r]] for r < n_rows (a device int, or all rows of src_row)."""
    if not x.is_cuda:
        return x[src_row.long()]
    n = src_row.shape[0]
    H = x.shape[1]
    if out is None:
        out = torch.empty(n, H, dtype=x.dtype, device=x.device)
    rc = _lib.lib().skein_gather_rows(x.data_ptr(), src_row.data_ptr(), out.data_ptr(), n, H, _lib.ptr(n_rows_dev),
                                      _lib.stream_ptr())
    _lib.check(rc, "gather_rows")
    _lib.count_launch()
    return out


def embed(ids, table, vocab_start=0, out=None):
    if not table.is_cuda:
        return ref.embed(ids, table, vocab_start)
    T = ids.shape[0]
    H = table.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = _lib.lib().skein_embed_gather(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, vocab_start,
                                       table.shape[0], _lib.stream_ptr())
    _lib.check(rc, "embed")
    _lib.count_launch()
    return out


def sample_argmax(logits, idx_offset=0, out=None, out_val=None):
    """Greedy token per row (ties -> lowest index). logits [B, V] bf16, row stride arbitrary."""
    if not logits.is_cuda:
        r = ref.sample_argmax(logits) + idx_offset
        return r
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    rc = _lib.lib().skein_sample_argmax(logits.data_ptr(), logits.stride(0), B, V, idx_offset, out.data_ptr(),
                                        _lib.ptr(out_val), _lib.stream_ptr())
    _lib.check(rc, "sample_argmax")
    _lib.count_launch()
    return out


def sample(logits, temperature, top_k, top_p, seeds, step, out=None):
    """Temperature / top-k / top-p sampling; per-row parameters are device tensors. `step` is the counter of the
    random stream: one int32 for the whole batch, or one per row (the token's position)."""
    if not logits.is_cuda:
        return ref.sample(logits, temperature, top_k, top_p, seeds, step)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    rc = _lib.lib().skein_sample_topk_topp(logits.data_ptr(), logits.stride(0), B, V, _lib.ptr(temperature),
                                           _lib.ptr(top_k), _lib.ptr(top_p), _lib.ptr(seeds), _lib.ptr(step),
                                           0 if (step is None or step.numel() == 1) else 1, out.data_ptr(),
                                           _lib.stream_ptr())
    _lib.check(rc, "sample")
    _lib.count_launch()
    return out


def quant_fp8_block128(x):
    """bf16 [rows, K] -> (e4m3 [rows, K], fp32 scales [rows, K/128])."""
    if not x.is_cuda:
        return ref.quant_fp8_block128(x)
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(rows, K // 128, dtype=torch.float32, device=x.device)
    rc = _lib.lib().skein_quant_fp8_block128(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, K, _lib.stream_ptr())
    _lib.check(rc, "quant_fp8_block128")
    _lib.count_launch()
    return q, s


def advance_decode_state(sampled, tokens, positions, seq_lens, step_counter=None):
    """tokens <- sampled, positions += 1, seq_lens += 1 for live rows (device-side token feedback)."""
    if not sampled.is_cuda:
        live = seq_lens > 0
        tokens[live] = sampled[live]
        positions[live] += 1
        seq_lens[live] += 1
        if step_counter is not None:
            step_counter += 1
        return
    rc = _lib.lib().skein_advance_decode_state(sampled.data_ptr(), tokens.data_ptr(), positions.data_ptr(),
                                               seq_lens.data_ptr(), sampled.shape[0], _lib.ptr(step_counter),
                                               _lib.stream_ptr())
    _lib.check(rc, "advance_decode_state")
    _lib.count_launch()


def linear_push(x, w, out_local, peer_flag, epoch, done_counter, ldo, grouped=None, n_tile=None, rows_hint=None,
                wait_budget_ms=0):
    """Row-parallel projection that publishes its partial result to the tensor-parallel peers.

    The partial is stored into `out_local` (a [rows, ldo] bf16 buffer of this rank that the peers have mapped) and,
    when the whole launch is done, this rank's flag word on every peer is set: peer_flag[i] are raw addresses valid
    in this process. `epoch` and `done_counter` are local int32 device tensors. grouped = (counts, offsets) selects
    the per-expert form. The consumers pull the buffer over NVLink (reduce_residual_rmsnorm with peer partials).
    """
    _check_act(x)
    rows, K = x.shape
    wv, rows_pg, packed = _wview(w)
    if grouped is None:
        F = w.shape[0]
        p = _base_params(x, wv, out_local, F, K, n_tile or pick_n_tile(rows, False), 2)
        p.w_rows_per_group = F
    else:
        counts, offsets = grouped
        E, F = w.shape[0], w.shape[1]
        if n_tile is None:
            avg = (rows_hint if rows_hint is not None else rows) / E
            n_tile = pick_n_tile(int(math.ceil(avg * 1.5)), False)
        p = _base_params(x, wv, out_local, F, K, n_tile, 2)
        p.G, p.w_rows_per_group = E, rows_pg
        p.group_off, p.group_cnt = offsets.data_ptr(), counts.data_ptr()
    p.w_packed = packed
    p.ldo = ldo
    p.n_peers = len(peer_flag)
    for i, pf in enumerate(peer_flag):
        p.peer_flag[i] = pf
    p.epoch = epoch.data_ptr()
    p.done_counter = done_counter.data_ptr()
    p.wait_budget_ms = wait_budget_ms
    _gemm_launch(p, "linear_push")


def tune_linear(x, w, swiglu=False, cache=None, budget=0):
    """Measure the launch configurations of this dense GEMM shape and record the fastest (tuning.py)."""
    F = w.shape[0] // 2 if swiglu else w.shape[0]
    out = torch.empty(x.shape[0], F, dtype=torch.bfloat16, device=x.device)
    run = (lambda c: swiglu_linear(x, w, out=out, _cfg=c)) if swiglu else (lambda c: linear(x, w, out=out, _cfg=c))
    return tuning.tune_gemm(run, 1 if swiglu else 0, 1, F, x.shape[1], x.shape[0], cache, budget=budget)


def tune_grouped(xs, w, counts, offsets, swiglu=False, cache=None, budget=0):
    """Same for a grouped (per-expert) GEMM with the given routing."""
    F = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.empty(xs.shape[0], F, dtype=torch.bfloat16, device=xs.device)
    run = lambda c: grouped_linear(xs, w, counts, offsets, swiglu=swiglu, out=out, _cfg=c)
    return tuning.tune_gemm(run, 1 if swiglu else 0, w.shape[0], F, xs.shape[1], xs.shape[0], cache, budget=budget)
