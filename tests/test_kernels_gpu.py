"""Numerics of every CUDA kernel against the fp32 PyTorch reference of the same operator.

Mirrors the reference project's CPU-vs-GPU op comparison (crates/skein_compile/tests/
cuda_vs_cpu_ops.rs:96-436: embedding, RMSNorm, matmul, attention, MoE combine at Mixtral widths).
"""
import math

import pytest
import torch

from skein_b200 import ops
from skein_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _check_status():
    torch.cuda.synchronize()
    ops.workspace().check_status()


@pytest.mark.parametrize("T,F,K", [(64, 256, 512), (1, 128, 64), (17, 384, 4096), (64, 6144, 4096),
                                    (200, 1000, 1024), (513, 4096, 512), (1000, 3200, 512)])
def test_linear(T, F, K):
    torch.manual_seed(0)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(F, K, device=DEV) / math.sqrt(K)).bfloat16()
    y = ops.linear(x, w)
    _check_status()
    assert _rel_err(y, ref.linear(x, w)) < 1e-2


def test_linear_residual_and_repeat():
    torch.manual_seed(1)
    x = torch.randn(48, 1024, device=DEV).bfloat16()
    w = (torch.randn(512, 1024, device=DEV) / 32).bfloat16()
    r = torch.randn(48, 512, device=DEV).bfloat16()
    y1 = ops.linear(x, w, residual=r)
    y2 = ops.linear(x, w, residual=r)
    _check_status()
    assert torch.equal(y1, y2), "same inputs must give bit-identical outputs (stream-K order is fixed)"
    assert _rel_err(y1, ref.linear(x, w, r)) < 1e-2


@pytest.mark.parametrize("T,I,K", [(64, 256, 512), (16, 1792, 4096), (130, 512, 1024)])
def test_swiglu_linear(T, I, K):
    torch.manual_seed(2)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w13 = (torch.randn(2 * I, K, device=DEV) / math.sqrt(K)).bfloat16()
    y = ops.swiglu_linear(x, w13)
    _check_status()
    assert _rel_err(y, ref.swiglu_linear(x, w13)) < 2e-2


@pytest.mark.parametrize("E,F,K,counts", [
    (4, 256, 512, [3, 0, 40, 17]),
    (8, 512, 1024, [16, 16, 16, 16, 16, 16, 16, 16]),
    (8, 4096, 1792, [1, 33, 0, 0, 70, 5, 12, 7]),
])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_linear(E, F, K, counts, swiglu):
    torch.manual_seed(3)
    rows = sum(counts)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    off = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    off[1:] = torch.cumsum(cnt, 0)
    xs = torch.randn(rows, K, device=DEV).bfloat16()
    w = (torch.randn(E, 2 * F if swiglu else F, K, device=DEV) / math.sqrt(K)).bfloat16()
    y = ops.grouped_linear(xs, w, cnt, off, swiglu=swiglu)
    _check_status()
    yr = ref.grouped_linear(xs, w, cnt.cpu(), off.cpu(), swiglu)
    assert _rel_err(y, yr) < 2e-2


def test_rmsnorm_and_combine():
    torch.manual_seed(4)
    B, H, topk, rows = 64, 4096, 2, 128
    res = torch.randn(B, H, device=DEV).bfloat16()
    gamma = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    y = ops.rmsnorm(res, gamma, 1e-5)
    assert _rel_err(y, ref.reduce_residual_rmsnorm(res, None, gamma, 1e-5)[1]) < 1e-2
    part = torch.randn(2, rows, H, device=DEV).bfloat16()
    idx = torch.randperm(rows, device=DEV)[: B * topk].view(B, topk).to(torch.int32)
    wts = torch.rand(B, topk, device=DEV)
    r1, n1 = ops.reduce_residual_rmsnorm(res, part, gamma, 1e-5, idx, wts)
    r2, n2 = ref.reduce_residual_rmsnorm(res, part, gamma, 1e-5, idx, wts)
    _check_status()
    assert _rel_err(r1, r2) < 1e-2 and _rel_err(n1, n2) < 1e-2
    r3, n3 = ops.reduce_residual_rmsnorm(res, part[:, :B], gamma, 1e-5)
    r4, n4 = ref.reduce_residual_rmsnorm(res, part[:, :B], gamma, 1e-5)
    assert _rel_err(r3, r4) < 1e-2 and _rel_err(n3, n4) < 1e-2


def _make_cache(B, ctx_lens, Hkv, D, page_size, extra_pages=3):
    max_blocks = max((l + page_size - 1) // page_size for l in ctx_lens) + 1
    num_pages = B * max_blocks + extra_pages
    kv = torch.randn(num_pages, 2, Hkv, page_size, D, device=DEV).bfloat16()
    perm = torch.randperm(num_pages, device=DEV)[: B * max_blocks].view(B, max_blocks).to(torch.int32)
    return kv, perm.contiguous(), max_blocks


@pytest.mark.parametrize("impl", ["mma", "scalar"])
@pytest.mark.parametrize("Hq,Hkv,splits", [(32, 8, 1), (32, 8, 4), (4, 1, 8), (8, 8, 2), (16, 2, 3)])
def test_attn_decode(Hq, Hkv, splits, impl):
    torch.manual_seed(5)
    B, D, ps = 9, 128, 16
    lens = [1, 15, 16, 17, 130, 512, 700, 33, 0]
    kv, bt, _ = _make_cache(B, lens, Hkv, D, ps)
    q = torch.randn(B, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    o = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=splits, impl=impl)
    o2 = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=splits, impl=impl)
    _check_status()
    assert torch.equal(o, o2)
    assert _rel_err(o, ref.attn_decode(q, kv, bt, sl, Hq, Hkv, D)) < 1e-2


@pytest.mark.parametrize("Hq,Hkv,ps,splits", [(16, 1, 16, 2), (8, 2, 32, 1), (8, 2, 32, 3), (4, 1, 64, 5)])
def test_attn_decode_mma_pages_and_unwritten_slots(Hq, Hkv, ps, splits):
    """Larger pages, 16 heads per kv head, many tiles per warp, and cache slots past each context's end holding
    NaN (never-written memory): they must not reach the output."""
    torch.manual_seed(6)
    B, D = 6, 128
    lens = [3, 40, 2500, 1, 1023, 97]
    kv, bt, _ = _make_cache(B, lens, Hkv, D, ps)
    for b, l in enumerate(lens):                       # poison every slot at or past the end of the context
        for blk in range(l // ps, bt.shape[1]):
            lo = l % ps if blk == l // ps else 0
            kv[int(bt[b, blk]), :, :, lo:, :] = float("nan")
    q = torch.randn(B, Hq * D, device=DEV).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    o = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=splits, impl="mma")
    _check_status()
    assert torch.isfinite(o.float()).all()
    kv_clean = torch.nan_to_num(kv.float(), nan=0.0).bfloat16()
    assert _rel_err(o, ref.attn_decode(q, kv_clean, bt, sl, Hq, Hkv, D)) < 1e-2


@pytest.mark.parametrize("Hq,Hkv,splits", [(32, 8, 1), (4, 1, 5), (16, 2, 3)])
def test_attn_decode_rope_fusion_equals_separate_kernels(Hq, Hkv, splits):
    """RoPE + KV append + attention in one launch against rope_kv_append followed by attn_decode."""
    torch.manual_seed(9)
    B, D, ps = 8, 128, 16
    lens = [1, 16, 17, 130, 640, 33, 0, 48]
    kv, bt, _ = _make_cache(B, [l + 1 for l in lens], Hkv, D, ps)
    kv2 = kv.clone()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv2 = qkv.clone()
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)     # -1 for the padding row
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tab = ref.rope_cos_sin_table(1024, D, 1e6, DEV)
    assert ops.can_fuse_rope(kv, Hq, Hkv)
    o1 = ops.attn_decode_rope(qkv, pos, bt, tab, kv, sl, Hq, Hkv, D, splits=splits)
    ops.rope_kv_append(qkv2, pos, None, bt, tab, kv2, Hq, Hkv, D)
    o2 = ops.attn_decode(qkv2, kv2, bt, sl, Hq, Hkv, D, splits=splits, impl="mma")
    _check_status()
    assert torch.equal(qkv[:, Hq * D:], qkv2[:, Hq * D:])          # the fused kernel leaves the projection untouched
    assert _rel_err(kv, kv2) < 1e-3
    assert _rel_err(o1, o2) < 5e-3


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 8), (16, 2), (4, 1), (6, 2)])
def test_attn_decode_tcgen05(Hq, Hkv):
    """The tensor-memory decode kernel (tokens on the M side, query heads on N): ragged lengths around the 16-token page
    and the 128-token tile, a padding row, NaN in every cache slot past a context's end."""
    torch.manual_seed(15)
    B, D, ps = 10, 128, 16
    lens = [1, 15, 16, 17, 127, 128, 129, 640, 700, 0]
    kv, bt, _ = _make_cache(B, lens, Hkv, D, ps)
    for b, l in enumerate(lens):
        for blk in range(l // ps, bt.shape[1]):
            lo = l % ps if blk == l // ps else 0
            kv[int(bt[b, blk]), :, :, lo:, :] = float("nan")
    q = torch.randn(B, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    o = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=1, impl="tc")
    o2 = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=1, impl="tc")
    _check_status()
    assert torch.isfinite(o.float()).all() and torch.equal(o, o2)
    clean = torch.nan_to_num(kv.float(), nan=0.0).bfloat16()
    assert _rel_err(o, ref.attn_decode(q, clean, bt, sl, Hq, Hkv, D)) < 1e-2
    assert _rel_err(o, ops.attn_decode(q, clean, bt, sl, Hq, Hkv, D, splits=1, impl="mma")) < 5e-3


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (4, 1), (16, 2)])
def test_attn_decode_tcgen05_rope_fusion_equals_separate_kernels(Hq, Hkv):
    """RoPE + KV append + attention in the tensor-memory kernel against rope_kv_append followed by the mma.sync kernel:
    same cache contents afterwards, same output."""
    torch.manual_seed(19)
    B, D, ps = 8, 128, 16
    lens = [1, 16, 17, 130, 640, 33, 0, 128]
    kv, bt, _ = _make_cache(B, [l + 1 for l in lens], Hkv, D, ps)
    kv2 = kv.clone()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv2 = qkv.clone()
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)     # -1 for the padding row
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tab = ref.rope_cos_sin_table(1024, D, 1e6, DEV)
    o1 = ops.attn_decode_rope(qkv, pos, bt, tab, kv, sl, Hq, Hkv, D, splits=1, impl="tc")
    ops.rope_kv_append(qkv2, pos, None, bt, tab, kv2, Hq, Hkv, D)
    o2 = ops.attn_decode(qkv2, kv2, bt, sl, Hq, Hkv, D, splits=1, impl="mma")
    _check_status()
    assert _rel_err(kv, kv2) < 1e-3
    assert _rel_err(o1, o2) < 5e-3


@pytest.mark.parametrize("impl", ["tc", "mma"])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4)])
def test_attn_prefill(Hq, Hkv, impl, monkeypatch):
    """tc: the tcgen05 kernel (tensor-memory accumulators, TMA page tiles); mma: the mma.sync fallback."""
    monkeypatch.setenv("SKEIN_ATTN_PREFILL", impl)
    torch.manual_seed(6)
    D, ps = 128, 16
    q_lens = [64, 1, 100, 37]
    kv_lens = [64, 50, 228, 37]   # sequences 1 and 2 are chunks on top of cached context
    kv, bt, _ = _make_cache(len(q_lens), kv_lens, Hkv, D, ps)
    T = sum(q_lens)
    q = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qs = torch.tensor([0, 64, 65, 165], dtype=torch.int32, device=DEV)
    ql = torch.tensor(q_lens, dtype=torch.int32, device=DEV)
    kl = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    o = ops.attn_prefill(q, kv, bt, qs, ql, kl, max(q_lens), Hq, Hkv, D)
    _check_status()
    assert _rel_err(o, ref.attn_prefill(q, kv, bt, qs, ql, kl, Hq, Hkv, D)) < 1e-2


@pytest.mark.parametrize("impl", ["tc", "mma"])
def test_attn_prefill_long_and_poisoned(impl, monkeypatch):
    """Several 128-row query tiles and 128-token context tiles per sequence, chunks that start off a tile boundary, and
    a cache whose slots past every sequence's length hold NaN: nothing beyond the context may reach the result."""
    monkeypatch.setenv("SKEIN_ATTN_PREFILL", impl)
    torch.manual_seed(16)
    Hq, Hkv, D, ps = 8, 2, 128, 16
    q_lens = [300, 129, 512, 5]
    kv_lens = [300, 641, 1000, 133]
    kv, bt, mb = _make_cache(len(q_lens), kv_lens, Hkv, D, ps)
    for s_, n in enumerate(kv_lens):                     # poison every slot past the context, and the unused pages
        for b in range(mb):
            lo = max(0, n - b * ps)
            if lo < ps:
                kv[bt[s_, b].long(), :, :, lo:, :] = float("nan")
    T = sum(q_lens)
    q = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    starts = [0]
    for n in q_lens[:-1]:
        starts.append(starts[-1] + n)
    qs = torch.tensor(starts, dtype=torch.int32, device=DEV)
    ql = torch.tensor(q_lens, dtype=torch.int32, device=DEV)
    kl = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    o = ops.attn_prefill(q, kv, bt, qs, ql, kl, max(q_lens), Hq, Hkv, D)
    o2 = ops.attn_prefill(q, kv, bt, qs, ql, kl, max(q_lens), Hq, Hkv, D)
    _check_status()
    assert torch.isfinite(o.float()).all()
    assert torch.equal(o, o2)
    clean = torch.nan_to_num(kv.float(), nan=0.0).bfloat16()
    assert _rel_err(o, ref.attn_prefill(q, clean, bt, qs, ql, kl, Hq, Hkv, D)) < 1e-2


def test_rope_kv_append_matches_reference():
    torch.manual_seed(7)
    T, Hq, Hkv, D, ps = 6, 8, 2, 128, 16
    kv, bt, _ = _make_cache(T, [40] * T, Hkv, D, ps)
    kv2 = kv.clone()
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv2 = qkv.clone()
    pos = torch.tensor([0, 5, 16, 39, -1, 31], dtype=torch.int32, device=DEV)
    tab = ref.rope_cos_sin_table(64, D, 1e6, DEV)
    ops.rope_kv_append(qkv, pos, None, bt, tab, kv, Hq, Hkv, D)
    ref.rope_kv_append(qkv2, pos, None, bt, tab, kv2, Hq, Hkv, D)
    _check_status()
    assert _rel_err(qkv[:, : Hq * D], qkv2[:, : Hq * D]) < 1e-2
    assert _rel_err(kv, kv2) < 1e-2


def test_router_topk_and_plan():
    torch.manual_seed(8)
    T, H, E, k = 64, 4096, 8, 2
    x = torch.randn(T, H, device=DEV).bfloat16()
    wg = (torch.randn(E, H, device=DEV) / 64).bfloat16()
    ids, w, lg = ops.router_topk(x, wg, k, want_logits=True)
    ids_r, w_r, lg_r = ref.router_topk(x, wg, k)
    torch.cuda.synchronize()
    assert (lg - lg_r).abs().max() < 0.1
    # compare selections where the reference margin is not a near-tie
    srt = torch.sort(lg_r, dim=-1, descending=True).values
    clear = (srt[:, k - 1] - srt[:, k]) > 0.05
    assert torch.equal(ids[clear].sort(dim=-1).values, ids_r[clear].sort(dim=-1).values)
    assert (w.sum(-1) - 1).abs().max() < 1e-5
    assert (w[clear].sort(dim=-1).values - w_r[clear].sort(dim=-1).values).abs().max() < 2e-2
    counts, offsets, row_of, src = ops.router_plan(ids, E)
    c2, o2, r2, s2 = ref.router_plan(ids.cpu(), E)
    assert torch.equal(counts.cpu(), c2) and torch.equal(offsets.cpu(), o2)
    assert torch.equal(row_of.cpu(), r2) and torch.equal(src.cpu()[: T * k], s2[: T * k])
    # expert-parallel view: only experts 2..3 are local
    counts, offsets, row_of, src = ops.router_plan(ids, E, e_first=2, e_count=2)
    c2, o2, r2, s2 = ref.router_plan(ids.cpu(), E, 2, 2)
    n = int(o2[-1])
    assert torch.equal(counts.cpu(), c2) and torch.equal(row_of.cpu(), r2) and torch.equal(src.cpu()[:n], s2[:n])


@pytest.mark.parametrize("T,H,E", [(64, 4096, 8), (5, 256, 4), (300, 8192, 16)])
def test_fused_route_equals_two_step(T, H, E):
    torch.manual_seed(11)
    x = torch.randn(T, H, device=DEV).bfloat16()
    wg = (torch.randn(E, H, device=DEV) / 32).bfloat16()
    for e_first, e_count in ((0, E), (E // 2, E // 2)):
        ids, w, counts, offsets, row_of, src = ops.route(x, wg, 2, e_first, e_count)
        ids2, w2, _ = ops.router_topk(x, wg, 2)
        c2, o2, r2, s2 = ops.router_plan(ids2, E, e_first, e_count)
        torch.cuda.synchronize()
        n = int(o2[-1])
        assert torch.equal(ids, ids2) and torch.equal(w, w2)
        assert torch.equal(counts, c2) and torch.equal(offsets, o2) and torch.equal(row_of, r2)
        assert torch.equal(src[:n], s2[:n])


@pytest.mark.parametrize("T,H,E,n_src", [(64, 4096, 8, 1), (5, 256, 4, 0), (128, 6144, 16, 2), (1, 4096, 8, 1)])
def test_reduce_norm_route_equals_separate_kernels(T, H, E, n_src):
    """The one-launch reduce + norm + router + scatter gives exactly what the three separate kernels give,
    on repeated launches (its grid-wide counter re-arms itself)."""
    torch.manual_seed(12)
    res = torch.randn(T, H, device=DEV).bfloat16()
    part = torch.randn(n_src, T, H, device=DEV).bfloat16() if n_src else None
    gamma = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    wg = (torch.randn(E, H, device=DEV) / 32).bfloat16()
    assert ops.can_fuse_route(T, 2)
    for e_first, e_count in ((0, E), (E // 2, E // 2), (0, E)):
        r1, n1 = ops.reduce_residual_rmsnorm(res, part, gamma, 1e-5)
        ids1, w1, c1, o1, row1, src1 = ops.route(n1, wg, 2, e_first, e_count)
        xs1 = ops.gather_rows(n1, src1, n_rows_dev=o1[E:])
        r2, n2, ids2, w2, c2, o2, row2, src2, xs2 = ops.reduce_norm_route(res, part, gamma, 1e-5, wg, 2, e_first, e_count)
        _check_status()
        n = int(o1[-1])
        assert torch.equal(r1, r2) and torch.equal(n1, n2)
        assert torch.equal(ids1, ids2) and torch.equal(w1, w2)
        assert torch.equal(c1, c2) and torch.equal(o1, o2) and torch.equal(row1, row2)
        assert torch.equal(src1[:n], src2[:n]) and torch.equal(xs1[:n], xs2[:n])
    assert ops.workspace().route_barrier.tolist() == [0, 0]


@pytest.mark.parametrize("V,off", [(1003, 0), (1003, 3), (7, 1), (32000, 5), (4099, 8)])
def test_argmax_ragged_rows(V, off):
    """Rows that start off a 16-byte boundary and lengths that are no multiple of eight: the vector scan's head and
    tail, ties included."""
    torch.manual_seed(V + off)
    B = 6
    buf = torch.randn(B, V + 16, device=DEV).bfloat16()
    logits = buf[:, off:off + V]
    logits[2, V - 1] = 40
    logits[3, 0] = 41
    logits[4, V - 1] = 39
    logits[4, min(V - 1, 2)] = 39   # tie -> lower index
    val = torch.empty(B, device=DEV)
    a = ops.sample_argmax(logits, idx_offset=11, out_val=val)
    want = ref.sample_argmax(logits.cpu().contiguous())
    assert torch.equal(a.cpu(), (want + 11).to(torch.int32))
    assert torch.equal(val.cpu(), logits.float().max(dim=1).values.cpu())


def test_sampling():
    torch.manual_seed(9)
    B, V = 5, 32000
    logits = torch.randn(B, V, device=DEV).bfloat16()
    logits[0, 77] = 50
    logits[1, 5] = 60
    logits[1, 4000] = 60  # tie -> lower index
    a = ops.sample_argmax(logits)
    assert torch.equal(a.cpu(), ref.sample_argmax(logits.cpu()))
    temp = torch.tensor([0.0, 1.0, 1.0, 0.7, 1.0], device=DEV)
    tk = torch.tensor([1, 1, 50, 40, 64], dtype=torch.int32, device=DEV)
    tp = torch.tensor([1.0, 1.0, 0.9, 0.5, 1.0], device=DEV)
    seeds = torch.arange(B, device=DEV, dtype=torch.int64)
    step = torch.zeros(1, dtype=torch.int32, device=DEV)
    s = ops.sample(logits, temp, tk, tp, seeds, step)
    torch.cuda.synchronize()
    assert int(s[0]) == 77 and int(s[1]) == 5
    top64 = logits.float().topk(64, dim=-1).indices
    for b in range(2, B):
        assert int(s[b]) in top64[b].tolist()
    # one random-stream counter per row (the token's position): the kernel and the CPU restatement of the same
    # generator draw the same tokens (a draw that lands within rounding of a bucket edge may differ)
    pos = torch.tensor([3, 9, 27, 81, 243], dtype=torch.int32, device=DEV)
    small = torch.randn(B, 4096, device=DEV).bfloat16()
    got = ops.sample(small, temp, tk, tp, seeds, pos).cpu()
    want = ref.sample(small.cpu(), temp.cpu(), tk.cpu(), tp.cpu(), seeds.cpu(), pos.cpu())
    assert int((got != want).sum()) <= 1, (got, want)
    again = ops.sample(small, temp, tk, tp, seeds, pos).cpu()
    assert torch.equal(got, again)
    other = ops.sample(small, temp, tk, tp, seeds + 100, pos).cpu()
    assert not torch.equal(got[2:], other[2:])


def test_split_kv_scratch_is_allocated_once():
    """Captured graphs keep the address of the split-KV scratch: it must not move when a larger batch arrives."""
    ws = ops.workspace()
    p0, c0 = ws.attn_ws.data_ptr(), ws.attn_counters.data_ptr()
    for B, Hq, Hkv, splits in ((1, 32, 8, 16), (8, 32, 8, 2), (64, 4, 1, 2)):
        buf = ws.attn_scratch(B, Hq, Hkv, splits)
        assert buf is not None and buf[0].data_ptr() == p0 and buf[1].data_ptr() == c0
        assert buf[0].numel() >= B * Hq * splits * 130
    assert ws.attn_scratch(256, 32, 8, 16) is None          # beyond what split-KV is ever used for: the caller runs unsplit


def test_embed_gather_rows_quant():
    torch.manual_seed(10)
    table = torch.randn(1000, 512, device=DEV).bfloat16()
    ids = torch.tensor([0, 999, 500, 250], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed(ids, table), table[ids.long()])
    shard = table[250:500]
    e = ops.embed(ids, shard, vocab_start=250)
    assert torch.equal(e[3], table[250]) and float(e[0].abs().sum()) == 0 and float(e[2].abs().sum()) == 0
    src = torch.tensor([3, 3, 0, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.gather_rows(table, src), table[src.long()])
    x = torch.randn(33, 1024, device=DEV).bfloat16()
    x[5] = 0
    q, s = ops.quant_fp8_block128(x)
    q2, s2 = ref.quant_fp8_block128(x)
    assert torch.allclose(s, s2, rtol=1e-6)
    deq = ref.dequant_fp8_block128(q, s)
    assert _rel_err(deq, x) < 0.04
    assert (q.float() - q2.float()).abs().max() <= 32  # at most one e4m3 step apart at the top binade
