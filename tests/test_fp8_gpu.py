"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 + per-K-block scaling in the epilogue) against the fp32
reference of the same quantised operands: dense, SwiGLU pair, grouped/ragged, and end-to-end error vs bf16."""
import math

import pytest
import torch

from skein_b200 import ops
from skein_b200.ops import fp8, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("T,F,K,swiglu", [(16, 256, 512, False), (64, 1024, 4096, False), (7, 384, 1024, True), (40, 1792, 4096, True),
                                          (130, 512, 2048, False)])
def test_fp8_linear(T, F, K, swiglu):
    torch.manual_seed(0)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(2 * F if swiglu else F, K, device=DEV) / math.sqrt(K)).bfloat16()
    wq = fp8.quantize_weight(w)
    xq, xs = ops.quant_fp8_block128(x)
    y = fp8.linear(xq, xs, wq, swiglu=swiglu)
    y2 = fp8.linear(xq, xs, wq, swiglu=swiglu)
    torch.cuda.synchronize(); ops.workspace().check_status()
    assert torch.equal(y, y2)
    want = fp8._ref_linear(xq.cpu(), xs.cpu(), fp8.Fp8Weight(wq.q.cpu(), wq.scale_t.cpu(), wq.shape), swiglu)
    assert rel(y, want) < 1e-2
    # and the quantisation error against the bf16 operator stays in the expected band
    full = ref.swiglu_linear(x, w) if swiglu else ref.linear(x, w)
    assert rel(y, full) < 0.08


@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_grouped(swiglu):
    torch.manual_seed(1)
    E, F, K = 8, 512, 1024
    counts = [1, 33, 0, 16, 40, 5, 12, 7]
    rows = sum(counts)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    off = torch.zeros(E + 1, dtype=torch.int32, device=DEV); off[1:] = torch.cumsum(cnt, 0)
    xs_ = torch.randn(rows, K, device=DEV).bfloat16()
    w = (torch.randn(E, 2 * F if swiglu else F, K, device=DEV) / math.sqrt(K)).bfloat16()
    wq = fp8.quantize_weight(w)
    xq, xs = ops.quant_fp8_block128(xs_)
    y = fp8.grouped_linear(xq, xs, wq, cnt, off, swiglu=swiglu)
    torch.cuda.synchronize(); ops.workspace().check_status()
    want = fp8.grouped_linear(xq.cpu(), xs.cpu(), fp8.Fp8Weight(wq.q.cpu(), wq.scale_t.cpu(), wq.shape), cnt.cpu(), off.cpu(), swiglu=swiglu)
    assert rel(y, want) < 1e-2


# ---- e4m3 weights with bf16 activations: e4m3 tiles streamed, rescaled to bf16 in shared memory, one accumulator --------
@pytest.mark.parametrize("T,F,K,swiglu", [(16, 256, 512, False), (64, 1024, 4096, False), (7, 384, 1024, True), (40, 1792, 4096, True),
                                          (130, 512, 2048, False), (64, 4096, 1792 + 128 * 2, False), (3, 200, 256, False)])
def test_fp8_weight_bf16_activation_linear(T, F, K, swiglu):
    torch.manual_seed(0)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(2 * F if swiglu else F, K, device=DEV) / math.sqrt(K)).bfloat16()
    wq = fp8.quantize_weight(w)
    y = fp8.linear_a16(x, wq, swiglu=swiglu)
    y2 = fp8.linear_a16(x, wq, swiglu=swiglu)
    torch.cuda.synchronize(); ops.workspace().check_status()
    assert torch.equal(y, y2)                                   # deterministic whatever the split of the K loop
    wd = fp8.Fp8Weight(wq.q.cpu(), wq.scale_t.cpu(), wq.shape).dequant()
    want = ref.swiglu_linear(x.cpu(), wd) if swiglu else ref.linear(x.cpu(), wd)     # fp32 reference on the dequantised weight
    assert rel(y, want) < 8e-3, rel(y, want)
    full = ref.swiglu_linear(x, w) if swiglu else ref.linear(x, w)
    assert rel(y, full) < 0.06                                  # quantisation error against the bf16 weight


@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_weight_bf16_activation_grouped(swiglu):
    torch.manual_seed(1)
    E, F, K = 8, 512, 1024
    counts = [1, 33, 0, 16, 40, 5, 12, 7]
    rows = sum(counts)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    off = torch.zeros(E + 1, dtype=torch.int32, device=DEV); off[1:] = torch.cumsum(cnt, 0)
    xs_ = torch.randn(rows, K, device=DEV).bfloat16()
    w = (torch.randn(E, 2 * F if swiglu else F, K, device=DEV) / math.sqrt(K)).bfloat16()
    wq = fp8.quantize_weight(w)
    y = fp8.grouped_linear_a16(xs_, wq, cnt, off, swiglu=swiglu)
    torch.cuda.synchronize(); ops.workspace().check_status()
    wd = fp8.Fp8Weight(wq.q.cpu(), wq.scale_t.cpu(), wq.shape).dequant()
    want = ref.grouped_linear(xs_.cpu(), wd, cnt.cpu(), off.cpu(), swiglu)
    assert rel(y, want) < 8e-3, rel(y, want)


@pytest.mark.parametrize("shape", [(384, 1024), (3, 256, 512), (1000, 128)])
@pytest.mark.parametrize("pow2", [True, False])
def test_fp8_weight_expansion_matches_reference(shape, pow2):
    """The one-pass expansion of an e4m3 weight to bf16 (prefill-sized projections) against the reference
    dequantisation of the same stored blocks; with power-of-two scales it is exact."""
    torch.manual_seed(5)
    w = (torch.randn(*shape, device=DEV) * 0.05).bfloat16()
    wq = fp8.quantize_weight(w, pow2_scales=pow2)
    got = wq.dequant()
    rows_total, K = wq.scale_t.shape[1], shape[-1]
    want = ref.dequant_fp8_block128(wq.q.reshape(rows_total, K).cpu(), wq.scale_t.t().contiguous().cpu()).view(*shape)
    assert got.shape == tuple(shape) and got.dtype == torch.bfloat16
    assert torch.equal(got.cpu(), want.to(torch.bfloat16))
    assert rel(got, w) < 0.05


def test_quantiser_matches_reference_blocks():
    """The block quantiser (half a warp per 1 x 128 block) against the CPU restatement: scales and codes."""
    torch.manual_seed(6)
    x = (torch.randn(77, 1024, device=DEV) * 3).bfloat16()
    x[5, 128:256] = 0          # a zero block keeps scale 1
    q, s = ops.quant_fp8_block128(x)
    q_ref, s_ref = ref.quant_fp8_block128(x.cpu())
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-6, atol=0)
    same = (q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean()
    assert same > 0.999, same          # a code may differ by one step where x / scale sits on a rounding boundary
