"""Single-GPU checks of the communication kernels: page transport, and the bounded flag wait that turns a
peer that never signals into a status code (the wait runs out on a flag that nothing sets; no fault, no hang)."""
import time

import pytest
import torch

from skein_b200 import ops
from skein_b200.ops import _lib
from skein_b200.parallel.kv_transport import LocalKvTransport

pytestmark = pytest.mark.gpu


def test_page_transport_copies_exactly_the_listed_pages():
    torch.manual_seed(0)
    src = [torch.randn(12, 2, 2, 16, 128, device="cuda").bfloat16() for _ in range(3)]
    dst = [torch.zeros(20, 2, 2, 16, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    LocalKvTransport().send_blocks(src, dst, [3, 7, 0], [19, 1, 5])
    torch.cuda.synchronize()
    for s, d in zip(src, dst):
        assert torch.equal(d[19], s[3]) and torch.equal(d[1], s[7]) and torch.equal(d[5], s[0])
        untouched = [i for i in range(20) if i not in (19, 1, 5)]
        assert float(d[untouched].abs().sum()) == 0.0


def test_flag_wait_times_out_with_a_status_instead_of_hanging():
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    t0 = time.time()
    rc = _lib.lib().skein_wait_flag(flag.data_ptr(), 1, 20, status.data_ptr(), _lib.stream_ptr())   # 20 ms budget, nobody sets it
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    assert status.tolist()[0] == 5                       # ST_TIMEOUT_PEER_FLAG
    # the context is still usable, and a flag that is already set passes at once
    flag.fill_(3)
    status.zero_()
    _lib.lib().skein_wait_flag(flag.data_ptr(), 2, 20, status.data_ptr(), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]
    assert torch.equal(ops.rmsnorm(torch.ones(2, 256, device="cuda").bfloat16(), torch.ones(256, device="cuda").bfloat16(), 1e-5).float(),
                       torch.ones(2, 256, device="cuda"))


def test_reduce_kernel_reports_a_missing_peer():
    """The fused reduce waits for per-source flags; a source that never publishes makes it return with status 5."""
    B, H = 4, 256
    part = torch.zeros(2, B, H, device="cuda", dtype=torch.bfloat16)
    flags = torch.tensor([1, 0], dtype=torch.int32, device="cuda")      # source 1 never reached epoch 1
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    res = torch.ones(B, H, device="cuda", dtype=torch.bfloat16)
    ops.reduce_residual_rmsnorm(res, part, torch.ones(H, device="cuda", dtype=torch.bfloat16), 1e-5, flags=flags, epoch=epoch,
                                wait_budget_ms=10)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.workspace().check_status()
    ops.workspace().check_status()                                      # cleared after being reported
