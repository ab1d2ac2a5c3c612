"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernel library may not allocate device memory when they run attention (an arena that
is closed after start-up, a plug-in inside a process whose allocator owns the device, a latency-critical
loop), so skein_attn_decode_noalloc keeps the split-KV scratch inside the library. This test calls the
raw symbol with ctypes, twice in a row on different inputs (the scratch is shared and keeps the previous
call's contents, so the second call proves it is cleared correctly), and compares each result with the
regular entry point, which receives caller-allocated scratch. It also checks that an oversized problem is
refused with the documented error instead of overrunning the built-in array.

Named test_zz_* so that pytest collects it after every other test file.
"""
import ctypes as C

import pytest
import torch

from skein_b200 import ops
from skein_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _symbol():
    L = _lib.lib()
    fn = L.skein_attn_decode_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                   C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]
    err = L.skein_attn_decode_noalloc_strerror
    err.restype = C.c_char_p
    err.argtypes = [C.c_int]
    return fn, err


def _case(seed, B, Hq, Hkv, lens, splits):
    torch.manual_seed(seed)
    D, ps = 128, 16
    max_blocks = max((l + ps - 1) // ps for l in lens) + 1
    num_pages = B * max_blocks + 5
    kv = torch.randn(num_pages, 2, Hkv, ps, D, device="cuda").bfloat16()
    bt = torch.randperm(num_pages, device="cuda")[: B * max_blocks].view(B, max_blocks).to(torch.int32).contiguous()
    q = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, kv, bt, sl, D, ps, max_blocks, num_pages


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    fn, err = _symbol()
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for seed, (B, Hq, Hkv, lens, splits) in enumerate([(6, 32, 8, [700, 33, 512, 1, 130, 257], 4), (5, 8, 8, [90, 600, 17, 300, 45], 3)]):
        q, kv, bt, sl, D, ps, max_blocks, num_pages = _case(seed, B, Hq, Hkv, lens, splits)
        # the entry point it is a variant of: the scalar split-KV kernel with caller-provided scratch
        want = ops.attn_decode(q, kv, bt, sl, Hq, Hkv, D, splits=splits, impl="scalar")
        out = torch.empty(B, Hq * D, dtype=torch.bfloat16, device="cuda")
        rc = fn(q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), status.data_ptr(), B, Hq, Hkv, D,
                ps, max_blocks, num_pages, splits, 1.0 / D ** 0.5, stream)
        assert rc == 0, err(rc)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0]
        rel = float((out.float() - want.float()).norm() / want.float().norm())
        assert rel < 1e-2, rel
        assert torch.equal(out, want)      # same kernel, same split boundaries: bit-identical


def test_noalloc_refuses_oversized_problems():
    fn, err = _symbol()
    q, kv, bt, sl, D, ps, max_blocks, num_pages = _case(0, 2, 8, 8, [20, 30], 1)
    out = torch.empty(2, 8 * D, dtype=torch.bfloat16, device="cuda")
    too_many_splits = 8192 // (2 * 8) + 1
    rc = fn(q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), None, 2, 8, 8, D, ps, max_blocks,
            num_pages, too_many_splits, 0.1, torch.cuda.current_stream().cuda_stream)
    assert rc == -2 and b"exceeds the built-in scratch" in err(rc)
    rc = fn(q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), None, 2, 8, 8, 64, ps, max_blocks,
            num_pages, 1, 0.1, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
