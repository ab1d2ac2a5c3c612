"""KV page transport for prefill/decode disaggregation: copy whole pages (all layers) from a prefill rank's
pools into a decode rank's pools.

    LocalKvTransport   both pools live on this device (one process serving both roles, and the tests)
    PeerKvTransport    the destination pools are another GPU's memory mapped into this process (symmetric
                       heap / CUDA IPC pointer): the copy kernel stores straight over NVLink, page by page,
                       one launch per layer so that layer i can leave while layer i + 1 is still being computed
                       ("layer_overlap" in the plan's transfer topology)

Counterpart of the reference's KvTransport trait with its local implementation, RDMA stubs and host-staged
NCCL send/recv of f32 blocks (crates/skein_runtime/src/kv_transport/mod.rs:6-40, cuda/rdma.rs:9-26,
cuda/nccl.rs:504-588).
"""
from __future__ import annotations

import torch

from ..ops import _lib


def copy_pages(src_cache: torch.Tensor, dst_ptr: int, src_pages: torch.Tensor, dst_pages: torch.Tensor) -> None:
    """dst[dst_pages[i]] = src[src_pages[i]] for one layer's pool. `dst_ptr` is a raw device address (local or peer)."""
    n = src_pages.shape[0]
    if n == 0:
        return
    page_bytes = src_cache.stride(0) * src_cache.element_size()
    if not src_cache.is_cuda:
        raise ValueError("copy_pages works on device pools")
    rc = _lib.lib().skein_copy_pages(src_cache.data_ptr(), dst_ptr, src_pages.data_ptr(), dst_pages.data_ptr(), n, page_bytes,
                                     _lib.stream_ptr())
    _lib.check(rc, "copy_pages")
    _lib.count_launch()


class LocalKvTransport:
    def send_blocks(self, src_pools, dst_pools, src_pages, dst_pages):
        """Pools: list of per-layer tensors [pages, 2, kv_heads, page_size, D]. Page lists: python ints."""
        if not src_pools:
            return
        dev = src_pools[0].device
        if dev.type != "cuda":
            for s, d in zip(src_pools, dst_pools):
                d[torch.tensor(dst_pages, dtype=torch.long)] = s[torch.tensor(src_pages, dtype=torch.long)]
            return
        sp = torch.tensor(src_pages, dtype=torch.int32, device=dev)
        dp = torch.tensor(dst_pages, dtype=torch.int32, device=dev)
        for s, d in zip(src_pools, dst_pools):
            copy_pages(s, d.data_ptr(), sp, dp)


class PeerKvTransport:
    """dst_pool_ptrs[layer] = address of the destination rank's pool of that layer, valid in this process."""

    def __init__(self, dst_pool_ptrs):
        self.dst_pool_ptrs = list(dst_pool_ptrs)

    def send_blocks(self, src_pools, src_pages, dst_pages):
        dev = src_pools[0].device
        sp = torch.tensor(src_pages, dtype=torch.int32, device=dev)
        dp = torch.tensor(dst_pages, dtype=torch.int32, device=dev)
        for s, ptr in zip(src_pools, self.dst_pool_ptrs):
            copy_pages(s, ptr, sp, dp)
