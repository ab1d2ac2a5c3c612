"""Prefill / decode disaggregation between two GPUs: the prefill rank computes a prompt's KV pages and stores them
straight into the decode rank's page pools over NVLink, the decode rank generates from there.

    HeapKvPools         per-layer KV page pools carved out of a symmetric heap, so that the peer's pools are mapped
                        into this process (CUDA IPC) and a kernel here can store into them
    ship_prompt         prefill rank: run the prompt, copy its pages into the peer's pools (one launch per layer,
                        `PeerKvTransport`), make the copies visible, send the first token
    receive_prompt      decode rank: wait for the first token (which arrives after the pages), return it

The plan side is `extract --disaggregate-decode-devices` (csrc/core/planner.hpp); this is the serving flow behind
it for one prefill rank and one decode rank. Counterpart of the reference's KV block transport between its
prefill and decode ranks (crates/skein_runtime/src/cuda/nccl.rs:504-588 send_blocks / recv_blocks, host-staged
f32 blocks over NCCL; crates/skein_extract/src/disaggregate.rs:73).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .kv_transport import PeerKvTransport
from .symm import SymmetricHeap


class HeapKvPools:
    """`n_layers` pools of shape [pages, 2, kv_heads, page_size, head_dim] (bf16) inside one symmetric heap."""

    def __init__(self, group, device, n_layers: int, num_pages: int, kv_heads: int, page_size: int, head_dim: int):
        self.shape = (num_pages, 2, kv_heads, page_size, head_dim)
        self.pool_bytes = num_pages * 2 * kv_heads * page_size * head_dim * 2
        self.heap = SymmetricHeap(group, device, n_layers * (self.pool_bytes + 256) + 4096)
        self.offsets = [self.heap.alloc(self.pool_bytes) for _ in range(n_layers)]
        self.pools = [self.heap.view(o, self.shape, torch.bfloat16) for o in self.offsets]
        self.rank, self.size = self.heap.rank, self.heap.size

    def peer_pool_ptrs(self, peer: int):
        """Addresses, valid in this process, of rank `peer`'s pools (one per layer)."""
        return [self.heap.peer_ptr(peer, o) for o in self.offsets]

    def close(self):
        self.pools = []
        self.heap.close()


def ship_prompt(runner, pools: HeapKvPools, decode_rank: int, prompt, table_here, table_there, group=None):
    """Prefill rank. Runs `prompt` through `runner` (its decoder must use `pools.pools` as KV cache) into pages
    `table_here`, copies those pages into pages `table_there` of the decode rank's pools, and sends the first token.
    Returns the first token."""
    first = runner.prefill([(list(prompt), list(table_here), 0)])[0]
    n = (len(prompt) + runner.dec.page_size - 1) // runner.dec.page_size
    PeerKvTransport(pools.peer_pool_ptrs(decode_rank)).send_blocks(pools.pools, list(table_here[:n]), list(table_there[:n]))
    # the stores went over NVLink from kernels on this stream: once the stream has drained they are complete at the
    # peer; the token that follows is the decode rank's signal that its pages are in place
    torch.cuda.current_stream().synchronize()
    tok = torch.tensor([first, len(prompt)], dtype=torch.int32, device=pools.pools[0].device)
    dist.send(tok, dst=decode_rank, group=group)
    return first


def receive_prompt(pools: HeapKvPools, prefill_rank: int, group=None):
    """Decode rank. Blocks until the prefill rank has shipped a prompt; returns (first token, prompt length)."""
    tok = torch.zeros(2, dtype=torch.int32, device=pools.pools[0].device)
    dist.recv(tok, src=prefill_rank, group=group)
    first, n = tok.tolist()
    return int(first), int(n)
