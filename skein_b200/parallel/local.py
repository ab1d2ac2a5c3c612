"""CPU ranks inside one process: N threads, one per rank, meeting at barriers.

`BarrierComm` implements the communicator interface the decoder uses (`linear_push`,
`vocab_parallel_argmax`, `all_reduce`) with plain tensors in shared slots and a `threading.Barrier`, so
a tensor-parallel (or any sharded) model can run on a machine without GPUs: every rank thread runs
its own Decoder shard through the fp32 reference operators. It is the oracle for the fused GPU
collectives and the vehicle for host-side failure tests (a rank that raises or never arrives breaks
the barrier and every other rank gets a CommError instead of waiting forever).

Counterpart of the reference's BarrierCollective (crates/skein_runtime/src/distributed/
barrier_collective.rs:29-170) and LocalTopology (distributed/local_topology.rs:25-334).
"""
from __future__ import annotations

import threading

import torch

from .. import ops


class CommError(RuntimeError):
    pass


class _Shared:
    def __init__(self, n: int, timeout_s: float):
        self.n = n
        self.barrier = threading.Barrier(n)
        self.slots = [None] * n
        self.timeout_s = timeout_s


class BarrierComm:
    mode = "barrier"

    def __init__(self, shared: _Shared, rank: int):
        self.sh, self.rank, self.size = shared, rank, shared.n

    def _wait(self):
        try:
            self.sh.barrier.wait(self.sh.timeout_s)
        except threading.BrokenBarrierError as e:
            raise CommError(f"rank {self.rank}: a peer did not reach the collective (barrier broken or timed out)") from e

    def _exchange(self, value):
        self.sh.slots[self.rank] = value
        self._wait()
        vals = list(self.sh.slots)
        self._wait()            # nobody overwrites a slot before everyone has read it
        return vals

    def linear_push(self, x, w, grouped=None):
        y = ops.grouped_linear(x, w, *grouped) if grouped is not None else ops.linear(x, w)
        return torch.stack(self._exchange(y)), None, None

    def all_reduce(self, x):
        return torch.stack([v.float() for v in self._exchange(x)]).sum(0).to(x.dtype)

    def embed_reduce(self, ids, table_shard, vocab_start, gamma, eps):
        """Vocabulary-parallel embedding: each rank looks up the rows it owns (zeros elsewhere), the sum is the row."""
        x = self.all_reduce(ops.embed(ids, table_shard, vocab_start))
        return x, ops.rmsnorm(x, gamma, eps)

    def all_gather(self, x):
        return torch.cat(self._exchange(x), dim=0)

    def vocab_parallel_argmax(self, logits, v_local):
        return ops.sample_argmax(torch.cat(self._exchange(logits), dim=1))

    def abort(self):
        self.sh.barrier.abort()

    def subgroup(self, ranks) -> "BarrierComm":
        """Communicator over a subset of the world's ranks (every member must ask for the same tuple)."""
        ranks = tuple(ranks)
        world = self.world_shared if hasattr(self, "world_shared") else self.sh
        with world_lock:
            groups = world.__dict__.setdefault("groups", {})
            if ranks not in groups:
                groups[ranks] = _Shared(len(ranks), world.timeout_s)
        my_world_rank = self.world_rank if hasattr(self, "world_rank") else self.rank
        c = BarrierComm(groups[ranks], ranks.index(my_world_rank))
        c.world_shared, c.world_rank = world, my_world_rank
        return c


world_lock = threading.Lock()


def run_ranks(n: int, fn, timeout_s: float = 60.0):
    """Run fn(rank, comm) on n threads. Returns the list of results; re-raises the first rank exception after
    aborting the barrier so that the other ranks fail fast with CommError."""
    shared = _Shared(n, timeout_s)
    results, errors = [None] * n, [None] * n

    def body(r):
        comm = BarrierComm(shared, r)
        try:
            results[r] = fn(r, comm)
        except BaseException as e:  # noqa: BLE001
            errors[r] = e
            shared.barrier.abort()

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s * 2)
    first = next((e for e in errors if e is not None and not isinstance(e, CommError)), None) or next((e for e in errors if e), None)
    if first is not None:
        raise first
    return results, errors
