"""Tensor-parallel communicator: the collectives of a decoder block, fused into its kernels.

Fused mode (decode and small prefill chunks). A row-parallel projection (o_proj, expert down)
stores its partial output from the GEMM epilogue into a local buffer that every peer has mapped, and
the last CTA of the launch sets this rank's flag word on every peer (one system-scope fence per
launch). The kernel that consumes the sum (residual + RMSNorm, csrc/kernels/norm.cu) waits on the
flags and pulls all ranks' partials over NVLink with plain peer loads, every load of a row in flight
at once, and adds them in rank order. A block therefore launches no collective, the GEMM issues no
remote store, and the NVLink traffic sits in a kernel with thousands of independent loads. (Pushing
the tile into every peer from the GEMM epilogue instead, as an earlier version did, measured 28 us per
all-reduce at 8 ranks: two system-scope fences and 8 stores per element on 128 epilogue threads.)
Two buffers alternate: a rank can only be one all-reduce ahead of the slowest peer, because it cannot
finish all-reduce k+1 without that peer's flag, which the peer sets only after it has consumed (read)
all-reduce k; so nobody overwrites a buffer that is still being read.

Comparison arms: SKEIN_COMM=unfused keeps the data path but takes the fusion out (GEMM stores to ordinary
memory, a copy kernel publishes, the reduce kernel pulls; still capturable into the step's CUDA graph, so
graph-against-graph it shows what the publish epilogue saves); SKEIN_COMM=nccl replaces the whole exchange by
a library all-reduce between the local GEMM and the reduce kernel, launched eagerly.

The stand-alone collectives (all_reduce, all_gather, reduce_scatter, all_to_all) are the same two steps
without a GEMM in front: copy into the published buffer and raise the flags, then one pull kernel
(csrc/kernels/comm.cu) that reads the chunks this rank needs out of every peer's buffer. Messages
larger than the buffer go through the library.

Greedy sampling is vocabulary-parallel: each rank reduces its logit shard to one candidate per row
and pushes 8 bytes per row to every peer.

The reference does these with ncclAllReduce + a device copy back (crates/skein_runtime/src/cuda/
nccl.rs:196-245), a 2-rank host-memory kernel under capture (cuda/shm_allreduce.rs:24-69) and an
all-gather of logits (nccl.rs:251-298).
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from .symm import SymmetricHeap


class PeerPartials:
    """Operand of the reduce kernels: rank s's partial result is the [rows, H] buffer at ptrs[s] (peer-mapped
    memory), complete once flags[s] has reached the device-side epoch."""

    def __init__(self, local, ptrs, n_src, flags, epoch, wait_budget_ms=0, mc=0):
        self.local, self.ptrs, self.n_src, self.flags, self.epoch = local, ptrs, n_src, flags, epoch
        self.mc = mc                           # multicast address of the same buffer on all ranks (0: none)
        self.rows = local.shape[0]
        self.wait_budget_ms = wait_budget_ms   # how long the consumer waits for a peer's flag (0: kernel default)


class TPComm:
    def __init__(self, group, device, hidden: int, fused_rows: int = 512, max_batch: int = 256, mode: str | None = None,
                 wait_budget_ms: int | None = None, multimem: bool | None = None, sp_min_rows: int = 512,
                 embed_rows: int | None = None):
        self.group, self.device = group, device
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.hidden, self.fused_rows, self.max_batch = hidden, fused_rows, max_batch
        self.sp_min_rows = sp_min_rows     # chunks with more token rows than this are sharded by rows between projections
        self.mode = mode or os.environ.get("SKEIN_COMM", "fused")
        self.wait_budget_ms = wait_budget_ms if wait_budget_ms is not None else int(os.environ.get("SKEIN_PEER_WAIT_MS", "10000"))
        N = self.size
        buf_bytes = fused_rows * hidden * 2
        # a third, smaller buffer carries the vocabulary-parallel embedding rows (one exchange per step, which must not
        # alternate with the two buffers of the per-block exchanges: a step has an even number of those)
        self.embed_rows = min(fused_rows, 8192) if embed_rows is None else embed_rows
        embed_bytes = self.embed_rows * hidden * 2
        heap_bytes = 2 * buf_bytes + embed_bytes + 6 * 256 + 2 * N * max_batch * 4 + 8192
        # In-switch reduction (SKEIN_MULTIMEM=1): the heap is bound to an NVLink multicast object and the reduce
        # kernels sum the ranks' partials with one multimem load. Off by default: a rank that dies while bound
        # faults its peers, and the plain peer loads are what the failure-handling tests exercise.
        self.multimem = (os.environ.get("SKEIN_MULTIMEM", "0") == "1") if multimem is None else bool(multimem)
        want_mc = self.multimem and self.mode in ("fused", "unfused")
        self.heap = None
        if want_mc:
            # a group without NVLink multicast (or a torch build without the symmetric-memory allocator) falls back to the
            # plain heap, on every rank or on none
            ok, err = 1, None
            try:
                self.heap = SymmetricHeap(group, device, heap_bytes, multicast=True)
            except Exception as e:      # noqa: BLE001
                ok, err = 0, e
            agreed = torch.tensor([ok], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if int(agreed[0]) == 0:
                if self.heap is not None:
                    self.heap.close()
                    self.heap = None
                if self.rank == 0:
                    import sys
                    print(f"skein: no in-switch reduction for this group ({err or 'a peer could not bind its heap'}); "
                          "using peer loads", file=sys.stderr)
                self.multimem = False
        if self.heap is None:
            self.heap = SymmetricHeap(group, device, heap_bytes, multicast=False)
        h = self.heap
        self.buf_off = [h.alloc(buf_bytes) for _ in range(2)]
        self.flag_off = [h.alloc(256) for _ in range(2)]
        self.cand_val_off = h.alloc(N * max_batch * 4)
        self.cand_idx_off = h.alloc(N * max_batch * 4)
        self.cand_flag_off = h.alloc(256)
        self.embed_off = h.alloc(max(embed_bytes, 256))
        self.embed_flag_off = h.alloc(256)
        self.embed_buf = h.view(self.embed_off, (self.embed_rows, hidden), torch.bfloat16) if self.embed_rows else None
        self.embed_flags = h.view(self.embed_flag_off, (N,), torch.int32)
        self.bufs = [h.view(o, (fused_rows, hidden), torch.bfloat16) for o in self.buf_off]   # this rank's partials
        self.flags = [h.view(o, (N,), torch.int32) for o in self.flag_off]                     # [source rank]
        self.cand_val = h.view(self.cand_val_off, (N, max_batch), torch.float32)
        self.cand_idx = h.view(self.cand_idx_off, (N, max_batch), torch.int32)
        self.cand_flags = h.view(self.cand_flag_off, (N,), torch.int32)
        # local, not shared: epochs and "all CTAs done" counters of buffers 0/1, of the candidate exchange and of
        # the embedding exchange
        self.epochs = torch.zeros(4, dtype=torch.int32, device=device)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        self.cur = 0
        r = self.rank
        VP = C.c_void_p * N
        self._src_ptrs = [VP(*[h.peer_ptr(p, self.buf_off[b]) for p in range(N)]) for b in range(2)]
        self._peer_flag = [[h.peer_ptr(p, self.flag_off[b] + 4 * r) for p in range(N)] for b in range(2)]
        self._cand_val_ptrs = VP(*[h.peer_ptr(p, self.cand_val_off + 4 * r * max_batch) for p in range(N)])
        self._cand_idx_ptrs = VP(*[h.peer_ptr(p, self.cand_idx_off + 4 * r * max_batch) for p in range(N)])
        self._cand_flag_ptrs = VP(*[h.peer_ptr(p, self.cand_flag_off + 4 * r) for p in range(N)])
        self._push_flag = [VP(*self._peer_flag[b]) for b in range(2)]
        self._embed_src_ptrs = VP(*[h.peer_ptr(p, self.embed_off) for p in range(N)])
        self._embed_push_flag = VP(*[h.peer_ptr(p, self.embed_flag_off + 4 * r) for p in range(N)])
        ops.workspace(device).peer_state.append((self.epochs, self.done))

    def even_out(self):
        """Called at the end of a step. The two published buffers alternate, and using the same buffer for two
        CONSECUTIVE exchanges is the one thing the protocol does not allow (a fast rank would overwrite what a slow peer
        still reads; any exchange in between proves that everybody has finished reading). A step with an odd number of
        exchanges would end on the buffer the next step (or the next replay of its captured graph) starts with, so it
        gets one empty exchange on the other buffer: flags only, no data."""
        if self.cur == 0 or self.mode == "nccl" or self.size == 1:
            return
        b = self.cur
        self.cur ^= 1
        L = _lib.lib()
        _lib.check(L.skein_publish_rows(None, 0, None, self._push_flag[b], self.size, self.epochs[b:b + 1].data_ptr(),
                                        self.done[b:b + 1].data_ptr(), _lib.stream_ptr()), "publish (empty exchange)")
        _lib.check(L.skein_pull_collective(self._PULL_ALL_GATHER, self._src_ptrs[b], self.size, self.rank, 0, self.bufs[b].data_ptr(),
                                           self.flags[b].data_ptr(), self.epochs[b:b + 1].data_ptr(),
                                           ops.workspace().status.data_ptr(), self.wait_budget_ms, _lib.stream_ptr()),
                   "wait (empty exchange)")
        _lib.count_launch(2)

    def reset(self):
        """Back to the state of a fresh communicator: flag words, epochs, arrival counters zero, buffer 0 next. Every
        rank of the group must call this between the same two steps, with none of its kernels in flight and a
        barrier on both sides (parallel/worker.py: make_resync)."""
        for f in self.flags:
            f.zero_()
        self.cand_flags.zero_()
        self.embed_flags.zero_()
        self.epochs.zero_()
        self.done.zero_()
        self.cur = 0

    def _partials(self, b: int, rows: int) -> PeerPartials:
        return PeerPartials(self.bufs[b][:rows], self._src_ptrs[b], self.size, self.flags[b], self.epochs[b:b + 1],
                            self.wait_budget_ms, mc=self.heap.mc_addr(self.buf_off[b]))

    # ---- row-parallel projection + all-reduce ------------------------------------------------------
    def _fused_ok(self, rows: int) -> bool:
        return self.mode in ("fused", "unfused") and rows <= self.fused_rows

    def _publish(self, y: torch.Tensor, b: int) -> None:
        """Copy a finished [rows, H] result into this rank's peer-mapped buffer `b` and raise the flags (one launch)."""
        rc = _lib.lib().skein_publish_rows(y.data_ptr(), y.numel() * 2, self.bufs[b].data_ptr(), self._push_flag[b],
                                           self.size, self.epochs[b:b + 1].data_ptr(), self.done[b:b + 1].data_ptr(),
                                           _lib.stream_ptr())
        _lib.check(rc, "publish_rows")
        _lib.count_launch()

    def _zeros(self, rows):
        return torch.zeros(rows, self.hidden, dtype=torch.bfloat16, device=self.device)

    def linear_push(self, x, w, grouped=None):
        """Returns (partial, flags, epoch) for ops.reduce_residual_rmsnorm: peer partials in fused mode, else the
        all-reduced [1, rows, H] tensor and no flags."""
        rows = x.shape[0]
        if not self._fused_ok(rows):
            # rows that belong to no local expert (expert parallelism) must add nothing to the sum
            y = (ops.grouped_linear(x, w, *grouped, out=self._zeros(rows)) if grouped is not None else ops.linear(x, w))
            dist.all_reduce(y, group=self.group)
            return y.unsqueeze(0), None, None
        b = self.cur
        self.cur ^= 1
        if self.mode == "unfused":
            # comparison arm: the same data path without the fusion. The GEMM stores into ordinary memory, a second
            # kernel copies the result into the published buffer and raises the flags; the consumer pulls as usual.
            y = ops.grouped_linear(x, w, *grouped) if grouped is not None else ops.linear(x, w)
            self._publish(y, b)
        else:
            ops.linear_push(x, w, self.bufs[b], self._peer_flag[b], self.epochs[b:b + 1], self.done[b:b + 1],
                            self.hidden, grouped=grouped, wait_budget_ms=0)
        part = self._partials(b, rows)
        return part, part.flags, part.epoch

    def linear_push_fp8(self, xq, xs, w8, grouped=None, rows_hint=None):
        """linear_push for a block-scaled e4m3 weight (ops/fp8.py). With `xs` None, `xq` holds bf16 activations
        (weights fp8, activations bf16: the form the decoder uses); otherwise pre-quantised e4m3 activations with
        their block scales."""
        from ..ops import fp8
        rows = xq.shape[0]
        if xs is None:
            x = xq
            if not self._fused_ok(rows):
                y = (fp8.grouped_linear_a16(x, w8, *grouped, rows_hint=rows_hint, out=self._zeros(rows)) if grouped is not None
                     else fp8.linear_a16(x, w8))
                dist.all_reduce(y, group=self.group)
                return y.unsqueeze(0), None, None
            b = self.cur
            self.cur ^= 1
            if self.mode == "unfused":
                y = fp8.grouped_linear_a16(x, w8, *grouped, rows_hint=rows_hint) if grouped is not None else fp8.linear_a16(x, w8)
                self._publish(y, b)
            else:
                fp8.linear_publish_a16(x, w8, self.bufs[b], self._peer_flag[b], self.epochs[b:b + 1], self.done[b:b + 1],
                                       self.hidden, grouped=grouped, rows_hint=rows_hint)
            part = self._partials(b, rows)
            return part, part.flags, part.epoch
        if not self._fused_ok(rows):
            y = (fp8.grouped_linear(xq, xs, w8, *grouped, rows_hint=rows_hint, out=self._zeros(rows)) if grouped is not None
                 else fp8.linear(xq, xs, w8))
            dist.all_reduce(y, group=self.group)
            return y.unsqueeze(0), None, None
        b = self.cur
        self.cur ^= 1
        if self.mode == "unfused":
            y = fp8.grouped_linear(xq, xs, w8, *grouped, rows_hint=rows_hint) if grouped is not None else fp8.linear(xq, xs, w8)
            self._publish(y, b)
        else:
            fp8.linear_publish(xq, xs, w8, self.bufs[b], self._peer_flag[b], self.epochs[b:b + 1], self.done[b:b + 1],
                               self.hidden, grouped=grouped, rows_hint=rows_hint)
        part = self._partials(b, rows)
        return part, part.flags, part.epoch

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Stand-alone sum all-reduce of a [rows, H] bf16 tensor (publish + pull-and-sum)."""
        rows = x.shape[0]
        if not self._fused_ok(rows) or x.shape[1] != self.hidden:
            y = x.clone()
            dist.all_reduce(y, group=self.group)
            return y
        b = self.cur
        self.cur ^= 1
        self._publish(x.contiguous(), b)
        out, _ = ops.reduce_residual_rmsnorm(None, self._partials(b, rows), None, 0.0,
                                             wait_budget_ms=self.wait_budget_ms)
        return out

    # ---- vocabulary-parallel embedding ---------------------------------------------------------------------------
    def embed_reduce(self, ids, table_shard, vocab_start: int, gamma, eps):
        """Embedding lookup with the table sharded by vocabulary rows: every rank gathers the rows it owns (zeros for
        the others) straight into its published buffer, raises its flags, and the first RMSNorm of the step sums the
        ranks' contributions as it reads them (the same pull / in-switch reduction as the per-block exchanges).
        Returns (residual stream [T, H], its RMSNorm with `gamma`). The reference's vocab_parallel_embed masks and
        all-reduces (crates/skein_emit/src/op_wiring.rs:1819)."""
        T = ids.shape[0]
        if T > self.embed_rows or self.mode == "nccl":
            x = ops.embed(ids, table_shard, vocab_start)
            dist.all_reduce(x, group=self.group)
            return x, ops.rmsnorm(x, gamma, eps)
        ops.embed(ids, table_shard, vocab_start, out=self.embed_buf[:T])
        rc = _lib.lib().skein_publish_rows(None, 0, None, self._embed_push_flag, self.size, self.epochs[3:4].data_ptr(),
                                           self.done[3:4].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "publish embedding rows")
        _lib.count_launch()
        part = PeerPartials(self.embed_buf[:T], self._embed_src_ptrs, self.size, self.embed_flags, self.epochs[3:4],
                            self.wait_budget_ms, mc=self.heap.mc_addr(self.embed_off))
        return ops.reduce_residual_rmsnorm(None, part, gamma, eps)

    # ---- expert-parallel token dispatch (data-parallel attention) ---------------------------------------------------
    def dispatch_fits(self, per: int, k: int) -> bool:
        """True when ep_dispatch can carry a step of `per` rows per rank with `k` experts per row: the rows and their
        expert choices share one published buffer, and the expert-sorted pairs of all ranks one receive buffer."""
        pairs = self.size * per * k
        return per * self.hidden * 2 + per * k * 4 <= self.fused_rows * self.hidden * 2 and pairs <= 2048 and pairs <= self.fused_rows

    def ep_dispatch(self, per: int, k: int, E: int, e_first: int, e_count: int, fill):
        """Token dispatch of an expert-parallel MoE block whose ranks each own `per` of the step's tokens.

        `fill(normed_out [per, H] bf16, ids_out [per, k] int32)` must launch the kernels that write this rank's
        normalised rows and expert choices into the given views of its published buffer. The flags are then raised and
        one pull kernel (csrc/kernels/ep_dispatch.cu) derives the global expert-sorted layout from all ranks' choices and
        gathers, over NVLink, the rows routed to this rank's experts. Returns (ids_all [T, k], counts [E], offsets [E + 1],
        row_of [T * k], src_token [T * k], xs [T * k, H]) with T = ranks x per, the tuple the grouped expert GEMMs and the
        owner-aware combine take."""
        H, N = self.hidden, self.size
        rows_bytes = per * H * 2
        if not self.dispatch_fits(per, k):
            raise ValueError("dispatch does not fit the published buffers")
        b = self.cur
        self.cur ^= 1
        normed_view = self.bufs[b][:per]
        ids_view = self.heap.view(self.buf_off[b] + rows_bytes, (per, k), torch.int32)
        fill(normed_view, ids_view)
        L = _lib.lib()
        _lib.check(L.skein_publish_rows(None, 0, None, self._push_flag[b], N, self.epochs[b:b + 1].data_ptr(),
                                        self.done[b:b + 1].data_ptr(), _lib.stream_ptr()), "publish dispatch rows")
        T = N * per
        dev = self.device
        ids_all = torch.empty(T, k, dtype=torch.int32, device=dev)
        meta = torch.empty(2 * E + 1 + 2 * T * k, dtype=torch.int32, device=dev)
        counts, offsets = meta[:E], meta[E:2 * E + 1]
        row_of, src_token = meta[2 * E + 1:2 * E + 1 + T * k], meta[2 * E + 1 + T * k:]
        xs = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
        VP = C.c_void_p * N
        ids_ptrs = VP(*[self.heap.peer_ptr(p, self.buf_off[b] + rows_bytes) for p in range(N)])
        _lib.check(L.skein_ep_dispatch_pull(self._src_ptrs[b], ids_ptrs, N, per, k, E, e_first, e_count, H,
                                            self.flags[b].data_ptr(), self.epochs[b:b + 1].data_ptr(),
                                            ops.workspace().status.data_ptr(), self.wait_budget_ms, ids_all.data_ptr(),
                                            counts.data_ptr(), offsets.data_ptr(), row_of.data_ptr(), src_token.data_ptr(),
                                            xs.data_ptr(), _lib.stream_ptr()), "ep_dispatch_pull")
        _lib.count_launch(2)
        return ids_all, counts, offsets, row_of, src_token, xs

    def all_gather_aux(self, x: torch.Tensor) -> torch.Tensor:
        """All-gather of a small tensor (the step's sampled tokens) through the third published buffer, which does not
        take part in the alternation of the two per-block buffers."""
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if self.mode == "nccl" or nbytes % 16 != 0 or nbytes > self.embed_rows * self.hidden * 2:
            dist.all_gather_into_tensor(out, x, group=self.group)
            return out
        L = _lib.lib()
        _lib.check(L.skein_publish_rows(x.data_ptr(), nbytes, self.embed_buf.data_ptr(), self._embed_push_flag, self.size,
                                        self.epochs[3:4].data_ptr(), self.done[3:4].data_ptr(), _lib.stream_ptr()), "publish_rows")
        _lib.check(L.skein_pull_collective(self._PULL_ALL_GATHER, self._embed_src_ptrs, self.size, self.rank, nbytes, out.data_ptr(),
                                           self.embed_flags.data_ptr(), self.epochs[3:4].data_ptr(),
                                           ops.workspace().status.data_ptr(), self.wait_budget_ms, _lib.stream_ptr()),
                   "pull_collective")
        _lib.count_launch(2)
        return out

    # ---- sequence-parallel dataflow for prefill-sized chunks ------------------------------------------------
    # Between a row-parallel projection and the next column-parallel one the activations are sharded by token rows:
    #   GEMM publishes its partial [T, H]  ->  rank r reduces rows [r*per, (r+1)*per) over all ranks (peer loads or one
    #   in-switch reducing load), adds its slice of the residual stream, normalises it  (reduce-scatter + norm)
    #   ->  the normalised slices are published and pulled into every rank's local [T, H]  (all-gather)
    #   ->  the next q/k/v or gate/up GEMM reads local memory.
    # Each rank moves (N-1)/N of the message twice instead of pulling N-1 whole copies, normalises T/N rows instead of
    # T, and the residual stream stays sharded from layer to layer. No library collective is launched.
    def sp_ok(self, rows: int, partial_rows: int | None = None) -> bool:
        """True when a chunk of `rows` tokens takes the sequence-parallel path: more rows than the replicated
        (decode-style) exchange is meant for, and the partial results fit the published buffers."""
        pr = partial_rows if partial_rows is not None else rows
        return (self.mode in ("fused", "unfused") and self.size > 1 and rows > self.sp_min_rows and pr <= self.fused_rows
                and self.sp_slice(rows)[2] * self.size <= self.fused_rows)

    def sp_slice(self, rows: int):
        """(first row, row count, rows per rank) of this rank's slice of a [rows, H] activation."""
        per = (rows + self.size - 1) // self.size
        per = (per + 7) // 8 * 8
        r0 = min(self.rank * per, rows)
        return r0, min(per, rows - r0), per

    def reduce_scatter_norm(self, res_loc, part: "PeerPartials", gamma, eps, rows: int, row_idx=None, row_w=None):
        """This rank's slice of (residual + sum over ranks of the partials), and its RMSNorm. `part` is what
        linear_push returned for the whole chunk; `row_idx` / `row_w` ([rows, k]) select the MoE combine form, whose
        partial rows are addressed through row_idx. Returns (residual slice [n, H], normed slice [per, H]: rows beyond n
        are padding so that every rank's slice has the same size)."""
        r0, n, per = self.sp_slice(rows)
        H = self.hidden
        normed = torch.zeros(per, H, dtype=torch.bfloat16, device=self.device) if n < per else \
            torch.empty(per, H, dtype=torch.bfloat16, device=self.device)
        res_out = torch.empty(n, H, dtype=torch.bfloat16, device=self.device)
        if n == 0:
            return res_out, normed
        if row_idx is not None:
            sl = PeerPartials(part.local, part.ptrs, part.n_src, part.flags, part.epoch, part.wait_budget_ms, mc=part.mc)
            ri, rw = row_idx[r0:r0 + n].contiguous(), row_w[r0:r0 + n].contiguous()
        else:
            off = r0 * H * 2
            VP = C.c_void_p * self.size
            sl = PeerPartials(part.local[r0:r0 + n], VP(*[int(p) + off for p in part.ptrs]), part.n_src, part.flags,
                              part.epoch, part.wait_budget_ms, mc=(part.mc + off) if part.mc else 0)
            ri = rw = None
        ops.reduce_residual_rmsnorm(res_loc, sl, gamma, eps, ri, rw, residual_out=res_out,
                                    normed_out=normed[:n] if gamma is not None else None)
        return res_out, normed

    def gather_rows(self, x_loc: torch.Tensor, rows: int) -> torch.Tensor:
        """All-gather of equally sized row slices ([per, H] on every rank) into the full [rows, H] activation, in local
        memory (publish + one pull kernel): the operand of the next column-parallel GEMM."""
        return self.all_gather(x_loc)[:rows]

    # ---- all-gather / reduce-scatter / all-to-all ----------------------------------------------------
    _PULL_ALL_GATHER, _PULL_ALL_TO_ALL, _PULL_REDUCE_SCATTER = 0, 1, 2

    def _publish_and_pull(self, x: torch.Tensor, mode: int, chunk_bytes: int, out: torch.Tensor) -> torch.Tensor:
        """Copy `x` into this rank's peer-mapped buffer, raise the flags, and pull what `mode` says from every rank."""
        b = self.cur
        self.cur ^= 1
        L = _lib.lib()
        _lib.check(L.skein_publish_rows(x.data_ptr(), x.numel() * x.element_size(), self.bufs[b].data_ptr(), self._push_flag[b],
                                        self.size, self.epochs[b:b + 1].data_ptr(), self.done[b:b + 1].data_ptr(),
                                        _lib.stream_ptr()), "publish_rows")
        _lib.check(L.skein_pull_collective(mode, self._src_ptrs[b], self.size, self.rank, chunk_bytes, out.data_ptr(),
                                           self.flags[b].data_ptr(), self.epochs[b:b + 1].data_ptr(),
                                           ops.workspace().status.data_ptr(), self.wait_budget_ms, _lib.stream_ptr()),
                   "pull_collective")
        _lib.count_launch(2)
        return out

    def _pull_ok(self, x: torch.Tensor, chunk_bytes: int) -> bool:
        nbytes = x.numel() * x.element_size()
        return (self.mode in ("fused", "unfused") and x.is_cuda and 0 < nbytes <= self.bufs[0].numel() * 2 and nbytes % 16 == 0
                and chunk_bytes % 16 == 0)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[rows, ...] on every rank -> [N * rows, ...] in rank order (any dtype; a byte copy)."""
        x = x.contiguous()
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        nbytes = x.numel() * x.element_size()
        if not self._pull_ok(x, nbytes):
            dist.all_gather_into_tensor(out, x, group=self.group)
            return out
        return self._publish_and_pull(x, self._PULL_ALL_GATHER, nbytes, out)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """[N * rows, W] bf16 partials on every rank -> this rank's [rows, W] block of the sum over ranks
        (fp32 accumulation in rank order, so every run gives the same bits)."""
        x = x.contiguous()
        if x.shape[0] % self.size != 0:
            raise ValueError(f"reduce_scatter: {x.shape[0]} rows do not divide into {self.size} ranks")
        out = torch.empty((x.shape[0] // self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        chunk = x.numel() * x.element_size() // self.size
        if x.dtype != torch.bfloat16 or not self._pull_ok(x, chunk):
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        return self._publish_and_pull(x, self._PULL_REDUCE_SCATTER, chunk, out)

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """[N * rows, ...]: block d goes to rank d; returns [N * rows, ...] whose block s came from rank s."""
        x = x.contiguous()
        if x.shape[0] % self.size != 0:
            raise ValueError(f"all_to_all: {x.shape[0]} rows do not divide into {self.size} ranks")
        out = torch.empty_like(x)
        chunk = x.numel() * x.element_size() // self.size
        if not self._pull_ok(x, chunk):
            dist.all_to_all_single(out, x, group=self.group)
            return out
        return self._publish_and_pull(x, self._PULL_ALL_TO_ALL, chunk, out)

    # ---- vocabulary-parallel greedy sampling ----------------------------------------------------------
    def vocab_parallel_argmax(self, logits: torch.Tensor, v_local: int) -> torch.Tensor:
        B, V = logits.shape
        if B > self.max_batch:
            # large prefill batches: gather (value, index) pairs with the library instead
            val = torch.empty(B, dtype=torch.float32, device=logits.device)
            idx = ops.sample_argmax(logits, idx_offset=self.rank * v_local, out_val=val)
            vals = [torch.empty_like(val) for _ in range(self.size)]
            idxs = [torch.empty_like(idx) for _ in range(self.size)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx, group=self.group)
            v = torch.stack(vals)
            i = torch.stack(idxs)
            best = v.max(dim=0, keepdim=True).values
            cand = torch.where(v == best, i, torch.full_like(i, 2 ** 31 - 1))
            return cand.min(dim=0).values
        rc = _lib.lib().skein_argmax_push(logits.data_ptr(), logits.stride(0), B, V, self.rank * v_local,
                                          self._cand_val_ptrs, self._cand_idx_ptrs, self._cand_flag_ptrs, self.size,
                                          self.epochs[2:3].data_ptr(), self.done[2:3].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "argmax_push")
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
        ws = ops.workspace()
        rc = _lib.lib().skein_merge_candidates(self.cand_val.data_ptr(), self.cand_idx.data_ptr(), self.size, B, self.max_batch,
                                               self.cand_flags.data_ptr(), self.epochs[2:3].data_ptr(),
                                               ws.status.data_ptr(), self.wait_budget_ms, out.data_ptr(),
                                               _lib.stream_ptr())
        _lib.check(rc, "merge_candidates")
        _lib.count_launch(2)
        return out

    def close(self):
        ws = ops.workspace(self.device)
        ws.peer_state[:] = [st for st in ws.peer_state if st[0] is not self.epochs]
        self.heap.close()
