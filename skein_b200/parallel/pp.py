"""Pipeline parallelism: the decoder's blocks are split into stages (remainder spread over the first stages);
the residual stream [tokens, hidden] crosses each stage boundary with NCCL point-to-point on the compute
stream (enqueued asynchronously, no host synchronisation), the last stage samples, and the sampled tokens
travel back to every stage of the pipeline group (they are the next step's embedding input on stage 0 and
the scheduler's input on every rank).

`PipelineStage` has the same `forward(inp) -> (tokens, logits)` contract as `Decoder`, so the runner and the
engine drive a pipeline exactly like a single stage. `pipelined_decode` additionally keeps `pp` micro-batches
in flight so that all stages work at the same time (steady-state 1F1B for any pp, not only pp == 2).

Within a stage, tensor parallelism uses that stage's own TPComm (fused collectives over the stage's ranks).

Counterpart of the reference's PP send/recv wiring (crates/skein_emit/src/op_wiring.rs:688,710;
crates/skein_runtime/src/distributed/rank_executor.rs:255-300), token broadcast (gpu_rank.rs:601-624) and the
pp == 2 micro-batched decode (gpu_rank.rs:1029-1290).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ParallelLayout
from ..models.decoder import BatchInputs, Decoder


def make_groups(layout_dims, rank: int, backend=None):
    """Create the TP group of every (stage, ep) and the PP group of every (ep, tp) position. Every rank must
    call this with the same arguments. Returns (my tp group, my pp group ranks, my pp group)."""
    tp, pp, ep = layout_dims
    me = ParallelLayout(tp=tp, pp=pp, ep=ep, rank=rank)
    my_tp = my_pp = None
    seen = set()
    for r in range(tp * pp * ep):
        g = tuple(ParallelLayout(tp=tp, pp=pp, ep=ep, rank=r).tp_group())
        if g not in seen:
            seen.add(g)
            grp = dist.new_group(list(g), backend=backend) if tp > 1 else None
            if rank in g:
                my_tp = grp
    seen = set()
    for r in range(tp * pp * ep):
        g = tuple(ParallelLayout(tp=tp, pp=pp, ep=ep, rank=r).pp_group())
        if g not in seen:
            seen.add(g)
            grp = dist.new_group(list(g), backend=backend) if pp > 1 else None
            if rank in g:
                my_pp = grp
    return my_tp, me.pp_group(), my_pp


class PipelineStage:
    def __init__(self, decoder: Decoder, layout: ParallelLayout, pp_ranks, pp_group):
        self.dec, self.layout, self.pp_ranks, self.pp_group = decoder, layout, pp_ranks, pp_group
        self.stage, self.n_stages = layout.pp_rank, layout.pp
        self.first, self.last = self.stage == 0, self.stage == layout.pp - 1
        self.prev = pp_ranks[self.stage - 1] if not self.first else None
        self.next = pp_ranks[self.stage + 1] if not self.last else None
        # attributes the runner / engine read from a decoder
        self.cfg, self.device, self.num_pages, self.page_size, self.max_pos, self.w = (
            decoder.cfg, decoder.device, decoder.num_pages, decoder.page_size, decoder.max_pos, decoder.w)
        self.comm = decoder.comm

    def _n_out_rows(self, inp: BatchInputs) -> int:
        return inp.logit_rows.shape[0] if (inp.is_prefill and inp.logit_rows is not None) else inp.token_ids.shape[0]

    def forward(self, inp: BatchInputs, sampling=None):
        """One step through the whole pipeline. Every stage calls this with the same `inp`."""
        T, H = inp.token_ids.shape[0], self.cfg.hidden_size
        hidden = None
        if not self.first:
            hidden = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
            dist.recv(hidden, src=self.prev)
        residual, normed = self.dec.forward_hidden(inp, hidden)
        n_out = self._n_out_rows(inp)
        if not self.last:
            dist.send(residual.contiguous(), dst=self.next)
            tokens = torch.empty(n_out, dtype=torch.int32, device=self.device)
            logits = None
        else:
            logits = self.dec.logits(normed, inp)
            tokens = self.dec.sample(logits, sampling)
        # token feedback to every stage of this pipeline group
        dist.broadcast(tokens, src=self.pp_ranks[-1], group=self.pp_group)
        return tokens, logits


def pipelined_decode(stage: PipelineStage, micro_inputs: list, steps: int, advance, feedback_group=None):
    """Steady-state pipelined greedy decode of len(micro_inputs) micro-batches for `steps` tokens each.

    micro_inputs[m] is the BatchInputs of micro-batch m (device tensors that `advance(inp, tokens)` updates in
    place for the next step; `tokens` is None on stages that do not embed). Stage s works on micro-batch m
    while stage s + 1 works on m - 1, so with at least `pp` micro-batches no stage idles after the fill phase.
    Point-to-point ops are enqueued in the same order on both sides of every boundary, which is what makes the
    send/recv pairs match. Sampled tokens go from the last stage to the first on `feedback_group`, a separate
    communicator, so that the feedback never queues behind activation traffic.
    Returns [steps][micro] token tensors on the last stage (None entries elsewhere).
    """
    M = len(micro_inputs)
    out = [[None] * M for _ in range(steps)]
    H = stage.cfg.hidden_size
    from .. import ops
    first_rank, last_rank = stage.pp_ranks[0], stage.pp_ranks[-1]
    pending = []   # keeps isend handles and their buffers alive
    for t in range(steps):
        for m in range(M):
            inp = micro_inputs[m]
            if t > 0:
                # token feedback of the previous step, received only now: the pipeline never waits on it while
                # it still has other micro-batches to work on
                toks_prev = None
                if stage.first and stage.n_stages > 1:
                    toks_prev = torch.empty(inp.token_ids.shape[0], dtype=torch.int32, device=stage.device)
                    dist.recv(toks_prev, src=last_rank, group=feedback_group)
                elif stage.n_stages == 1:
                    toks_prev = out[t - 1][m]
                advance(inp, toks_prev)
            hidden = None
            if not stage.first:
                hidden = torch.empty(inp.token_ids.shape[0], H, dtype=torch.bfloat16, device=stage.device)
                dist.recv(hidden, src=stage.prev)
            residual, normed = stage.dec.forward_hidden(inp, hidden)
            if not stage.last:
                dist.send(residual.contiguous(), dst=stage.next)
                continue
            lg = stage.dec.logits(normed, inp)
            toks = stage.dec.comm.vocab_parallel_argmax(lg, stage.dec.sh["V_local"]) if (stage.dec.comm and stage.dec.comm.size > 1) else ops.sample_argmax(lg)
            out[t][m] = toks
            if stage.n_stages > 1 and t + 1 < steps:
                # asynchronous on the feedback communicator: the compute stream goes on with the next micro-batch
                pending.append((dist.isend(toks, dst=first_rank, group=feedback_group), toks))
    for w, _ in pending:
        w.wait()
    return out
