"""Pipeline parallelism: the decoder's blocks are split into stages (remainder spread over the first stages);
the residual stream [tokens, hidden] crosses each stage boundary with NCCL point-to-point, the last stage
samples, and the sampled tokens travel back (they are the next step's embedding input on stage 0 and the
scheduler's input on every rank).

Three levels:

* `PipelineStage.forward(inp)` has the contract of `Decoder.forward`, so the runner and the serving engine drive a
  pipeline like a single stage. A decode step is cut into `pp` micro-batches (row slices of the step's static
  buffers) that follow one another through the stages, so stage s works on micro-batch m while stage s + 1 works
  on m - 1. Point-to-point transfers are asynchronous (`isend` / `irecv` run on the communicator's own stream;
  the compute stream only waits, by event, for the transfer it needs next) and the compute between a receive
  and a send is captured as a per-stage, per-micro-batch CUDA graph.
* `pipelined_decode(...)` is the steady-state loop of a generation job: `pp` micro-batches stay in flight ACROSS
  steps (1F1B), positions advance on the device, and the token feedback from the last stage to the first
  travels on its own communicator, so that in steady state no stage idles.
* Within a stage, tensor parallelism uses that stage's own TPComm (fused collectives over the stage's ranks).

Counterpart of the reference's PP send/recv wiring (crates/skein_emit/src/op_wiring.rs:688,710;
crates/skein_runtime/src/distributed/rank_executor.rs:255-300), its grouped send/recv (crates/skein_runtime/
src/cuda/nccl.rs:362-445), token broadcast (gpu_rank.rs:601-624), the pp == 2 micro-batched decode
(gpu_rank.rs:1029-1290) and its continuous pipelined loops (gpu_rank.rs:1293,1566).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ParallelLayout
from ..models.decoder import BatchInputs, Decoder, SamplingInputs


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


def make_feedback_group(layout_dims, rank: int, backend=None):
    """A second communicator over every pipeline group, for the sampled tokens that travel from the last stage back to the
    others: on a communicator of its own the feedback never queues behind activation traffic. Every rank must call this
    with the same arguments (after make_groups). Returns this rank's group, or None without pipeline parallelism."""
    tp, pp, ep = layout_dims
    mine, seen = None, set()
    for r in range(tp * pp * ep):
        g = tuple(ParallelLayout(tp=tp, pp=pp, ep=ep, rank=r).pp_group())
        if g not in seen:
            seen.add(g)
            grp = dist.new_group(list(g), backend=backend) if pp > 1 else None
            if rank in g:
                mine = grp
    return mine


class _Flight:
    """One decode step of a group of sequences on its way through the pipeline (PipelineStage.launch / collect)."""
    __slots__ = ("tokens", "sends", "recv")

    def __init__(self):
        self.tokens, self.sends, self.recv = None, (), None


def _rows(inp: BatchInputs, lo: int, hi: int) -> BatchInputs:
    """Rows lo..hi of a decode step's inputs (views of the same static buffers)."""
    return BatchInputs(token_ids=inp.token_ids[lo:hi], positions=inp.positions[lo:hi], block_table=inp.block_table[lo:hi],
                       seq_lens=inp.seq_lens[lo:hi], ctx_hint=inp.ctx_hint)


def _sampling_rows(s: SamplingInputs | None, lo: int, hi: int):
    if s is None:
        return None
    return SamplingInputs(s.temperature[lo:hi], s.top_k[lo:hi], s.top_p[lo:hi], s.seeds[lo:hi], s.step[lo:hi])


class _StageGraph:
    """The captured compute of one stage for one micro-batch: static receive buffer in, residual (or tokens) out."""

    def __init__(self):
        self.graph = None
        self.hidden_in = None
        self.out = None          # residual stream [rows, H] (not last stage) or sampled tokens [rows] (last stage)
        self.logits = None
        self.seen = 0
        self.pending_send = None


class PipelineStage:
    def __init__(self, decoder: Decoder, layout: ParallelLayout, pp_ranks, pp_group, micro_batches: int | None = None,
                 use_graphs: bool | None = None):
        self.dec, self.layout, self.pp_ranks, self.pp_group = decoder, layout, pp_ranks, pp_group
        self.stage, self.n_stages = layout.pp_rank, layout.pp
        self.first, self.last = self.stage == 0, self.stage == layout.pp - 1
        self.prev = pp_ranks[self.stage - 1] if not self.first else None
        self.next = pp_ranks[self.stage + 1] if not self.last else None
        # attributes the runner / engine read from a decoder
        self.cfg, self.device, self.num_pages, self.page_size, self.max_pos, self.w = (
            decoder.cfg, decoder.device, decoder.num_pages, decoder.page_size, decoder.max_pos, decoder.w)
        self.comm = decoder.comm
        self.micro_batches = micro_batches if micro_batches is not None else self.n_stages
        fused = decoder.comm is None or decoder.comm.mode != "nccl"
        self.use_graphs = (self.device.type == "cuda" and fused) if use_graphs is None else (use_graphs and self.device.type == "cuda")
        self._graphs: dict = {}
        self.feedback_group = None      # communicator of the sampled tokens (launch / collect); None: the pp group itself
        self.stage_busy_events = []     # (start, end) CUDA events around this stage's compute, when `time_stages` is set
        self.time_stages = False

    # ---- one stage's compute for one (micro-)batch ------------------------------------------------------------------
    def _compute(self, inp: BatchInputs, hidden, sampling):
        residual, normed = self.dec.forward_hidden(inp, hidden)
        if not self.last:
            return residual.contiguous(), None
        logits = self.dec.logits(normed, inp)
        return self.dec.sample(logits, sampling), logits

    def _run_stage(self, inp: BatchInputs, sampling, key):
        """Receive (if not first), compute (captured graph when enabled), return (out, logits). The receive is waited for
        by the compute stream only; the host does not block."""
        rows, H = inp.token_ids.shape[0], self.cfg.hidden_size
        sg = self._graphs.get(key)
        if sg is None:
            sg = self._graphs[key] = _StageGraph()
            if not self.first:
                sg.hidden_in = torch.empty(rows, H, dtype=torch.bfloat16, device=self.device)
        if sg.pending_send is not None:       # last step's send of this slot must have left before its buffer is rewritten
            sg.pending_send.wait()
            sg.pending_send = None
        if not self.first:
            dist.irecv(sg.hidden_in, src=self.prev).wait()
        ev = None
        if self.time_stages and self.device.type == "cuda":
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        sg.seen += 1
        if self.use_graphs and not inp.is_prefill:
            if sg.graph is None and sg.seen >= 2:      # the first sight runs eagerly: it allocates workspaces and caches
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize()
                # thread-local capture mode: the process group's watchdog thread keeps querying the events of transfers
                # in flight, which the default (global) mode would count as a violation of this thread's capture
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    sg.out, sg.logits = self._compute(inp, sg.hidden_in, sampling)
                sg.graph = g
            if sg.graph is not None:
                sg.graph.replay()
            else:
                sg.out, sg.logits = self._compute(inp, sg.hidden_in, sampling)
        else:
            sg.out, sg.logits = self._compute(inp, sg.hidden_in, sampling)
        if ev is not None:
            ev[1].record()
            self.stage_busy_events.append(ev)
        if not self.last:
            sg.pending_send = dist.isend(sg.out, dst=self.next)
        return sg.out, sg.logits

    # ---- continuous serving: several groups of sequences in flight at once ---------------------------------------------
    def launch(self, inp: BatchInputs, sampling, key) -> _Flight:
        """Enqueue this stage's share of one decode step of a group of sequences and return without waiting for the
        step's tokens. Every stage calls launch and, later, collect for the same groups in the same order. The last stage
        sends the sampled tokens to every other stage on the feedback communicator as soon as they exist; the others post
        the receive now and wait for it in collect, so a stage keeps working on other groups while this one's tokens
        travel. `key` names the group (its stage compute is captured as a CUDA graph from the second sight on)."""
        out, _ = self._run_stage(inp, sampling, key)
        f = _Flight()
        grp = self.feedback_group if self.feedback_group is not None else self.pp_group
        if self.last:
            f.tokens = out.clone()      # the graph's output buffer is rewritten by the next replay
            f.sends = [dist.isend(f.tokens, dst=r, group=grp) for r in self.pp_ranks[:-1]]
        else:
            f.tokens = torch.empty(inp.token_ids.shape[0], dtype=torch.int32, device=self.device)
            f.recv = dist.irecv(f.tokens, src=self.pp_ranks[-1], group=grp)
        return f

    def collect(self, f: _Flight) -> torch.Tensor:
        """The sampled tokens of a launched step (a device tensor; on CUDA the current stream waits for their arrival)."""
        if f.recv is not None:
            f.recv.wait()
            f.recv = None
        for w in f.sends:
            w.wait()
        f.sends = ()
        return f.tokens

    def _n_out_rows(self, inp: BatchInputs) -> int:
        return inp.logit_rows.shape[0] if (inp.is_prefill and inp.logit_rows is not None) else inp.token_ids.shape[0]

    def forward(self, inp: BatchInputs, sampling=None):
        """One step through the whole pipeline. Every stage calls this with the same `inp`."""
        n_out = self._n_out_rows(inp)
        T = inp.token_ids.shape[0]
        M = self.micro_batches if (not inp.is_prefill and self.n_stages > 1 and T >= 2 * self.micro_batches
                                   and T % self.micro_batches == 0) else 1
        if M == 1:
            key = ("whole", inp.token_ids.data_ptr(), T, sampling is not None) if not inp.is_prefill else ("prefill", T)
            if inp.is_prefill:
                self._graphs.pop(key, None)          # prefill chunks differ in shape from call to call: nothing is kept
            out, logits = self._run_stage(inp, sampling, key)
            tokens = out if self.last else torch.empty(n_out, dtype=torch.int32, device=self.device)
            if inp.is_prefill:
                sg = self._graphs.pop(key, None)
                if sg is not None and sg.pending_send is not None:
                    sg.pending_send.wait()
        else:
            per = T // M
            tokens = torch.empty(T, dtype=torch.int32, device=self.device)
            logits = None
            for m in range(M):
                lo, hi = m * per, (m + 1) * per
                out, _ = self._run_stage(_rows(inp, lo, hi), _sampling_rows(sampling, lo, hi),
                                         ("micro", inp.token_ids.data_ptr(), T, m, sampling is not None))
                if self.last:
                    tokens[lo:hi].copy_(out)
        # token feedback to every stage of this pipeline group
        dist.broadcast(tokens, src=self.pp_ranks[-1], group=self.pp_group)
        return tokens, logits

    def forward_prefill_micro(self, items):
        """Prefill of several micro-chunks (whole sequences each) through the pipeline: `items` is a list of
        (BatchInputs, SamplingInputs or None), the same on every stage. A stage starts on chunk i + 1 as soon as its send of
        chunk i is under way, so the stages overlap as they do in decode; the first tokens of all chunks travel back in one
        broadcast at the end. Returns the tokens of all chunks, in order."""
        outs, keys = [], []
        for i, (inp, smp) in enumerate(items):
            key = ("prefill-micro", i)
            self._graphs.pop(key, None)          # shapes differ from call to call: nothing is kept
            keys.append(key)
            out, _ = self._run_stage(inp, smp, key)
            outs.append(out)
        for key in keys:
            sg = self._graphs.pop(key, None)
            if sg is not None and sg.pending_send is not None:
                sg.pending_send.wait()
        n_out = sum(self._n_out_rows(inp) for inp, _ in items)
        tokens = torch.cat(outs) if self.last else torch.empty(n_out, dtype=torch.int32, device=self.device)
        dist.broadcast(tokens, src=self.pp_ranks[-1], group=self.pp_group)
        return tokens

    def idle_fraction(self, wall_ms: float) -> float | None:
        """1 - (time this stage spent computing) / wall time, from the CUDA events recorded while `time_stages` was set."""
        if not self.stage_busy_events or wall_ms <= 0:
            return None
        torch.cuda.synchronize()
        busy = sum(s.elapsed_time(e) for s, e in self.stage_busy_events)
        return max(0.0, 1.0 - busy / wall_ms)


def pipelined_decode(stage: PipelineStage, micro_inputs: list, steps: int, advance, feedback_group=None,
                     resume: bool = False, more: bool = False, prev_tokens=None):
    """Steady-state pipelined greedy decode of len(micro_inputs) micro-batches for `steps` tokens each.

    micro_inputs[m] is the BatchInputs of micro-batch m (device tensors that `advance(inp, tokens)` updates in
    place for the next step; `tokens` is None on stages that do not embed). Stage s works on micro-batch m
    while stage s + 1 works on m - 1, so with at least `pp` micro-batches no stage idles after the fill phase.
    Point-to-point ops are enqueued in the same order on both sides of every boundary, which is what makes the
    send/recv pairs match; they run on the communicators' own streams and the compute stream waits, by event,
    only for the transfer it needs next. Each micro-batch's stage compute is a captured CUDA graph (from its second
    step on). Sampled tokens go from the last stage to the first on `feedback_group`, a separate communicator, so
    that the feedback never queues behind activation traffic.
    `more`: another call will continue this decode, so the last step's tokens are fed back as well; `resume`: this
    call continues one that ended with `more` (its first step receives that feedback; a single-stage "pipeline" takes
    the tokens from `prev_tokens`). Returns [steps][micro] token tensors on the last stage (None entries elsewhere).
    """
    M = len(micro_inputs)
    out = [[None] * M for _ in range(steps)]
    first_rank, last_rank = stage.pp_ranks[0], stage.pp_ranks[-1]
    pending = []   # isend handles of the token feedback, with their buffers
    tok_in = [torch.empty(inp.token_ids.shape[0], dtype=torch.int32, device=stage.device) for inp in micro_inputs]
    for t in range(steps):
        for m in range(M):
            inp = micro_inputs[m]
            if t > 0 or resume:
                # token feedback of the previous step, received only now: the pipeline never waits on it while
                # it still has other micro-batches to work on
                toks_prev = None
                if stage.first and stage.n_stages > 1:
                    dist.irecv(tok_in[m], src=last_rank, group=feedback_group).wait()
                    toks_prev = tok_in[m]
                elif stage.n_stages == 1:
                    toks_prev = out[t - 1][m] if t > 0 else prev_tokens[m]
                advance(inp, toks_prev)
            res, _ = stage._run_stage(inp, None, ("steady", m))
            if not stage.last:
                continue
            toks = res.clone()          # the graph's output buffer is rewritten by the next replay
            out[t][m] = toks
            if stage.n_stages > 1 and (t + 1 < steps or more):
                pending.append((dist.isend(toks, dst=first_rank, group=feedback_group), toks))
    for w, _ in pending:
        w.wait()
    for sg in stage._graphs.values():
        if sg.pending_send is not None:
            sg.pending_send.wait()
            sg.pending_send = None
    return out
