"""ModelRunner: static step buffers, CUDA-graph capture per batch bucket, prefill chunks.

The decode step of one batch bucket is captured once into a CUDA graph (every kernel of the step,
sampling included) and replayed. A step's host inputs travel in ONE pinned buffer and ONE
host-to-device copy (int32 words; B = bucket size):

    [ token ids B | positions B | seq_lens B | temperature B (fp32) | top_k B | top_p B (fp32)
      | seeds B (64-bit) | block table B x max_blocks ]

and its result in one device-to-host copy:

    [ sampled tokens B | device status word 2 | nanoseconds the step waited for peers (64-bit) ]

Two graphs exist per bucket: the greedy one (arg-max, vocabulary-parallel under TP) and the sampling one
(temperature / top-k / top-p per row, rows with temperature 0 stay greedy); a step uses the second only
when one of its requests asked for sampling.

Capture classes are padded batch sizes (the reference keys its full-step captures per micro-batch:
crates/skein_runtime/src/distributed/gpu_rank.rs:466-555; its dispatcher for capture classes is a
stub: crates/skein_runtime/src/dispatch/mod.rs:48-58). Padding rows carry position -1 / seq_len 0
and are skipped by the kernels.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..models.decoder import BatchInputs, Decoder, SamplingInputs

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
N_RESULT_EXTRA = 4    # status code, detail, peer-wait nanoseconds (2 words)


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    raise ValueError(f"batch {n} exceeds the largest capture class {BUCKETS[-1]}")


def split_by_tokens(lengths, m: int):
    """Cuts the sequence indices 0 .. len(lengths) - 1 into at most `m` contiguous, non-empty groups of about equal token
    counts (a group is closed as soon as the running total reaches its share, or when the sequences left are needed to
    fill the remaining groups)."""
    total = sum(lengths)
    groups, cur, acc = [], [], 0
    for i, n in enumerate(lengths):
        cur.append(i)
        acc += n
        left = len(lengths) - i - 1
        if len(groups) < m - 1 and (acc >= total * (len(groups) + 1) / m or left <= m - 1 - len(groups)) and left >= 1:
            groups.append(cur)
            cur = []
    if cur:
        groups.append(cur)
    return groups


class _Bucket:
    def __init__(self, B: int, max_blocks: int, device):
        self.B, self.max_blocks = B, max_blocks
        n_in = 8 * B + B * max_blocks
        pin = device.type == "cuda"
        self.host_in = torch.zeros(n_in, dtype=torch.int32, pin_memory=pin)
        self.dev_in = torch.zeros(n_in, dtype=torch.int32, device=device)
        self.host_out = torch.zeros(B + N_RESULT_EXTRA, dtype=torch.int32, pin_memory=pin)
        self.dev_out = torch.zeros(B + N_RESULT_EXTRA, dtype=torch.int32, device=device)
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.graphs = {}           # (feedback, sampling) -> captured step
        self.np_views = None
        self.host_in[B:2 * B] = -1
        self.host_in[5 * B:6 * B].view(torch.float32).fill_(1.0)     # top_p

    def views(self, buf):
        """(token ids, positions, seq_lens, block table) views of a staging buffer."""
        B, mb = self.B, self.max_blocks
        return buf[:B], buf[B:2 * B], buf[2 * B:3 * B], buf[8 * B:].view(B, mb)

    def sampling_views(self, buf):
        """(temperature fp32, top_k int32, top_p fp32, seeds int64) views of a staging buffer."""
        B = self.B
        return (buf[3 * B:4 * B].view(torch.float32), buf[4 * B:5 * B], buf[5 * B:6 * B].view(torch.float32),
                buf[6 * B:8 * B].view(torch.int64))

    @property
    def h2d_bytes(self):
        return self.host_in.numel() * 4

    @property
    def d2h_bytes(self):
        return self.host_out.numel() * 4

    # kept for callers that hold one graph per kind
    @property
    def graph(self):
        return self.graphs.get((False, False))

    @property
    def graph_loop(self):
        return self.graphs.get((True, False))


class ModelRunner:
    def __init__(self, decoder: Decoder, max_blocks_per_seq: int, use_graphs: bool = True, ctx_hint: int = 1024):
        self.dec = decoder
        self.device = decoder.device
        self.max_blocks = max_blocks_per_seq
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self.ctx_hint = ctx_hint
        self.buckets: dict[int, _Bucket] = {}
        self.graph_captures = 0
        self.graph_replays = 0
        self.last_wait_ns = 0      # running total of the device-side peer-wait counter, as of the last synchronised step

    # ---- decode -----------------------------------------------------------------------------------
    def bucket(self, n: int, slot: int | None = None) -> _Bucket:
        """The staging buffers (and captured graphs) of batches of up to bucket_for(n) rows. `slot` asks for a set of its
        own: steps of different groups of sequences that are on the device at the same time must not share buffers."""
        B = bucket_for(n)
        key = B if slot is None else (B, slot)
        bk = self.buckets.get(key)
        if bk is None:
            bk = self.buckets[key] = _Bucket(B, self.max_blocks, self.device)
            bk.slot = slot
        return bk

    def _decode_body(self, bk: _Bucket, feedback: bool, sampling: bool = False):
        tok, pos, lens, bt = bk.views(bk.dev_in)
        inp = BatchInputs(token_ids=tok, positions=pos, block_table=bt, seq_lens=lens, ctx_hint=self.ctx_hint)
        smp = None
        if sampling:
            t, k, p, seeds = bk.sampling_views(bk.dev_in)
            smp = SamplingInputs(t, k, p, seeds, pos)      # the random stream is indexed by the token's position
        sampled, _ = self.dec.forward(inp, sampling=smp)
        bk.dev_out[:bk.B].copy_(sampled)
        if self.device.type == "cuda":
            bk.dev_out[bk.B:].copy_(ops.workspace().status)
        if feedback:
            ops.advance_decode_state(sampled, tok, pos, lens, bk.step_counter)

    def _ensure_graph(self, bk: _Bucket, feedback: bool, sampling: bool = False):
        key = (feedback, sampling)
        g = bk.graphs.get(key)
        if g is not None:
            return g
        # eager warm-up allocates workspaces and descriptor caches outside the capture
        saved = bk.dev_in.clone()
        self._decode_body(bk, False, sampling)
        torch.cuda.synchronize()
        bk.dev_in.copy_(saved)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._decode_body(bk, feedback, sampling)
        torch.cuda.synchronize()
        bk.dev_in.copy_(saved)  # the capture itself does not run, but keep the inputs pristine
        self.graph_captures += 1
        bk.graphs[key] = g
        return g

    def capture_buckets(self, max_batch: int, sampling: bool = False) -> int:
        """Captures the decode step of every batch bucket up to `max_batch` ahead of time (a server does this while it
        starts, so that no request pays for a capture: a first-seen bucket otherwise costs an eager warm-up step plus the
        capture in the middle of serving). Padding rows only: nothing is read from or written to the cache.
        Returns the number of graphs captured."""
        if not self.use_graphs:
            return 0
        n = 0
        inner = getattr(self.dec, "dec", self.dec)
        dp = inner.dp_ways() if hasattr(inner, "dp_ways") else 1
        for b in BUCKETS:
            if dp > 1 and not inner.dp_rows_ok(b, getattr(inner, "device", None)):
                if b >= max_batch:      # data-parallel attention: only steps of equal slices per rank ever run
                    break
                continue
            bk = self.bucket(b)
            if (False, sampling) not in bk.graphs:
                self.load_decode_inputs(bk, [], [], [], [])
                bk.dev_in.copy_(bk.host_in)
                self._ensure_graph(bk, False, sampling)
                n += 1
            if b >= max_batch:
                break
        return n

    def load_decode_inputs(self, bk: _Bucket, tokens, positions, seq_lens, block_tables, sampling=None):
        """Fill the pinned staging buffer from host lists (rows beyond len(tokens) are padding). `sampling` is a
        list of (temperature, top_k, top_p, seed) per row, or None for an all-greedy step."""
        n = len(tokens)
        if bk.np_views is None:   # numpy views share the pinned buffer: no tensor objects per row on the hot path
            bk.np_views = tuple(v.numpy() for v in bk.views(bk.host_in)) + tuple(v.numpy() for v in bk.sampling_views(bk.host_in))
        t, p, l, bt, st, sk, sp, ss = bk.np_views
        t[:n] = tokens
        p[:n] = positions
        l[:n] = seq_lens
        t[n:] = 0
        p[n:] = -1
        l[n:] = 0
        for i, row in enumerate(block_tables):
            bt[i, :len(row)] = row
        if sampling is not None:
            st[:n] = [s[0] for s in sampling]
            sk[:n] = [s[1] for s in sampling]
            sp[:n] = [s[2] for s in sampling]
            ss[:n] = [s[3] for s in sampling]
            st[n:] = 0.0
        else:
            st[:] = 0.0

    def stage_decode_inputs(self, bk: _Bucket, batcher, ids, sampling=None):
        """load_decode_inputs for the serving engine: the C++ batcher writes tokens, positions, lengths and block tables of
        the listed requests straight into the pinned staging buffer (one call, no per-row Python objects)."""
        t, p, l, bt = bk.views(bk.host_in)
        batcher.fill_decode_inputs(ids, t.data_ptr(), p.data_ptr(), l.data_ptr(), bt.data_ptr(), bk.max_blocks, bk.B)
        if bk.np_views is None:
            bk.np_views = tuple(v.numpy() for v in bk.views(bk.host_in)) + tuple(v.numpy() for v in bk.sampling_views(bk.host_in))
        st, sk, sp, ss = bk.np_views[4:]
        n = len(ids)
        if sampling is not None:
            st[:n] = [s[0] for s in sampling]
            sk[:n] = [s[1] for s in sampling]
            sp[:n] = [s[2] for s in sampling]
            ss[:n] = [s[3] for s in sampling]
            st[n:] = 0.0
            bk.sampling_dirty = True
        elif getattr(bk, "sampling_dirty", True):
            st[:] = 0.0
            bk.sampling_dirty = False

    def decode_step(self, bk: _Bucket, sync: bool = True, sampling: bool = False):
        """H2D of the staged inputs, one step, D2H of the result. Returns the host result view."""
        bk.dev_in.copy_(bk.host_in, non_blocking=True)
        if self.use_graphs:
            self._ensure_graph(bk, False, sampling).replay()
            self.graph_replays += 1
        else:
            self._decode_body(bk, False, sampling)
        bk.host_out.copy_(bk.dev_out, non_blocking=True)
        if sync and self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
            if int(bk.host_out[bk.B]) != 0:
                ops.workspace().check_status()
            lo, hi = int(bk.host_out[bk.B + 2]), int(bk.host_out[bk.B + 3])      # a 64-bit total in two words
            self.last_wait_ns = ((hi & 0xFFFFFFFF) << 32) | (lo & 0xFFFFFFFF)
        return bk.host_out[:bk.B]

    def decode_launch(self, bk: _Bucket, sampling: bool = False) -> None:
        """decode_step without the wait: H2D of the staged inputs, the step, D2H of the result, all enqueued."""
        self.decode_step(bk, sync=False, sampling=sampling)

    def decode_wait(self, bk: _Bucket):
        """Waits for a step enqueued by decode_launch; returns the host result view."""
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
            if int(bk.host_out[bk.B]) != 0:
                ops.workspace().check_status()
            lo, hi = int(bk.host_out[bk.B + 2]), int(bk.host_out[bk.B + 3])      # a 64-bit total in two words
            self.last_wait_ns = ((hi & 0xFFFFFFFF) << 32) | (lo & 0xFFFFFFFF)
        return bk.host_out[:bk.B]

    # ---- pipeline parallelism with several groups of sequences in flight -------------------------------------------------
    def _finish_flight(self, bk: _Bucket, toks) -> None:
        """Device-to-host copy of a flight's tokens and of the device status, followed by the event the host waits for."""
        bk.dev_out[:bk.B].copy_(toks)
        if self.device.type == "cuda":
            bk.dev_out[bk.B:].copy_(ops.workspace().status)
        bk.host_out.copy_(bk.dev_out, non_blocking=True)
        if self.device.type == "cuda":
            if getattr(bk, "done", None) is None:
                bk.done = torch.cuda.Event()
            bk.done.record()

    def pp_launch(self, bk: _Bucket, sampling: bool = False) -> None:
        """Host-to-device copy of the staged inputs and this stage's share of the step, enqueued without waiting for the
        step's tokens (PipelineStage.launch). The last stage, which has the tokens as soon as its compute ends, enqueues
        their copy to the host right behind it; the other stages do that in pp_collect, on a side stream, so that the
        copy does not wait for the steps of other groups that were enqueued in between."""
        bk.dev_in.copy_(bk.host_in, non_blocking=True)
        tok, pos, lens, bt = bk.views(bk.dev_in)
        inp = BatchInputs(token_ids=tok, positions=pos, block_table=bt, seq_lens=lens, ctx_hint=self.ctx_hint)
        smp = None
        if sampling:
            t, k, p, seeds = bk.sampling_views(bk.dev_in)
            smp = SamplingInputs(t, k, p, seeds, pos)
        bk.flight = self.dec.launch(inp, smp, ("group", bk.slot, bk.B, sampling))
        if self.dec.last:
            self._finish_flight(bk, bk.flight.tokens)

    def pp_collect(self, bk: _Bucket):
        """Waits for the tokens of a step enqueued by pp_launch; returns the host result view."""
        if self.dec.last:
            self.dec.collect(bk.flight)         # the sends of the tokens left long ago; this only retires their handles
        else:
            if self.device.type == "cuda":
                if getattr(self, "_fb_stream", None) is None:
                    self._fb_stream = torch.cuda.Stream(device=self.device)
                with torch.cuda.stream(self._fb_stream):
                    self._finish_flight(bk, self.dec.collect(bk.flight))
            else:
                self._finish_flight(bk, self.dec.collect(bk.flight))
        bk.flight = None
        if self.device.type == "cuda":
            bk.done.synchronize()
            if int(bk.host_out[bk.B]) != 0:
                ops.workspace().check_status()
        return bk.host_out[:bk.B]

    def decode_loop_step(self, bk: _Bucket):
        """One step with device-side token feedback (no host traffic). Inputs must already be on the device."""
        if self.use_graphs:
            self._ensure_graph(bk, True).replay()
            self.graph_replays += 1
        else:
            self._decode_body(bk, True)

    # ---- prefill ----------------------------------------------------------------------------------
    def _prefill_inputs(self, seqs, sampling):
        """BatchInputs (and SamplingInputs) of one eager chunk holding every new token of every listed sequence."""
        dev = self.device
        toks, pos, sot, qs, ql, kl, rows = [], [], [], [], [], [], []
        S = len(seqs)
        bt = torch.zeros(S, self.max_blocks, dtype=torch.int32)
        for s, (ids, table, cached) in enumerate(seqs):
            qs.append(len(toks)); ql.append(len(ids)); kl.append(cached + len(ids))
            toks.extend(ids); pos.extend(range(cached, cached + len(ids))); sot.extend([s] * len(ids))
            rows.append(len(toks) - 1)
            bt[s, :len(table)] = torch.as_tensor(table, dtype=torch.int32)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        inp = BatchInputs(token_ids=i32(toks), positions=i32(pos), block_table=bt.to(dev), seq_lens=i32(kl),
                          is_prefill=True, seq_of_token=i32(sot), q_start=i32(qs), q_len=i32(ql), max_q_len=max(ql),
                          logit_rows=torch.tensor(rows, dtype=torch.int64, device=dev))
        smp = None
        if sampling is not None and any(s[0] > 0 for s in sampling):
            smp = SamplingInputs(torch.tensor([s[0] for s in sampling], dtype=torch.float32, device=dev),
                                 i32([s[1] for s in sampling]),
                                 torch.tensor([s[2] for s in sampling], dtype=torch.float32, device=dev),
                                 torch.tensor([s[3] for s in sampling], dtype=torch.int64, device=dev),
                                 i32([n - 1 for n in kl]))
        return inp, smp

    def prefill(self, seqs, want_logits: bool = False, sampling=None):
        """seqs: list of (new_token_ids, block_table_row, cached_len). Runs one eager chunk holding every new
        token of every listed sequence. Returns the next token of every sequence (host list) [and logits]; greedy
        unless `sampling` gives (temperature, top_k, top_p, seed) per sequence. Behind a pipeline of several stages the
        chunk is cut, at sequence boundaries, into one micro-chunk per stage so that the stages overlap."""
        n_stages = getattr(self.dec, "n_stages", 1)
        if (n_stages > 1 and len(seqs) >= 2 and not want_logits and hasattr(self.dec, "forward_prefill_micro")
                and os.environ.get("SKEIN_PP_PREFILL_MICRO", "1") != "0"):
            total = sum(len(s[0]) for s in seqs)
            # at least one micro-chunk per stage; up to two per stage while a micro-chunk keeps 2048 tokens (fill and drain
            # of the pipeline cost one micro-chunk's time per call, and the projections want a few thousand tokens)
            M = min(len(seqs), max(n_stages, min(2 * n_stages, total // 2048)))
            groups = split_by_tokens([len(s[0]) for s in seqs], M)
            items = [self._prefill_inputs([seqs[i] for i in g], None if sampling is None else [sampling[i] for i in g])
                     for g in groups if g]
            return self.dec.forward_prefill_micro(items).cpu().tolist()
        inp, smp = self._prefill_inputs(seqs, sampling)
        tok, lg = self.dec.forward(inp, sampling=smp)
        out = tok.cpu().tolist()
        return (out, lg) if want_logits else out
