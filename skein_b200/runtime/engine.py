"""Serving engine: continuous batching over paged KV, one scheduler iteration per `step()`.

    submit()  -> admission decision from the C++ batcher (admit / delay / reject); admitted requests get
                 their KV pages (with radix prefix reuse) at once
    step()    -> promote delayed requests, ask the batcher for the step's work, run the prefill chunks
                 (eager) and the decode batch (CUDA-graph replay of the batch-size bucket), hand the
                 sampled tokens back to the batcher, retire finished requests, record metrics

While sequences are decoding, a step carries at most `interleave_prefill_tokens` of waiting prompt, so
a long prompt is spread over several steps instead of stalling every decoding sequence for its whole
prefill. Requests may ask for temperature / top-k / top-p sampling with their own seed; the step then
runs the sampling variant of the captured graph.

Under tensor parallelism every rank runs the same engine on the same request stream (rank 0
announces submissions and the clock, see runtime/driver.py), so all ranks take identical scheduling
decisions and meet in the fused collectives.

A failing step does not take the server down: the batch is retired, its streams are closed with an
error, queued requests stay queued (the reference wraps each step in catch_unwind for the same
purpose: crates/skein_runtime/src/server/forward.rs:237-420).

Counterpart of the reference's driver loops (crates/skein_runtime/src/server/forward.rs:237-420 single
process; distributed/batch_driver.rs:77-514 single-GPU continuous batching; distributed/gpu_rank.rs
724-877 multi-GPU generation).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

from .. import core
from ..utils import otlp
from .runner import ModelRunner


@dataclass
class EngineConfig:
    max_batch: int = 64
    chunk_tokens: int = 0              # 0 = whole prompt in one chunk (bounded by max_prefill_tokens)
    max_prefill_tokens: int = 8192
    interleave_prefill_tokens: int = 2048   # prompt tokens per step while other sequences decode (0: no limit)
    ttft_ms: float = 500.0
    tpot_ms: float = 50.0
    decode_us_at_b1: float = 8000.0
    batch_exponent: float = 0.7
    prefill_per_token_us: float = 25.0
    prefix_cache: bool = True
    eos_token: int = -1
    use_graphs: bool = True
    warm_graphs: bool = False          # capture the decode graph of every batch bucket up to max_batch at start-up
    prelaunch: bool = True             # enqueue the next decode step as soon as this one's tokens are accepted (see _prelaunch)
    pp_continuous: bool = False        # pipeline parallelism: keep one group of sequences per stage in flight across steps
                                       # instead of draining the pipeline at the end of every step (see _run_continuous)
    drift_baseline: tuple = ()         # prompt lengths the plan was extracted for (workload drift monitor)
    drift_threshold_kl: float = 0.05


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 = greedy. top_k 0 = the sampler's maximum (64 candidates). One random stream per seed."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def row(self):
        return (float(self.temperature), int(self.top_k), float(self.top_p), int(self.seed))


GREEDY = SamplingParams()


@dataclass
class TokenEvent:
    request_id: int
    token: int
    is_final: bool
    error: str | None = None


class Engine:
    def __init__(self, decoder, cfg: EngineConfig | None = None, metrics=None, clock=None):
        self.dec = decoder
        self.cfg = cfg or EngineConfig()
        c = self.cfg
        if decoder.num_pages <= 0:
            raise ValueError("the decoder was built without a KV page pool")
        self.kv = core.KvBlockManager(decoder.num_pages, decoder.page_size, c.prefix_cache)
        # Expert parallelism with data-parallel attention: each decoding sequence belongs to one rank's slice of the
        # step's rows for its whole life (only that rank's cache receives its new tokens). Every rank's engine takes
        # the same decisions, so the assignment needs no communication. A slice is never larger than
        # ceil(max_batch / ranks) rows (a sequence joins the least loaded slice), so bounding max_batch bounds the slices
        # to what the dispatch kernels carry.
        inner = getattr(decoder, "dec", decoder)
        self._dp = inner.dp_ways() if hasattr(inner, "dp_ways") else 1
        max_batch = c.max_batch
        if self._dp > 1:
            inner.dp_strict = True
            dev = getattr(inner, "device", None)
            if dev is not None and getattr(dev, "type", "cpu") == "cuda":
                from .runner import BUCKETS
                limit = inner.dp_rows_limit(dev)
                if limit == 0:
                    raise ValueError("data-parallel attention is on, but no decode step fits its dispatch buffers")
                max_batch = min(max_batch, limit * self._dp, BUCKETS[-1])
        self.max_batch = max_batch
        self.batcher = core.ContinuousBatcher(
            max_batch=max_batch, chunk_tokens=c.chunk_tokens, ttft_ms=c.ttft_ms, tpot_ms=c.tpot_ms,
            decode_us_at_b1=c.decode_us_at_b1, batch_exponent=c.batch_exponent,
            prefill_per_token_us=c.prefill_per_token_us, kv=self.kv, max_prefill_tokens=c.max_prefill_tokens,
            interleave_prefill_tokens=c.interleave_prefill_tokens)
        self.cfg_vocab = int(decoder.cfg.vocab_size)
        self.max_blocks = max(1, (decoder.max_pos + decoder.page_size - 1) // decoder.page_size)
        self.runner = ModelRunner(decoder, self.max_blocks, use_graphs=c.use_graphs)
        if c.warm_graphs:
            # data-parallel attention: a step has at least 4 rows per rank, whatever the number of sequences
            self.runner.capture_buckets(max(max_batch, 4 * self._dp) if self._dp > 1 else max_batch)
        self.metrics = metrics or core.MetricsRegistry()
        self.clock = clock or (lambda: int(time.monotonic() * 1000))
        self._next_id = 1
        self._step = 0
        self._graph_seen = (0, 0)   # runner.graph_captures / graph_replays already added to the metrics
        self._sampling = {}      # request id -> SamplingParams (only requests that sample)
        self._dp_of: dict[int, int] = {}
        self._dp_load = [0] * self._dp
        self._wait_ns_seen = 0
        # the next decode step, already enqueued on the device: (bucket, request ids as planned, rows as laid out, sampling rows)
        self._pre = None
        self._prelaunch_ok = c.prelaunch and getattr(decoder, "n_stages", 1) == 1
        # Pipeline parallelism, continuous form: the decoding sequences are split into one group per stage; a step launches
        # every group that is not on the device and accepts the tokens of the oldest launch, so that in the steady state
        # every stage always has a group to work on.
        self._groups = getattr(decoder, "n_stages", 1) if (c.pp_continuous and hasattr(decoder, "launch")) else 1
        self._grp_of: dict[int, int] = {}
        self._grp_load = [0] * self._groups
        self._flights: list = []       # (group, bucket, request ids), oldest first
        self.metrics.set_gauge("skein_pipeline_groups_in_flight_max", float(max(0, self._groups - 1)))
        # optional trace export (SKEIN_OTLP_ENDPOINT): one span per engine step and one per finished request
        self._otlp = otlp.exporter(getattr(getattr(inner, "layout", None), "rank", 0))
        self._req_t0: dict[int, tuple] = {}      # request id -> (trace id, wall-clock ns at submission), while exporting
        self.failure_injector = None   # tests: callable(step_index) that may raise inside the step
        self.last_step_failed = False
        self.step_started_at = None    # monotonic time at which the step in progress began (the rank's heartbeat reads it)
        # workload drift: prompt lengths seen so far against the lengths the plan was made for
        self._drift = core.DriftMonitor(list(c.drift_baseline), c.drift_threshold_kl) if c.drift_baseline else None
        self._seen_lengths: list[int] = []

    # ---- admission ----------------------------------------------------------------------------------------
    def submit(self, prompt_ids, max_new_tokens: int = 32, now_ms: int | None = None, request_id: int | None = None,
               sampling: SamplingParams | None = None):
        """Returns (request_id, decision) with decision.kind in {"admit", "delay", "reject"}."""
        rid = request_id if request_id is not None else self._next_id
        self._next_id = max(self._next_id, rid) + 1
        now = self.clock() if now_ms is None else now_ms
        prompt = [int(t) for t in prompt_ids]
        if not prompt or min(prompt) < 0 or max(prompt) >= self.cfg_vocab:
            # an id outside the table reads as a zero row on the device and fails the whole step on the CPU path: refuse it here
            raise ValueError(f"prompt must be a non-empty list of token ids in [0, {self.cfg_vocab})")
        if len(prompt) + max_new_tokens > self.dec.max_pos:
            self.metrics.record_request(rid, "rejected", 0.0, 0.0, 0, 0)
            raise ValueError(f"prompt + max_new_tokens exceeds the position limit {self.dec.max_pos}")
        d = self.batcher.submit(rid, prompt, max_new_tokens, now)
        if d.kind == "reject":
            self.metrics.record_request(rid, "rejected", 0.0, 0.0, 0, 0)
        else:
            if sampling is not None and not sampling.greedy:
                self._sampling[rid] = sampling
            self._observe_length(len(prompt))
            if self._otlp is not None:
                self._req_t0[rid] = (self._otlp.new_trace_id(), time.time_ns(), len(prompt))
        return rid, d

    def _observe_length(self, n: int) -> None:
        if self._drift is None:
            return
        self._seen_lengths.append(n)
        if len(self._seen_lengths) > 4096:
            del self._seen_lengths[:2048]
        if len(self._seen_lengths) % 32 == 0:
            kl, drifted, _ = self._drift.assess(self._seen_lengths)
            self.metrics.set_gauge("skein_workload_drift_kl", float(kl))
            self.metrics.set_gauge("skein_workload_drifted", 1.0 if drifted else 0.0)

    def drift(self):
        """(kl, drifted, samples) of the prompt lengths seen so far against the plan's workload, or None."""
        return self._drift.assess(self._seen_lengths) if self._drift is not None else None

    # ---- one scheduler iteration ----------------------------------------------------------------------------
    def step(self, now_ms: int | None = None) -> list[TokenEvent]:
        now = self.clock() if now_ms is None else now_ms
        self.batcher.promote_ready(now)
        prefill, decode = self.batcher.next_step_batch()
        self.last_step_failed = False
        if not prefill and not decode:
            self._drop_prelaunched()
            return []
        t0 = time.perf_counter()
        self.step_started_at = time.monotonic()
        try:
            if self.failure_injector is not None:
                self.failure_injector(self._step)
            events = self._run(prefill, decode, now)
        except Exception as e:  # retire the batch, keep serving
            events = self.abort_all(f"{type(e).__name__}: {e}")
            self.last_step_failed = True
            self.metrics.count("skein_step_failures_total")
            if getattr(e, "peer_timeout", False) or "peer flag" in str(e):
                # a bounded device wait on another rank ran out (ops.Workspace.check_status)
                self.metrics.count("skein_comm_timeout_total")
        self._count_graph_activity()
        us = (time.perf_counter() - t0) * 1e6
        wait_ns = getattr(self.runner, "last_wait_ns", 0)
        comm_us = max(0, wait_ns - self._wait_ns_seen) / 1e3     # time the reduce kernels stood waiting for peers
        self._wait_ns_seen = wait_ns
        self.metrics.record_step(self._step, len(decode) + len(prefill), max(0.0, us - comm_us), comm_us, self.kv.in_use_pages)
        if self._otlp is not None:
            end = time.time_ns()
            self._otlp.span("engine.step", end - int(us * 1e3), end,
                            attrs={"step": self._step, "decode_sequences": len(decode), "prefill_sequences": len(prefill),
                                   "peer_wait_us": float(comm_us), "kv_pages_in_use": int(self.kv.in_use_pages)},
                            error="step failed" if self.last_step_failed else None)
        self._step += 1
        self.step_started_at = None
        return events

    def abort_all(self, reason: str) -> list[TokenEvent]:
        """Drop everything in flight (a step failed here or on another rank): the requests' streams end with an
        error and their pages leave the prefix cache; queued requests stay queued."""
        self._drop_prelaunched()
        self._drop_flights()
        events = [TokenEvent(rid, -1, True, error=reason) for rid in self.batcher.retire_all()]
        if self._otlp is not None:
            for ev in events:
                tr = self._req_t0.pop(ev.request_id, None)
                if tr is not None:
                    self._otlp.span("request", tr[1], time.time_ns(), trace_id=tr[0],
                                    attrs={"request_id": int(ev.request_id), "prompt_tokens": tr[2]}, error=reason)
        for ev in events:
            self._sampling.pop(ev.request_id, None)
            self._dp_release(ev.request_id)
            self.metrics.record_request(ev.request_id, "failed", 0.0, 0.0, 0, 0)
        return events

    def _count_graph_activity(self) -> None:
        """skein_graph_captures_total / skein_graph_replays_total follow the runner's CUDA-graph counters."""
        cap, rep = getattr(self.runner, "graph_captures", 0), getattr(self.runner, "graph_replays", 0)
        seen_cap, seen_rep = self._graph_seen
        if cap > seen_cap:
            self.metrics.count("skein_graph_captures_total", cap - seen_cap)
        if rep > seen_rep:
            self.metrics.count("skein_graph_replays_total", rep - seen_rep)
        self._graph_seen = (cap, rep)

    def _rows(self, rids):
        """Per-row sampling parameters of a step, or None when every request in it is greedy."""
        if not self._sampling or not any(r in self._sampling for r in rids):
            return None
        return [self._sampling.get(r, GREEDY).row() for r in rids]      # id 0 (a padding row) is greedy like any other

    def _run_prefill(self, prefill, stamp, events) -> None:
        seqs = []
        for rid, start, end, last in prefill:
            prompt = self.batcher.prompt(rid)
            seqs.append((prompt[start:end], self.kv.pages_for(rid), start))
        toks = self.runner.prefill(seqs, sampling=self._rows([p[0] for p in prefill]))
        for (rid, start, end, last), tok in zip(prefill, toks):
            self.batcher.prefill_advanced(rid, end)
            if last:
                events.append(self._accept(rid, tok, stamp()))

    def _run_continuous(self, prefill, decode, now) -> list[TokenEvent]:
        """One step of the continuous pipeline: prefill chunks as usual, then every group of decoding sequences that is not
        on the device is launched (PipelineStage.launch: the host does not wait), then the tokens of the oldest launch
        are accepted. A sequence belongs to one group from its first decode step to its last (the least loaded group
        when it starts). With one group per stage the launches of the other groups keep every stage busy while one
        group's tokens travel back, so the pipeline is drained only by a prefill chunk or when sequences run out.
        Counterpart of the reference's continuous pipelined loops (run_continuous_pipelined and run_continuous_pipelined_mb,
        crates/skein_runtime/src/distributed/gpu_rank.rs:1293, 1566; two stages and equal-length rows there, any number of
        stages and ragged sequences here)."""
        events: list[TokenEvent] = []
        t_begin = time.perf_counter()
        stamp = lambda: now + int((time.perf_counter() - t_begin) * 1000)   # noqa: E731
        if prefill:
            self._run_prefill(prefill, stamp, events)
            started = {p[0] for p in prefill if p[3]}
            decode = list(decode) + [ev.request_id for ev in events if ev.request_id in started and not ev.is_final]
        flying = {g for g, _, _ in self._flights}
        for rid in decode:
            if rid not in self._grp_of:
                g = min(range(self._groups), key=lambda i: (self._grp_load[i], i))
                self._grp_of[rid] = g
                self._grp_load[g] += 1
        for g in range(self._groups):
            if g in flying:
                continue
            ids = [rid for rid in decode if self._grp_of[rid] == g]
            if not ids:
                continue
            bk = self.runner.bucket(len(ids), slot=g)
            rows = self._rows(ids)
            self.runner.stage_decode_inputs(bk, self.batcher, ids, sampling=rows)
            self.runner.pp_launch(bk, sampling=rows is not None)
            self._flights.append((g, bk, ids))
        if self._flights:
            g, bk, ids = self._flights.pop(0)
            out = self.runner.pp_collect(bk)
            fin, counts = self.batcher.accept_tokens(ids, out.data_ptr(), stamp(), self.cfg.eos_token)
            toks = out[:len(ids)].tolist()
            for rid, tok, f, n in zip(ids, toks, fin, counts):
                if f:
                    self._finish(rid, n)
                events.append(TokenEvent(rid, tok, bool(f)))
        return events

    def _drop_flights(self) -> None:
        """Wait for every launch that is still on the device and forget its result (the step failed, or the engine is being
        torn down): the next launch of a group must not find its buffers in use."""
        flights, self._flights = self._flights, []
        for _, bk, _ in flights:
            try:
                self.runner.pp_collect(bk)
            except Exception:       # noqa: BLE001  (the results are being thrown away)
                pass
        self._grp_of.clear()
        self._grp_load = [0] * self._groups

    def _run(self, prefill, decode, now) -> list[TokenEvent]:
        if self._groups > 1:
            return self._run_continuous(prefill, decode, now)
        events: list[TokenEvent] = []
        t_begin = time.perf_counter()
        # a token's time stamp is the step's clock plus the time the step has taken so far, so that TTFT and TPOT
        # include the step that produced the token
        stamp = lambda: now + int((time.perf_counter() - t_begin) * 1000)
        if prefill:
            self._run_prefill(prefill, stamp, events)
        pre, self._pre = self._pre, None
        if pre is not None and pre[1] != list(decode):
            self.runner.decode_wait(pre[0])     # the plan changed under it (requests were dropped): its result is not used
            pre = None
        if decode:
            if pre is not None:
                bk, _, decode, rows = pre
            else:
                bk, _, decode, rows = self._launch_decode(decode)
            out = self.runner.decode_wait(bk)
            fin, counts = self.batcher.accept_tokens(decode, out.data_ptr(), stamp(), self.cfg.eos_token)
            toks = out[:len(decode)].tolist()
            for rid, f, n in zip(decode, fin, counts):
                if f and rid != 0:
                    self._finish(rid, n)
            # everything the next decode step depends on is settled: put it on the device before the Python-side
            # bookkeeping of this one, so that the device does not wait for it
            self._prelaunch()
            for rid, tok, f in zip(decode, toks, fin):
                if rid != 0:                # 0: a padding row of a data-parallel slice
                    events.append(TokenEvent(rid, tok, bool(f)))
        return events

    def _launch_decode(self, decode):
        """Stages and enqueues one decode step for the planned request ids; returns (bucket, ids as planned, rows as laid
        out on the device, sampling rows)."""
        plan = list(decode)
        if self._dp > 1:
            decode = self._dp_layout(decode)
        bk = self.runner.bucket(len(decode))
        rows = self._rows(decode)
        self.runner.stage_decode_inputs(bk, self.batcher, decode, sampling=rows)
        self.runner.decode_launch(bk, sampling=rows is not None)
        return bk, plan, decode, rows

    def _prelaunch(self) -> None:
        """Enqueue the next step's decode right after this step's tokens were accepted (positions, pages and the set of
        decoding sequences are final then). The next call of step() finds it running and only waits for it; a prefill
        chunk planned for that step is queued behind it (different sequences). New requests are admitted as before;
        their prefill simply follows the decode launch of the step instead of preceding it."""
        if not self._prelaunch_ok:
            return
        _, decode = self.batcher.next_step_batch()
        if decode:
            self._pre = self._launch_decode(decode)

    def _drop_prelaunched(self) -> None:
        pre, self._pre = self._pre, None
        if pre is not None:
            try:
                self.runner.decode_wait(pre[0])
            except Exception:       # noqa: BLE001  (the step is being thrown away)
                pass

    def _dp_layout(self, decode):
        """Rows of a decode step under data-parallel attention: one equally sized slice per rank, a sequence always in
        the slice of the rank it was assigned to when it started decoding (the least loaded one), padding rows (id 0)
        at the end of every slice."""
        from .runner import BUCKETS, bucket_for
        groups = [[] for _ in range(self._dp)]
        for rid in decode:
            r = self._dp_of.get(rid)
            if r is None:
                r = min(range(self._dp), key=lambda i: (self._dp_load[i], i))
                self._dp_of[rid] = r
                self._dp_load[r] += 1
            groups[r].append(rid)
        per = max(4, bucket_for(max(len(g) for g in groups)))
        if per * self._dp > BUCKETS[-1]:
            raise RuntimeError(f"{per} rows per rank x {self._dp} ranks exceed the largest capture class {BUCKETS[-1]}")
        rows = []
        for g in groups:
            rows.extend(g + [0] * (per - len(g)))
        return rows

    def _dp_release(self, rid) -> None:
        r = self._dp_of.pop(rid, None)
        if r is not None:
            self._dp_load[r] -= 1

    def _accept(self, rid, tok, now) -> TokenEvent:
        finished, n = self.batcher.accept_token(rid, int(tok), now, self.cfg.eos_token)
        if finished:
            self._finish(rid, n)
        return TokenEvent(rid, int(tok), bool(finished))

    def _finish(self, rid, n) -> None:
        info = self.batcher.request_info(rid)
        ttft = float(info["first_token_ms"] - info["arrival_ms"])
        tpot = float(info["last_token_ms"] - info["first_token_ms"]) / max(1, n - 1)
        self.metrics.record_request(rid, "ok", ttft, tpot, info["prefix_hit_tokens"], n)
        if self._otlp is not None:
            tr = self._req_t0.pop(rid, None)
            if tr is not None:
                self._otlp.span("request", tr[1], time.time_ns(), trace_id=tr[0],
                                attrs={"request_id": int(rid), "prompt_tokens": tr[2], "output_tokens": int(n), "ttft_ms": ttft,
                                       "tpot_ms": tpot, "prefix_hit_tokens": int(info["prefix_hit_tokens"])})
        self.batcher.retire(rid)
        self._sampling.pop(rid, None)
        self._dp_release(rid)
        g = self._grp_of.pop(rid, None)
        if g is not None:
            self._grp_load[g] -= 1

    # ---- helpers ------------------------------------------------------------------------------------------------
    @property
    def idle(self) -> bool:
        return self.batcher.inflight_len == 0 and self.batcher.queued_len == 0

    def run_until_done(self, max_steps: int = 1 << 20, on_event=None) -> dict[int, list[int]]:
        out: dict[int, list[int]] = {}
        steps = 0
        while not self.idle and steps < max_steps:
            evs = self.step()
            if not evs and self.batcher.inflight_len == 0:
                time.sleep(0.001)   # only delayed requests left: wait for their retry time
            for ev in evs:
                if ev.error is None:
                    out.setdefault(ev.request_id, []).append(ev.token)
                if on_event:
                    on_event(ev)
            steps += 1
        return out

    def generate(self, prompts, max_new_tokens: int = 32, sampling: SamplingParams | None = None) -> list[list[int]]:
        """Convenience: submit every prompt now and run to completion. Returns generated ids per prompt."""
        ids = []
        for p in prompts:
            rid, d = self.submit(p, max_new_tokens, sampling=sampling)
            if d.kind == "reject":
                raise RuntimeError(f"request rejected: {d.reason}")
            ids.append(rid)
        res = self.run_until_done()
        return [res.get(i, []) for i in ids]
