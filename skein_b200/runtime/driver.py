"""Engine driver and control plane: one thread owns the engine and steps it; on a multi-rank job rank 0
leads and the other ranks follow in lock step.

Control plane. Every rank runs the same engine on the same request stream, so all of them take the same
scheduling decisions and meet in the fused collectives. What the followers need from the leader each
iteration is small: "step now, clock = t", and only sometimes a payload (new requests, a stop, an admin
command). The iteration header therefore lives in a shared-memory page (`SharedControl`: a memory-mapped
file, one writer per word) that followers poll, and the pickled payload is broadcast over the gloo group
only on iterations that have one. After every step each rank publishes "done, failed?" in its own slot and
all ranks read every slot before the next step: if any rank's step failed (a device wait that ran out, an
exception), every rank drops the batch and the communicators are re-armed behind a barrier, so the ranks
never drift apart in what they schedule or in their flag epochs.

The reference broadcasts every token and every control decision with a host collective per step
(crates/skein_runtime/src/distributed/gpu_rank.rs:601-624, batch_driver.rs:219-514) and drives the engine
from a dedicated thread behind the HTTP handlers (crates/skein_runtime/src/server/forward.rs:237-420).
"""
from __future__ import annotations

import mmap
import os
import queue
import threading
import time

from .engine import Engine, SamplingParams, TokenEvent


class LocalControl:
    """Single-rank job: nothing to announce, nothing to agree on."""
    world, rank = 1, 0

    def lead(self, payload, now_ms):
        return payload

    def agree_failed(self, failed: bool) -> bool:
        return failed

    def barrier(self):
        pass

    def close(self):
        pass


class SharedControl:
    """Lock-step control for the ranks of one node.

    Header (written by rank 0): [seq, has_payload, now_ms]; then one slot per rank: [seq_done, failed].
    Words are 8 bytes and each has a single writer; the header's `seq` is written last, a rank's
    `seq_done` is written after its `failed`, so a reader that sees the new sequence number sees the rest.
    """
    HDR = 8

    def __init__(self, path: str, rank: int, world: int, group=None, wait_s: float = 120.0):
        import numpy as np
        self.rank, self.world, self.group, self.wait_s = rank, world, group, wait_s
        n_words = self.HDR + 2 * world
        size = n_words * 8
        if rank == 0:
            with open(path + ".tmp", "wb") as f:
                f.write(b"\0" * size)
            os.replace(path + ".tmp", path)
        if group is not None:
            # nobody maps the page before rank 0 has put a fresh one in place (a restarted job finds the old file)
            import torch.distributed as dist
            dist.barrier(group=group)
        elif rank != 0:
            t0 = time.monotonic()
            while not os.path.exists(path) or os.path.getsize(path) < size:
                if time.monotonic() - t0 > wait_s:
                    raise TimeoutError(f"control page {path} never appeared")
                time.sleep(0.01)
        self._f = open(path, "r+b")
        self._mm = mmap.mmap(self._f.fileno(), size)
        self.w = np.frombuffer(self._mm, dtype=np.int64)
        self.seq = 0
        self.path = path

    def _spin(self, cond, what):
        t0 = time.monotonic()
        n = 0
        while not cond():
            n += 1
            if n > 2000:
                time.sleep(0.00005)
                if time.monotonic() - t0 > self.wait_s:
                    raise TimeoutError(f"control plane: {what} (waited {self.wait_s:g} s)")

    def _bcast(self, payload):
        import torch.distributed as dist
        box = [payload]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]

    # ---- leader ----
    def lead(self, payload, now_ms: int):
        """Announce one iteration. `payload` (a dict or None) is broadcast only when there is one."""
        self.seq += 1
        self.w[1] = 1 if payload is not None else 0
        self.w[2] = int(now_ms)
        self.w[0] = self.seq
        if payload is not None:
            self._bcast(payload)
        return payload

    # ---- follower ----
    def follow(self):
        """Block until the leader announces the next iteration. Returns (payload or None, now_ms)."""
        nxt = self.seq + 1
        self._spin(lambda: self.w[0] >= nxt, "the leader stopped announcing iterations")
        self.seq = nxt
        has, now = int(self.w[1]), int(self.w[2])
        return (self._bcast(None) if has else None), now

    # ---- both ----
    def agree_failed(self, failed: bool) -> bool:
        """Publish this rank's outcome of iteration `seq` and return whether the step failed on ANY rank."""
        base = self.HDR + 2 * self.rank
        self.w[base + 1] = 1 if failed else 0
        self.w[base] = self.seq
        seq = self.seq
        self._spin(lambda: all(self.w[self.HDR + 2 * r] >= seq for r in range(self.world)), "a rank never finished its step")
        return any(int(self.w[self.HDR + 2 * r + 1]) for r in range(self.world))

    def barrier(self):
        import torch.distributed as dist
        dist.barrier(group=self.group)

    def close(self):
        try:
            self.w = None
            self._mm.close()
            self._f.close()
        except (BufferError, ValueError, OSError):
            pass


def _apply(engine: Engine, payload, now_ms: int, replies=None):
    """Apply an iteration's payload identically on every rank. Returns the streams opened (leader only)."""
    opened = {}
    if not payload:
        return opened
    for i, (rid, prompt, max_new, smp) in enumerate(payload.get("new", ())):
        sampling = SamplingParams(*smp) if smp else None
        reply = replies[i] if replies else None
        try:
            _, d = engine.submit(prompt, max_new, now_ms=now_ms, request_id=rid, sampling=sampling)
        except ValueError as e:
            if reply:
                reply.put((rid, "reject", str(e), None))
            continue
        if not reply:
            continue
        if d.kind == "reject":
            reply.put((rid, "reject", d.reason, None))
        else:
            q: "queue.Queue[TokenEvent]" = queue.Queue()
            opened[rid] = q
            reply.put((rid, d.kind, d.reason, q))
    return opened


def _after_step(engine: Engine, control, events, resync):
    """Agree on the step's outcome; if it failed anywhere, drop the batch everywhere and re-arm the communicators."""
    failed_any = control.agree_failed(engine.last_step_failed)
    if failed_any:
        if not engine.last_step_failed:
            events = list(events) + engine.abort_all("StepFailed: the step failed on another rank")
            engine.metrics.count("skein_step_failures_total")
        if resync is not None:
            resync(control)
    return events


def _mount(engine: Engine, swap, rank: int):
    from .hotswap import mount_weights
    mount_weights(engine, swap["artifact"], rank)


class EngineDriver:
    """Runs the engine on its own thread. Thread-safe `submit` returns an event queue; `swap` replaces the weights
    between two steps once the in-flight requests have drained. With a `SharedControl` this is rank 0 of a
    multi-rank job and every iteration is announced to the followers first."""

    def __init__(self, engine: Engine, control=None, rank: int = 0, resync=None, idle_sleep_s: float = 0.001):
        self.engine, self.control, self.rank, self.resync = engine, control or LocalControl(), rank, resync
        self._inbox: "queue.Queue" = queue.Queue()
        self._streams: dict[int, "queue.Queue[TokenEvent]"] = {}
        self._stop = threading.Event()
        self._idle_sleep = idle_sleep_s
        self._thread = threading.Thread(target=self._run, name="skein-engine-driver", daemon=True)
        self.draining = False
        self._pending_swap = None      # (artifact path, deadline, reply queue)
        self._next_id = 1
        self.error = None

    def start(self):
        self._thread.start()
        return self

    def stop(self, timeout: float = 10.0):
        self._stop.set()
        self._thread.join(timeout)
        from ..utils import otlp
        otlp.shutdown()          # ships the spans still queued (no-op without SKEIN_OTLP_ENDPOINT)

    def submit(self, prompt_ids, max_new_tokens, sampling: SamplingParams | None = None):
        """Returns (request_id, decision_kind, reason, event_queue or None). Blocks until the driver has decided."""
        reply: "queue.Queue" = queue.Queue(maxsize=1)
        self._inbox.put(("req", prompt_ids, max_new_tokens, sampling, reply))
        return reply.get()

    def swap(self, artifact_path: str, timeout_s: float) -> tuple[bool, str]:
        """Drain, then mount the weights of `artifact_path` on every rank between two steps. Returns (ok, message);
        on a drain time-out the old weights stay mounted and admission resumes."""
        reply: "queue.Queue" = queue.Queue(maxsize=1)
        self._inbox.put(("swap", str(artifact_path), float(timeout_s), reply))
        return reply.get()

    @property
    def inflight(self) -> int:
        return len(self._streams)

    def drain(self, timeout_s: float) -> bool:
        """Stop admitting, wait for in-flight requests to finish. True if drained in time."""
        self.draining = True
        t0 = time.monotonic()
        while self._streams and time.monotonic() - t0 < timeout_s:
            time.sleep(0.005)
        ok = not self._streams
        if not ok:
            self.draining = False     # timeout: keep serving on the old state
        return ok

    # ---- the loop ----
    def _collect(self, block: bool):
        items = []
        try:
            items.append(self._inbox.get(timeout=0.02) if block else self._inbox.get_nowait())
            while True:
                items.append(self._inbox.get_nowait())
        except queue.Empty:
            pass
        return items

    def _run(self):
        try:
            self._loop()
        except BaseException as e:   # the thread must not die silently: fail what is open
            self.error = e
            for q in list(self._streams.values()):
                q.put(TokenEvent(0, -1, True, error=f"driver stopped: {type(e).__name__}: {e}"))
            self._streams.clear()
            raise

    def _loop(self):
        eng, ctl = self.engine, self.control
        while True:
            items = self._collect(block=eng.idle and self._pending_swap is None and not self._stop.is_set())
            new, replies = [], []
            for it in items:
                if it[0] == "swap":
                    _, path, timeout_s, reply = it
                    if self._pending_swap is not None:
                        reply.put((False, "another swap is in progress"))
                    else:
                        self.draining = True
                        self._pending_swap = (path, time.monotonic() + timeout_s, reply)
                    continue
                _, prompt, max_new, smp, reply = it
                if self.draining:
                    reply.put((0, "reject", "draining", None))
                    continue
                rid = self._next_id
                self._next_id += 1
                new.append((rid, list(prompt), int(max_new), smp.row() if smp is not None and not smp.greedy else None))
                replies.append(reply)
            swap_now = None
            if self._pending_swap is not None:
                path, deadline, reply = self._pending_swap
                if not self._streams and eng.idle:
                    swap_now = {"artifact": path}
                elif time.monotonic() > deadline:
                    self._pending_swap, self.draining = None, False
                    reply.put((False, "drain timed out; the old artifact stays mounted"))
            stop = self._stop.is_set() and eng.idle and not new and swap_now is None
            if eng.idle and not new and swap_now is None and not stop:
                continue
            now = eng.clock()
            payload = None
            if new or stop or swap_now:
                payload = {"new": new, "stop": stop, "swap": swap_now}
            ctl.lead(payload, now)
            if stop:
                return
            if swap_now:
                path, _, reply = self._pending_swap
                try:
                    _mount(eng, swap_now, self.rank)
                    ctl.barrier()
                    reply.put((True, "mounted"))
                except Exception as e:
                    reply.put((False, f"{type(e).__name__}: {e}"))
                self._pending_swap, self.draining = None, False
            self._streams.update(_apply(eng, payload, now, replies))
            events = eng.step(now)
            events = _after_step(eng, ctl, events, self.resync)
            for ev in events:
                q = self._streams.get(ev.request_id)
                if q is not None:
                    q.put(ev)
                    if ev.is_final:
                        del self._streams[ev.request_id]
            if not events and not eng.idle:
                time.sleep(self._idle_sleep)    # only delayed requests: wait for their retry time


def follower_loop(engine: Engine, control: SharedControl, rank: int, resync=None):
    """Ranks other than 0: apply what the leader announces, step, agree on the outcome."""
    while True:
        payload, now = control.follow()
        if payload and payload.get("stop"):
            return
        if payload and payload.get("swap"):
            _mount(engine, payload["swap"], rank)
            control.barrier()
        _apply(engine, payload, now)
        events = engine.step(now)
        _after_step(engine, control, events, resync)
