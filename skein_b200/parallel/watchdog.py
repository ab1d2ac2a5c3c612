"""Host-side failure detection: heartbeats in a shared directory and a monitor that declares a rank dead.

Each rank touches `<dir>/rank_<r>.hb` with a monotonically increasing counter from a daemon thread; the thread
stops beating while the rank's main loop has been inside one step for longer than `stall_limit_s` (the engine
publishes when a step began), so a rank whose main thread is stuck in a synchronisation or a collective looks
dead to the monitor although its process is alive, while an idle rank keeps beating. The
monitor (any rank, or the launcher: `launcher.launch_ranks` watches the ranks it started) reads the files; a rank whose counter has not moved for
`missed_beats x interval` is reported dead, after which the caller aborts its communicator / stops launching
fused steps and fails in-flight requests with a retriable status. Nothing here touches a GPU: device-side
waits are bounded on their own (status word), this layer catches ranks that died on the host.

The reference has no heartbeat (its launcher only counts failed children at exit:
crates/skein_cli/src/cmd/serve.rs:256-298); its shared-memory all-reduce spins forever on a dead peer
(crates/skein_runtime/src/cuda/shm_allreduce.rs:53).
"""
from __future__ import annotations

import os
import threading
import time
from pathlib import Path


class Heartbeat:
    def __init__(self, directory: str, rank: int, interval_s: float = 0.2, step_started_at=None, stall_limit_s: float = 30.0):
        """step_started_at: callable returning the monotonic time at which the step in progress began, or None
        between steps."""
        self.path = Path(directory) / f"rank_{rank}.hb"
        self.interval_s = interval_s
        self.step_started_at, self.stall_limit_s = step_started_at, stall_limit_s
        self._stop = threading.Event()
        self._n = 0
        self._t = threading.Thread(target=self._run, daemon=True)
        Path(directory).mkdir(parents=True, exist_ok=True)

    def start(self):
        self._beat()
        self._t.start()
        return self

    def stop(self):
        self._stop.set()
        self._t.join(2.0)

    def _beat(self):
        self._n += 1
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(str(self._n))
        os.replace(tmp, self.path)

    def stalled(self, now: float | None = None) -> bool:
        if self.step_started_at is None:
            return False
        t = self.step_started_at()
        return t is not None and (time.monotonic() if now is None else now) - t > self.stall_limit_s

    def _run(self):
        while not self._stop.wait(self.interval_s):
            if not self.stalled():
                self._beat()


class Monitor:
    def __init__(self, directory: str, world: int, interval_s: float = 0.2, missed_beats: int = 5):
        self.dir, self.world = Path(directory), world
        self.limit_s = interval_s * missed_beats
        self._last = {}     # rank -> (counter, time it last changed)

    def dead_ranks(self, now: float | None = None, started_only: bool = False) -> list[int]:
        """Ranks whose counter has not moved for the limit. started_only: a rank that has not written its first
        beat yet (still importing, loading weights) is not judged."""
        now = time.monotonic() if now is None else now
        dead = []
        for r in range(self.world):
            p = self.dir / f"rank_{r}.hb"
            try:
                n = int(p.read_text() or 0)
            except (FileNotFoundError, ValueError):
                n = -1
            if n < 0 and started_only:
                continue
            prev = self._last.get(r)
            if prev is None or prev[0] != n:
                self._last[r] = (n, now)
            elif now - prev[1] > self.limit_s:
                dead.append(r)
        return dead
