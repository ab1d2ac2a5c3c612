"""One process per GPU: launch plan, per-rank command/environment, file rendezvous, wait-and-count.

The parent computes one command per rank (environment: SKEIN_RANK, SKEIN_WORLD_SIZE, SKEIN_RENDEZVOUS,
CUDA_VISIBLE_DEVICES, SKEIN_LOCAL_DEVICE), spawns them, waits, and reports how many failed. Every rank sees all
GPUs of the job, in job order, and computes on the one at index SKEIN_LOCAL_DEVICE: the tensor-parallel kernels read
the peers' buffers through CUDA IPC mappings, which can only be opened for a device the process can see. If one
rank dies, the others get a grace period and are then terminated, so a job never outlives a lost rank; with
`restarts` the whole group is then started again from the artifact (the ranks hold no other state). SIGTERM / SIGINT
to the launcher is passed on to rank 0 only, which shuts the group down cleanly between steps. Ranks meet through a file
rendezvous: the leader publishes a small blob atomically (tmp + rename), the others poll for it with a
timeout and get a clear error if it never appears. torch.distributed is then initialised from the
address carried in the blob.

Counterpart of crates/skein_runtime/src/distributed/launcher.rs:20-72, rendezvous.rs:19,48 and
crates/skein_cli/src/cmd/serve.rs:256-300.
"""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time
from dataclasses import dataclass
from pathlib import Path


class RendezvousError(RuntimeError):
    pass


@dataclass
class RankLaunch:
    rank: int
    world_size: int
    gpu: int
    rendezvous: str
    gpus: tuple = ()      # all devices of the job, in rank order (empty: only `gpu`)


def parse_gpus(spec: str) -> list[int]:
    gpus = [int(x) for x in spec.split(",") if x.strip() != ""]
    if not gpus:
        raise ValueError("--gpus needs at least one device id")
    if len(set(gpus)) != len(gpus):
        raise ValueError("--gpus lists a device twice")
    return gpus


def plan_launch(gpus: list[int], rendezvous: str) -> list[RankLaunch]:
    return [RankLaunch(r, len(gpus), g, rendezvous, tuple(gpus)) for r, g in enumerate(gpus)]


def visible_devices(gpus, parent_visible: str | None) -> str:
    """CUDA_VISIBLE_DEVICES of a child: the job's devices in rank order. Ids given to --gpus index the devices the
    parent itself can see, so a launcher that runs under a restricted CUDA_VISIBLE_DEVICES hands down the right ones."""
    if parent_visible:
        seen = [x.strip() for x in parent_visible.split(",") if x.strip()]
        if any(g >= len(seen) for g in gpus):
            raise ValueError(f"--gpus names device {max(gpus)} but only {len(seen)} are visible ({parent_visible})")
        return ",".join(seen[g] for g in gpus)
    return ",".join(str(g) for g in gpus)


def build_command(launch: RankLaunch, argv: list[str], base_env: dict | None = None):
    """Returns (argv, env) of the child for this rank."""
    env = dict(base_env if base_env is not None else os.environ)
    gpus = launch.gpus or (launch.gpu,)
    env.update({"SKEIN_RANK": str(launch.rank), "SKEIN_WORLD_SIZE": str(launch.world_size),
                "SKEIN_RENDEZVOUS": launch.rendezvous, "SKEIN_LOCAL_DEVICE": str(gpus.index(launch.gpu)),
                "CUDA_VISIBLE_DEVICES": visible_devices(gpus, env.get("CUDA_VISIBLE_DEVICES"))})
    return [sys.executable, "-m", "skein_b200.parallel.worker", *argv], env


def wait_ranks(procs, timeout_s: float | None = None, grace_s: float = 10.0, poll_s: float = 0.05, monitor=None,
               log=None) -> list[int]:
    """Wait for every rank. Once one has failed, the rest get `grace_s` to finish by themselves (they usually notice
    through their own time-outs) and are then terminated. `monitor` (watchdog.Monitor over the ranks' heartbeat
    files) also catches a rank whose process is alive but has stopped beating: it is terminated, which makes it a
    failed rank like any other. Returns the exit codes in rank order."""
    t0 = time.monotonic()
    first_failure = None
    next_beat_check = t0
    codes: list = [None] * len(procs)
    while any(c is None for c in codes):
        for i, p in enumerate(procs):
            if codes[i] is None:
                codes[i] = p.poll()
                if codes[i] not in (None, 0) and first_failure is None:
                    first_failure = time.monotonic()
        now = time.monotonic()
        if monitor is not None and now >= next_beat_check:
            next_beat_check = now + 0.2
            for r in monitor.dead_ranks(now, started_only=True):
                if r < len(procs) and codes[r] is None:
                    if log is not None:
                        log(f"rank {r} stopped beating: terminating it")
                    procs[r].terminate()
        overdue = timeout_s is not None and now - t0 > timeout_s
        orphaned = first_failure is not None and now - first_failure > grace_s
        if overdue or orphaned:
            for i, p in enumerate(procs):
                if codes[i] is None:
                    p.terminate()
            for i, p in enumerate(procs):
                if codes[i] is None:
                    try:
                        p.wait(5.0)
                    except subprocess.TimeoutExpired:
                        p.kill()
                        p.wait()
                    codes[i] = p.returncode if p.returncode != 0 else -15
            break
        time.sleep(poll_s)
    return codes


class StopRequest:
    """Set by the launcher's SIGTERM / SIGINT handler. The signal is passed on to rank 0 only: rank 0 closes its HTTP
    front end, drains, and announces the stop to the other ranks over the control group, so that every rank leaves
    between steps with nothing in flight. A stopped group is never restarted."""

    def __init__(self):
        self.requested = False
        self.procs = []

    def __call__(self, signum=None, frame=None):
        import signal
        self.requested = True
        if self.procs and self.procs[0].poll() is None:
            self.procs[0].send_signal(signal.SIGTERM)


def supervise(spawn, restarts: int = 0, timeout_s: float | None = None, grace_s: float = 10.0, log=None, make_monitor=None,
              stop: "StopRequest | None" = None):
    """Run a rank group to completion, starting it again (from scratch: the ranks keep no state outside the
    artifact) up to `restarts` times when a rank is lost. `spawn()` starts one process per rank and returns them.
    Returns (number of ranks that failed in the last attempt, attempts made)."""
    attempt = 0
    while True:
        attempt += 1
        procs = spawn()
        if stop is not None:
            stop.procs = procs
            if stop.requested:       # the signal came while the group was being started
                stop()
        codes = wait_ranks(procs, timeout_s, grace_s, monitor=make_monitor() if make_monitor else None, log=log)
        failed = sum(rc != 0 for rc in codes)
        if failed == 0 or attempt > restarts or (stop is not None and stop.requested):
            return failed, attempt
        if log is not None:
            log(f"rank group lost {failed} rank(s) (exit codes {codes}); restart {attempt} of {restarts}")


def launch_ranks(gpus: list[int], rendezvous: str, argv: list[str], timeout_s: float | None = None, grace_s: float = 10.0,
                 restarts: int = 0) -> int:
    """Spawn every rank, wait for all, return the number of ranks that failed (after `restarts` fresh starts of the
    whole group, if asked for)."""
    from .watchdog import Monitor
    hb_dir = Path(rendezvous + ".hb")

    def spawn():
        rdv = Path(rendezvous)
        if rdv.exists():
            rdv.unlink()            # a restarted group must not meet through the previous group's blob
        if hb_dir.is_dir():
            for f in hb_dir.glob("rank_*.hb"):
                f.unlink()
        procs = []
        for l in plan_launch(gpus, rendezvous):
            cmd, env = build_command(l, argv)
            env["SKEIN_HEARTBEAT_DIR"] = str(hb_dir)
            procs.append(subprocess.Popen(cmd, env=env))
        return procs

    import signal
    import threading
    stop = StopRequest()
    previous = {}
    if threading.current_thread() is threading.main_thread():      # handlers can only be installed there
        for sig in (signal.SIGTERM, signal.SIGINT):
            previous[sig] = signal.signal(sig, stop)
    try:
        # a beat every 0.5 s; 120 missed beats (60 s) before a rank that is still running counts as lost: weight
        # loading and graph capture can hold the interpreter for seconds at a time
        failed, _ = supervise(spawn, restarts, timeout_s, grace_s, log=lambda m: print(m, file=sys.stderr, flush=True),
                              make_monitor=lambda: Monitor(str(hb_dir), len(gpus), interval_s=0.5, missed_beats=120),
                              stop=stop)
    finally:
        for sig, h in previous.items():
            signal.signal(sig, h)
    return failed


def local_device_index() -> int:
    """Index (within this process's visible devices) of the GPU this rank computes on."""
    return int(os.environ.get("SKEIN_LOCAL_DEVICE", "0"))


def world_from_env():
    """(rank, world_size, rendezvous path) from SKEIN_RANK / SKEIN_WORLD_SIZE / SKEIN_RENDEZVOUS, or None."""
    if "SKEIN_RANK" not in os.environ or "SKEIN_WORLD_SIZE" not in os.environ:
        return None
    return int(os.environ["SKEIN_RANK"]), int(os.environ["SKEIN_WORLD_SIZE"]), os.environ.get("SKEIN_RENDEZVOUS", "/tmp/skein_rendezvous")


# ---- file rendezvous ------------------------------------------------------------------------------------------
def publish(path: str, payload: bytes) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    tmp = p.with_name(p.name + f".{os.getpid()}.tmp")
    tmp.write_bytes(payload)
    os.replace(tmp, p)     # readers see either nothing or the whole blob


def fetch(path: str, timeout_s: float = 60.0, poll_s: float = 0.02) -> bytes:
    p = Path(path)
    t0 = time.monotonic()
    while True:
        if p.exists():
            data = p.read_bytes()
            if data:
                return data
        if time.monotonic() - t0 > timeout_s:
            raise RendezvousError(f"rendezvous file {path} did not appear within {timeout_s:g} s (is rank 0 running?)")
        time.sleep(poll_s)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_process_group(rank: int, world: int, rendezvous: str, backend: str = "nccl", timeout_s: float = 120.0, device=None):
    """Rank 0 picks a port and publishes it; everyone initialises torch.distributed over 127.0.0.1."""
    import datetime

    import torch.distributed as dist

    if rank == 0:
        blob = {"addr": "127.0.0.1", "port": free_port(), "world": world}
        publish(rendezvous, json.dumps(blob).encode())
    else:
        blob = json.loads(fetch(rendezvous, timeout_s))
        if blob["world"] != world:
            raise RendezvousError(f"rendezvous was published for world size {blob['world']}, this rank expects {world}")
    kw = {"device_id": device} if (device is not None and backend == "nccl") else {}
    dist.init_process_group(backend, init_method=f"tcp://{blob['addr']}:{blob['port']}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=max(timeout_s, 60.0)), **kw)
    return dist.group.WORLD
