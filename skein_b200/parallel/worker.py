"""Rank worker: one process per GPU. Loads its shard of an artifact, joins the group, and either serves HTTP
(rank 0 hosts the front end and broadcasts the request stream) or runs a generation job.

Every rank runs the same Engine on the same inputs: rank 0 is the only one that sees clients; each
scheduler iteration it broadcasts {new requests, clock, stop} over a CPU (gloo) control group, all ranks
apply it and step. Data-plane traffic (the fused collectives) never touches the host.

Counterpart of RankServer::bootstrap / run_rank (crates/skein_runtime/src/distributed/gpu_rank.rs:104-410,
crates/skein_cli/src/cmd/serve.rs:322), with the HTTP server in front of the multi-GPU workers instead
of a single-process executor.
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import sys
import threading
import time

import torch
import torch.distributed as dist

from ..compile.artifact import Artifact
from ..models.decoder import Decoder
from ..runtime.engine import Engine, EngineConfig, TokenEvent
from ..runtime.tokenizer import Tokenizer
from . import launcher


def size_kv_pool(art: Artifact, lay, device, total_kv_bytes: int, page_size: int = 16, reserve_frac: float = 0.08) -> int:
    """Pages in the per-layer pool: from an explicit byte budget, else from the memory left after the weights."""
    cfg = art.cfg
    n_layers = len(lay.stage_layers(cfg.num_layers))
    kv_heads = cfg.num_kv_heads // lay.tp
    page_bytes = 2 * kv_heads * page_size * cfg.head_dim * 2 * n_layers
    if total_kv_bytes > 0:
        return max(8, total_kv_bytes // page_bytes)
    if device.type != "cuda":
        return 256
    free, total = torch.cuda.mem_get_info(device)
    return max(8, int((free - reserve_frac * total) // page_bytes))


def build_engine(art: Artifact, rank: int, device, comm, args, comm_moe=None, pp_info=None) -> Engine:
    lay = art.layout(rank)
    art.check_lowering(rank)
    tuned = art.path / "cache" / "kernel_configs.json"
    if tuned.exists() and device.type == "cuda":
        from ..ops import tuning
        tuning.activate(tuning.KernelConfigCache(tuned, strict=False))   # measured configurations win over the heuristics
    weights = art.load_weights(rank, device)
    pages = size_kv_pool(art, lay, device, args.total_kv_bytes)
    pages = min(pages, max(8, (args.max_seq_len // 16 + 1) * max(1, args.max_batch or art.plan["batching"]["max_batch"]) * 2))
    dec = Decoder(art.cfg, weights, lay, num_pages=pages, page_size=art.plan["kv"]["layout"].get("page_size", 16),
                  max_pos=min(args.max_seq_len, art.cfg.max_position_embeddings), comm=comm, comm_moe=comm_moe)
    if pp_info is not None:
        from .pp import PipelineStage
        dec = PipelineStage(dec, lay, *pp_info)
    batching = art.plan["batching"]
    fused = all(c is None or c.mode == "fused" for c in (comm, comm_moe))
    ecfg = EngineConfig(max_batch=args.max_batch or batching["max_batch"], chunk_tokens=batching.get("chunk_tokens", 0),
                        prefix_cache=art.plan["execution"]["prefix_cache"]["enable"],
                        # stage-to-stage NCCL p2p and library collectives are launched eagerly, never captured
                        use_graphs=device.type == "cuda" and art.plan["execution"]["cuda_graphs"]["enable"] and fused and pp_info is None)
    if args.workload:
        from .. import core
        w = core.workload_parse(open(args.workload).read())
        ecfg.ttft_ms, ecfg.tpot_ms = w["ttft_p95_ms"], w["tpot_p95_ms"]
    if args.cost:
        from .. import core
        c = json.loads(core.cost_constants_json(open(args.cost).read())).get("runtime_estimator", {})
        ecfg.decode_us_at_b1 = c.get("per_token_decode_us_at_b1", ecfg.decode_us_at_b1)
        ecfg.batch_exponent = c.get("batch_scaling_exponent", ecfg.batch_exponent)
        ecfg.prefill_per_token_us = c.get("prefill_per_token_us", ecfg.prefill_per_token_us)
    return Engine(dec, ecfg)


class ControlPlane:
    """Keeps the ranks' engines in lock step. Rank 0 calls `lead`, the others `follow`."""

    def __init__(self, group, rank: int):
        self.group, self.rank = group, rank

    def lead(self, new_requests, now_ms: int, stop: bool = False):
        msg = [{"new": new_requests, "now": now_ms, "stop": stop}]
        if self.group is not None:
            dist.broadcast_object_list(msg, src=0, group=self.group)
        return msg[0]

    def follow(self):
        msg = [None]
        dist.broadcast_object_list(msg, src=0, group=self.group)
        return msg[0]


class DistributedDriver:
    """Rank 0's engine driver for a multi-rank job: like runtime.server.EngineDriver, but every iteration is
    announced to the follower ranks first."""

    def __init__(self, engine: Engine, control: ControlPlane):
        self.engine, self.control = engine, control
        self._inbox: "queue.Queue" = queue.Queue()
        self._streams = {}
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="skein-dist-driver", daemon=True)
        self.draining = False
        self._next_id = 1

    def start(self):
        self._thread.start()
        return self

    def stop(self, timeout=10.0):
        self._stop.set()
        self._thread.join(timeout)

    @property
    def inflight(self):
        return len(self._streams)

    def submit(self, prompt_ids, max_new_tokens):
        reply: "queue.Queue" = queue.Queue(maxsize=1)
        self._inbox.put((prompt_ids, max_new_tokens, reply))
        return reply.get()

    def _run(self):
        eng = self.engine
        while True:
            batch = []
            try:
                block = eng.idle and not self._stop.is_set()
                item = self._inbox.get(timeout=0.05) if block else self._inbox.get_nowait()
                batch.append(item)
                while True:
                    batch.append(self._inbox.get_nowait())
            except queue.Empty:
                pass
            stop = self._stop.is_set() and eng.idle and not batch
            if eng.idle and not batch and not stop:
                continue
            now = eng.clock()
            new = []
            for prompt, max_new, reply in batch:
                rid = self._next_id
                self._next_id += 1
                new.append((rid, prompt, max_new))
            self.control.lead(new, now, stop)
            if stop:
                return
            for (rid, prompt, max_new), (_, _, reply) in zip(new, batch):
                try:
                    _, d = eng.submit(prompt, max_new, now_ms=now, request_id=rid)
                except ValueError as e:
                    reply.put((rid, "reject", str(e), None))
                    continue
                if d.kind == "reject":
                    reply.put((rid, "reject", d.reason, None))
                else:
                    q: "queue.Queue[TokenEvent]" = queue.Queue()
                    self._streams[rid] = q
                    reply.put((rid, d.kind, d.reason, q))
            for ev in eng.step(now):
                q = self._streams.get(ev.request_id)
                if q is not None:
                    q.put(ev)
                    if ev.is_final:
                        del self._streams[ev.request_id]


def follower_loop(engine: Engine, control: ControlPlane):
    while True:
        msg = control.follow()
        if msg["stop"]:
            return
        for rid, prompt, max_new in msg["new"]:
            try:
                engine.submit(prompt, max_new, now_ms=msg["now"], request_id=rid)
            except ValueError:
                pass
        engine.step(msg["now"])


def run_rank(args) -> int:
    env = launcher.world_from_env()
    rank, world, rdv = env if env else (0, 1, args.rendezvous)
    use_cuda = torch.cuda.is_available() and not args.cpu
    # every rank sees all GPUs of the job (the peers' buffers are mapped through CUDA IPC) and computes on its own
    device = torch.device("cuda", launcher.local_device_index()) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    beat = None
    if os.environ.get("SKEIN_HEARTBEAT_DIR"):      # set by the launcher, which watches the file (watchdog.py)
        from .watchdog import Heartbeat
        beat = Heartbeat(os.environ["SKEIN_HEARTBEAT_DIR"], rank, interval_s=0.5).start()
    art = Artifact(args.artifact)
    if art.num_devices != world:
        raise SystemExit(f"artifact was compiled for {art.num_devices} devices, launched with {world}")
    comm, comm_moe, pp_info, control_group = None, None, None, None
    if world > 1:
        from . import pp as pp_mod
        launcher.init_process_group(rank, world, rdv, "nccl" if use_cuda else "gloo", device=device if use_cuda else None)
        control_group = dist.new_group(backend="gloo")
        tp, pp, ep = art.layout_dims
        lay = art.layout(rank)
        tp_group, pp_ranks, pp_group = pp_mod.make_groups(art.layout_dims, rank)
        # one group per pipeline stage (its tp x ep ranks): the expert-parallel combine runs over it
        stage_group = None
        for s in range(pp):
            ranks = list(range(s * tp * ep, (s + 1) * tp * ep))
            g = dist.new_group(ranks) if (ep > 1 and len(ranks) > 1) else None
            if rank in ranks:
                stage_group = g
        if use_cuda:
            from .tp import TPComm
            if tp > 1:
                comm = TPComm(tp_group, device, hidden=art.cfg.hidden_size)
            if ep > 1:
                comm_moe = TPComm(stage_group, device, hidden=art.cfg.hidden_size)
        elif tp > 1 or ep > 1:
            raise SystemExit("tensor/expert-parallel serving needs GPUs (CPU ranks are covered by skein_b200.parallel.local)")
        if pp > 1:
            pp_info = (pp_ranks, pp_group)
    engine = build_engine(art, rank, device, comm, args, comm_moe, pp_info)
    control = ControlPlane(control_group, rank)
    tok = Tokenizer(art.cfg.vocab_size, art.tokenizer_path())
    rc = 0
    if rank != 0:
        follower_loop(engine, control)
    else:
        driver = DistributedDriver(engine, control).start()
        try:
            if args.prompt is not None or args.demo_prompts:
                prompts = [args.prompt] if args.prompt is not None else [p for p in args.demo_prompts.split("|") if p]
                t0 = time.perf_counter()
                subs = [driver.submit(tok.encode(p), args.max_new_tokens) for p in prompts]
                results, first = [], None
                for rid, kind, reason, q in subs:
                    toks = []
                    while q is not None:
                        ev = q.get()
                        if first is None:
                            first = time.perf_counter() - t0
                        if ev.error is None:
                            toks.append(ev.token)
                        if ev.is_final:
                            break
                    results.append(toks)
                dt = time.perf_counter() - t0
                n = sum(len(r) for r in results)
                print(json.dumps({"generated": results, "text": [tok.decode(r) for r in results], "ttft_ms": round((first or 0) * 1e3, 2),
                                  "tokens_per_s": round(n / dt, 2), "tpot_p99_ms": engine.metrics.tpot_p99()}))
            else:
                from aiohttp import web

                from ..runtime.server import build_app
                web.run_app(build_app(driver, tok), host="0.0.0.0", port=args.port, print=None)
        finally:
            driver.stop()
    if world > 1:
        dist.barrier()
        for c in (comm, comm_moe):
            if c is not None:
                c.close()
        dist.destroy_process_group()
    if beat is not None:
        beat.stop()
    return rc


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="skein-worker")
    ap.add_argument("--artifact", required=True)
    ap.add_argument("--workload", default=None)
    ap.add_argument("--cost", default=None)
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--total-kv-bytes", type=int, default=0)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--demo-prompts", default=None)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--rendezvous", default="/tmp/skein_rendezvous")
    ap.add_argument("--max-batch", type=int, default=0)
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--cpu", action="store_true")
    return ap.parse_args(argv)


if __name__ == "__main__":
    sys.exit(run_rank(parse()))
