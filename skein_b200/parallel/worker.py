"""Rank worker: one process per GPU. Loads its shard of an artifact, joins the group, and either serves HTTP
(rank 0 hosts the front end and broadcasts the request stream) or runs a generation job.

Every rank runs the same Engine on the same inputs: rank 0 is the only one that sees clients; each
scheduler iteration it announces {clock, has payload} through a shared-memory control page and broadcasts
the payload (new requests, stop, hot swap) over a CPU (gloo) group only when there is one; all ranks apply
it, step, and agree on whether the step failed anywhere (runtime/driver.py). Data-plane traffic (the fused
collectives) never touches the host.

Counterpart of RankServer::bootstrap / run_rank (crates/skein_runtime/src/distributed/gpu_rank.rs:104-410,
crates/skein_cli/src/cmd/serve.rs:322), with the HTTP server in front of the multi-GPU workers instead
of a single-process executor.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

from ..compile.artifact import Artifact
from ..models.decoder import Decoder
from ..runtime.driver import EngineDriver, LocalControl, SharedControl, follower_loop
from ..runtime.engine import Engine, EngineConfig, SamplingParams
from ..runtime.tokenizer import Tokenizer
from . import launcher


def size_kv_pool(art: Artifact, lay, device, total_kv_bytes: int, page_size: int = 16, reserve_frac: float = 0.08,
                 bytes_per_token: int = 0) -> int:
    """Pages in the per-layer pool: from an explicit byte budget (with the model's KV bytes per token on this rank,
    or the caller's `bytes_per_token`), else from the memory left after the weights."""
    cfg = art.cfg
    n_layers = len(lay.stage_layers(cfg.num_layers))
    kv_heads = cfg.num_kv_heads // lay.tp
    page_bytes = 2 * kv_heads * page_size * cfg.head_dim * 2 * n_layers
    if bytes_per_token > 0:
        page_bytes = bytes_per_token * page_size
    if total_kv_bytes > 0:
        return max(8, total_kv_bytes // page_bytes)
    if device.type != "cuda":
        return 256
    free, total = torch.cuda.mem_get_info(device)
    return max(8, int((free - reserve_frac * total) // page_bytes))


def prefill_slice_for_slo(tpot_ms: float, decode_us_at_b1: float, batch_exponent: float, max_batch: int, prefill_per_token_us: float,
                          max_prefill_tokens: int) -> int:
    """Prompt tokens a step may carry while other sequences decode, so that the step (the decode of a full batch plus the
    slice) stays within the TPOT target: what is left of the target after the estimated decode step, divided by the
    estimated prefill time per token, in multiples of 256 tokens between 256 and the engine's prefill limit."""
    step_ms = decode_us_at_b1 * max(1, max_batch) ** batch_exponent / 1e3
    room_us = max(0.0, tpot_ms - step_ms) * 1e3
    n = int(room_us / max(prefill_per_token_us, 1e-3)) // 256 * 256
    return max(256, min(int(max_prefill_tokens), n))


def build_engine(art: Artifact, rank: int, device, comm, args, comm_moe=None, pp_info=None) -> Engine:
    lay = art.layout(rank)
    art.check_lowering(rank)
    tuned = art.path / "cache" / "kernel_configs.json"
    if tuned.exists() and device.type == "cuda":
        from ..ops import tuning
        tuning.activate(tuning.KernelConfigCache(tuned, strict=False))   # measured configurations win over the heuristics
    weights = art.load_weights(rank, device)
    pages = size_kv_pool(art, lay, device, args.total_kv_bytes, bytes_per_token=getattr(args, "bytes_per_token", 0))
    pages = min(pages, max(8, (args.max_seq_len // 16 + 1) * max(1, args.max_batch or art.plan["batching"]["max_batch"]) * 2))
    dec = Decoder(art.cfg, weights, lay, num_pages=pages, page_size=art.plan["kv"]["layout"].get("page_size", 16),
                  max_pos=min(args.max_seq_len, art.cfg.max_position_embeddings), comm=comm, comm_moe=comm_moe)
    # Pure expert parallelism decodes with data-parallel attention: every rank attends over its own share of the step's
    # sequences and the MoE blocks exchange tokens over peer memory (SKEIN_EP_DP_ATTENTION=0: attention over all
    # sequences on every rank, the expert outputs all-reduced).
    if (device.type == "cuda" and comm_moe is not None and comm_moe.mode != "nccl" and lay.ep > 1 and lay.tp == 1 and pp_info is None
            and art.cfg.is_moe and os.environ.get("SKEIN_EP_DP_ATTENTION", "1") != "0"):
        dec.dp_attention = True
        if dec.dp_rows_limit(device) == 0:      # e.g. the fused router is switched off: nothing to dispatch from
            dec.dp_attention = False
    if pp_info is not None:
        from .pp import PipelineStage
        dec = PipelineStage(dec, lay, *pp_info[:2])
        dec.feedback_group = pp_info[2] if len(pp_info) > 2 else None
    batching = art.plan["batching"]
    fused = all(c is None or c.mode != "nccl" for c in (comm, comm_moe))
    ecfg = EngineConfig(max_batch=args.max_batch or batching["max_batch"], chunk_tokens=batching.get("chunk_tokens", 0),
                        prefix_cache=art.plan["execution"]["prefix_cache"]["enable"],
                        # stage-to-stage NCCL p2p and library collectives are launched eagerly, never captured
                        use_graphs=(device.type == "cuda" and art.plan["execution"]["cuda_graphs"]["enable"] and fused
                                    and pp_info is None and not getattr(args, "no_cuda_graphs", False)))
    ecfg.warm_graphs = ecfg.use_graphs      # every batch bucket is captured while the server starts, not under load
    # a checkpoint that ships its tokenizer is a real model: its generations end at the model's end-of-sequence token
    # (an artifact without one is driven with byte tokens and random weights, where no token means "stop")
    if art.tokenizer_path() is not None and not getattr(args, "ignore_eos", False):
        ecfg.eos_token = art.cfg.eos_token_id
    # pipeline parallelism: one group of sequences per stage kept in flight across engine steps instead of a pipeline
    # drained at the end of every step
    ecfg.pp_continuous = pp_info is not None and os.environ.get("SKEIN_PP_CONTINUOUS", "0") == "1"
    if args.workload:
        from .. import core
        text = open(args.workload).read()
        w = core.workload_parse(text)
        ecfg.ttft_ms, ecfg.tpot_ms = w["ttft_p95_ms"], w["tpot_p95_ms"]
        # the prompt lengths the plan was extracted for are the baseline of the workload drift monitor
        lens = [json.loads(l).get("prompt_tokens") for l in text.splitlines()[1:] if l.strip()]
        ecfg.drift_baseline = tuple(int(x) for x in lens if x)
        ecfg.drift_threshold_kl = float(w.get("recompile_drift_threshold_kl", ecfg.drift_threshold_kl))
    est = art.path / "runtime_estimator.json"
    if est.exists() and not args.cost:
        # the latency estimator that `compile` derived from the cost model for this plan and cluster
        c = json.loads(est.read_text())
        ecfg.decode_us_at_b1 = c.get("per_token_decode_us_at_b1", ecfg.decode_us_at_b1)
        ecfg.batch_exponent = c.get("batch_scaling_exponent", ecfg.batch_exponent)
        ecfg.prefill_per_token_us = c.get("prefill_per_token_us", ecfg.prefill_per_token_us)
        if args.workload:
            ecfg.interleave_prefill_tokens = prefill_slice_for_slo(ecfg.tpot_ms, ecfg.decode_us_at_b1, ecfg.batch_exponent, ecfg.max_batch,
                                                                   ecfg.prefill_per_token_us, ecfg.max_prefill_tokens)
    if args.cost:
        from .. import core
        c = json.loads(core.cost_constants_json(open(args.cost).read())).get("runtime_estimator", {})
        ecfg.decode_us_at_b1 = c.get("per_token_decode_us_at_b1", ecfg.decode_us_at_b1)
        ecfg.batch_exponent = c.get("batch_scaling_exponent", ecfg.batch_exponent)
        ecfg.prefill_per_token_us = c.get("prefill_per_token_us", ecfg.prefill_per_token_us)
    return Engine(dec, ecfg)


def make_resync(comms):
    """Re-arm the fused communicators after a step that failed on any rank: behind a barrier (no rank is still
    launching), every rank zeroes its flag words, epochs and arrival counters and clears its device status, so that
    all ranks start the next step from the same epoch. A rank that is really gone makes the barrier time out, the
    process exits and the launcher restarts the group."""
    comms = [c for c in comms if c is not None]

    def resync(control):
        import torch as _t
        control.barrier()
        if _t.cuda.is_available():
            _t.cuda.synchronize()
        for c in comms:
            c.reset()
        if comms:
            from .. import ops
            ops.workspace().reset_after_error()
            _t.cuda.synchronize()
        control.barrier()
    return resync


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
            # the published buffers hold the partials of one prefill chunk (its expert-sorted rows for a MoE model)
            rows = max(512, 8192 * max(1, art.cfg.top_k if art.cfg.is_moe else 1))
            if tp > 1:
                # in-switch reduction (6 % of a step at 8 ranks) stays opt-in for a server (SKEIN_MULTIMEM=1): a rank that dies
                # while its heap is bound to a multicast object takes its peers' GPUs with it, and a server must survive a rank
                comm = TPComm(tp_group, device, hidden=art.cfg.hidden_size, fused_rows=rows)
            if ep > 1:
                comm_moe = TPComm(stage_group, device, hidden=art.cfg.hidden_size, fused_rows=rows)
        elif tp > 1 or ep > 1:
            raise SystemExit("tensor/expert-parallel serving needs GPUs (CPU ranks are covered by skein_b200.parallel.local)")
        if pp > 1:
            pp_info = (pp_ranks, pp_group, pp_mod.make_feedback_group(art.layout_dims, rank))
    engine = build_engine(art, rank, device, comm, args, comm_moe, pp_info)
    if beat is not None:
        beat.step_started_at = lambda: engine.step_started_at     # a rank stuck inside a step stops beating
    if world > 1:
        control = SharedControl(str(rdv) + ".control", rank, world, control_group)
    else:
        control = LocalControl()
    resync = make_resync([comm, comm_moe]) if world > 1 else None
    tok = Tokenizer(art.cfg.vocab_size, art.tokenizer_path())
    sampling = SamplingParams(args.temperature, args.top_k, args.top_p, args.seed) if args.temperature > 0 else None
    rc = 0
    if rank != 0:
        follower_loop(engine, control, rank, resync)
    else:
        driver = EngineDriver(engine, control, rank=0, resync=resync).start()
        try:
            if args.prompt is not None or args.demo_prompts:
                prompts = [args.prompt] if args.prompt is not None else [p for p in args.demo_prompts.split("|") if p]
                if args.speculative_draft and world == 1:
                    print(json.dumps(_speculative_job(art, engine, tok, prompts, args, device)))
                else:
                    print(json.dumps(_generation_job(driver, engine, tok, prompts, args.max_new_tokens, sampling)))
            else:
                from aiohttp import web

                from ..runtime.server import build_app
                hs = None
                if args.enable_hot_swap:
                    from ..runtime.hotswap import HotSwap
                    hs = HotSwap(driver, art, rank=0)
                web.run_app(build_app(driver, tok, hs, art.path.parent), host="0.0.0.0", port=args.port, print=None)
        finally:
            driver.stop()
    control.close()
    if world > 1:
        dist.barrier()
        for c in (comm, comm_moe):
            if c is not None:
                c.close()
        dist.destroy_process_group()
    if beat is not None:
        beat.stop()
    return rc


def _generation_job(driver, engine, tok, prompts, max_new_tokens, sampling=None) -> dict:
    """Submit every prompt, collect the streams (the reference's multi-GPU generation job,
    crates/skein_runtime/src/distributed/gpu_rank.rs:724-877)."""
    t0 = time.perf_counter()
    subs = [driver.submit(tok.encode(p), max_new_tokens, sampling) for p in prompts]
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
    return {"generated": results, "text": [tok.decode(r) for r in results], "ttft_ms": round((first or 0) * 1e3, 2),
            "tokens_per_s": round(n / dt, 2), "tpot_p99_ms": engine.metrics.tpot_p99()}


def _speculative_job(art, engine, tok, prompts, args, device) -> dict:
    """Generation with a draft model proposing `--speculative-k` tokens per verification step of the target
    (runtime/speculative.py; the reference's run_speculative_generation, distributed/gpu_rank.rs:2197)."""
    from ..runtime.speculative import SpeculativeDecoder
    draft_art = Artifact(args.speculative_draft)
    draft = Decoder(draft_art.cfg, draft_art.load_weights(0, device), draft_art.layout(0), num_pages=engine.dec.num_pages,
                    page_size=engine.dec.page_size, max_pos=engine.dec.max_pos)
    spec = SpeculativeDecoder(engine.dec, draft, k=args.speculative_k)
    t0 = time.perf_counter()
    results, stats = [], {"proposed": 0, "accepted": 0, "target_steps": 0}
    for p in prompts:
        out, st = spec.generate(tok.encode(p), args.max_new_tokens, temperature=args.temperature, seed=args.seed)
        results.append(out)
        for k in stats:
            stats[k] += st[k]
    dt = time.perf_counter() - t0
    n = sum(len(r) for r in results)
    return {"generated": results, "text": [tok.decode(r) for r in results], "tokens_per_s": round(n / dt, 2),
            "speculative": dict(stats, acceptance=round(stats["accepted"] / max(1, stats["proposed"]), 3))}


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
    ap.add_argument("--bytes-per-token", type=int, default=0)
    ap.add_argument("--enable-hot-swap", action="store_true")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--speculative-draft", default=None)
    ap.add_argument("--speculative-k", type=int, default=4)
    return ap.parse_args(argv)


if __name__ == "__main__":
    sys.exit(run_rank(parse()))
