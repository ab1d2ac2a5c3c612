"""Bodies of the `skein` sub-commands. Each returns a process exit code and reports through `emit`."""
from __future__ import annotations

import json
import os
import time
from collections import Counter
from pathlib import Path

from .. import core


def _read(p) -> str:
    return Path(p).read_text()


def _search_options(args) -> dict:
    o = {"objective": getattr(args, "objective", "latency")}
    for env, key in (("SKEIN_FORCE_TP", "force_tp"), ("SKEIN_FORCE_PP", "force_pp"), ("SKEIN_FORCE_EP", "force_ep"), ("SKEIN_FORCE_BATCH", "force_batch")):
        if os.environ.get(env):
            o[key] = int(os.environ[env])
    return o


def _plan_summary(plan: dict) -> dict:
    dm = Counter((d["weight"], d["activation"], d["kv_cache"]) for d in plan["dtype_map"]["per_layer"])
    return {"parallelism": plan["parallelism"], "kv": plan["kv"], "batching": plan["batching"],
            "dtype_histogram": {"/".join(k): v for k, v in sorted(dm.items())},
            "cuda_graphs": plan["execution"]["cuda_graphs"]["enable"], "disaggregated": plan["disaggregation"] is not None}


def cmd_extract(args, emit) -> int:
    t0 = time.time()
    ins = (_read(args.model), _read(args.cluster), _read(args.trace), _read(args.drift), _read(args.cost))
    if args.disaggregate_decode_devices:
        r = core.extract_disaggregated_plan(*ins, args.disaggregate_decode_devices, _search_options(args))
    else:
        r = core.extract_plan(*ins, _search_options(args))
    Path(args.out).write_text(r["plan_json"])
    plan = json.loads(r["plan_json"])
    tok_s = plan["batching"]["max_batch"] / max(r["cost_us"], 1e-9) * 1e6      # every sequence of a full batch gains a token per step
    report = {"plan_path": str(args.out), "content_hash": r["content_hash"], "cost_us": r["cost_us"], "predicted_tokens_per_s": round(tok_s, 1),
              "objective": getattr(args, "objective", "throughput"), "search": json.loads(r["counters_json"]),
              "summary": _plan_summary(plan), "wall_s": round(time.time() - t0, 3)}
    s = report["summary"]
    emit(args, report, f"plan written to {args.out}\n  hash        {r['content_hash']}\n  cost        {r['cost_us']:.1f} us per decode step"
                       f" ({tok_s:.0f} tokens/s at a full batch; objective: {report['objective']})\n"
                       f"  placement   tp={s['parallelism']['tp']} pp={s['parallelism']['pp']} ep={s['parallelism']['ep']}\n"
                       f"  batching    {s['batching']}\n  kv          {s['kv']}\n  dtypes      {s['dtype_histogram']}\n"
                       f"  search      {report['search']}")
    return 0


def cmd_compile(args, emit) -> int:
    from ..compile.pipeline import compile_model

    prompts = None
    if args.parity_prompts_path:
        prompts = [json.loads(l)["tokens"] for l in _read(args.parity_prompts_path).splitlines() if l.strip()]
    r = compile_model(_read(args.model), _read(args.cluster), _read(args.trace), _read(args.drift), _read(args.cost), args.out,
                      weights=args.weights, options=_search_options(args), n_parity_prompts=args.n_parity_prompts, prompts=prompts,
                      enforce_parity=args.enforce_parity, seed=args.seed, search_budget=args.search_budget)
    if r.replans:
        Path(args.drift).write_text(r.drift_toml)    # the feedback edge: the next extract sees the raised entries
    rep = r.report
    payload = {"artifact": str(r.artifact_dir), "content_hash": r.artifact_dir.name, "summary": _plan_summary(r.plan), "replans": r.replans,
               "parity": None if rep is None else {"passed": rep.passed, "avg_final_kl": rep.avg_final_kl, "failing_layers": len(rep.failing)}}
    emit(args, payload, f"artifact {r.artifact_dir}\n  parity      {'skipped' if rep is None else ('passed' if rep.passed else 'FAILED')}"
                        f"{'' if rep is None else f' (avg final KL {rep.avg_final_kl:.3g})'}\n  re-plans    {r.replans}")
    return 0


def cmd_verify(args, emit) -> int:
    import torch

    from ..compile import parity
    from ..compile.artifact import Artifact
    from ..compile.pipeline import default_parity_prompts

    art = Artifact(args.artifact)
    if args.tokens_file:
        prompts = [json.loads(l)["tokens"] if l.strip().startswith("{") else [int(t) for t in l.split()] for l in _read(args.tokens_file).splitlines() if l.strip()]
    elif args.sample_from:
        prompts = [json.loads(l)["tokens"] for l in _read(args.sample_from).splitlines() if l.strip()][:args.n_prompts]
    else:
        prompts = default_parity_prompts(art.cfg, min(args.n_prompts, 8))
    cand = parity.ArtifactForward(art, args.device)
    if args.dump_only:
        dump_dir = Path(os.environ.get("SKEIN_DUMP_DIR", "."))
        dump_dir.mkdir(parents=True, exist_ok=True)
        for i, p in enumerate(prompts):
            _, lg = cand.run(p)
            torch.save(lg, dump_dir / f"logits_{i}.pt")
        emit(args, {"dumped": len(prompts), "dir": str(dump_dir)}, f"dumped {len(prompts)} logit vectors to {dump_dir}")
        return 0
    ref_art = Artifact(args.reference) if args.reference else Artifact(art.path / "reference_bf16")
    if args.hf_reference:
        if args.reference_dtype not in ("bfloat16", "float32"):
            raise ValueError("reference dtype must be bfloat16 or float32")
        reference = None
        if args.hf_checkpoint:      # HuggingFace transformers on the original checkpoint: the outside oracle
            reference = parity.HFForward(args.hf_checkpoint, args.reference_dtype)
        if reference is None:       # no checkpoint given: the in-process dense model on the artifact's bf16 weights
            refw = ref_art.load_full_weights(args.device)
            reference = parity.DenseForward(art.cfg, refw)
    else:
        reference = parity.ArtifactForward(ref_art, args.device)
    tol = json.loads(core.cost_constants_json(_read(args.cost))).get("parity_tolerance_mse", {})
    rep = parity.verify(cand, reference, prompts, art.plan, args.max_accuracy_drift, tol)
    (art.path / "parity_report.json").write_text(rep.to_json())
    emit(args, json.loads(rep.to_json()), f"parity {'passed' if rep.passed else 'FAILED'}: avg final KL {rep.avg_final_kl:.3g} "
                                          f"(limit {rep.max_accuracy_drift:g}), {len(rep.failing)} failing layers over {rep.prompts} prompts")
    return 1 if (args.enforce and not rep.passed) else 0


def cmd_serve(args, emit) -> int:
    from ..parallel import launcher, worker

    argv = ["--artifact", args.artifact, "--port", str(args.port), "--total-kv-bytes", str(args.total_kv_bytes), "--max-new-tokens",
            str(args.max_new_tokens), "--rendezvous", args.rendezvous, "--max-batch", str(args.max_batch), "--max-seq-len", str(args.max_seq_len),
            "--bytes-per-token", str(args.bytes_per_token), "--temperature", str(args.temperature), "--top-k", str(args.top_k),
            "--top-p", str(args.top_p), "--seed", str(args.seed)]
    if args.enable_hot_swap:
        argv.append("--enable-hot-swap")
    if not args.cuda_graphs:
        argv.append("--no-cuda-graphs")
    if getattr(args, "ignore_eos", False):
        argv.append("--ignore-eos")
    if args.speculative_draft:
        argv += ["--speculative-draft", args.speculative_draft, "--speculative-k", str(args.speculative_k)]
    for flag, val in (("--workload", args.workload), ("--cost", args.cost), ("--prompt", args.prompt), ("--demo-prompts", args.demo_prompts)):
        if val is not None:
            argv += [flag, val]
    if args.batch_demo and not args.demo_prompts and args.prompt is None:
        argv += ["--demo-prompts", "The quick brown fox|Blackwell tensor cores|Paged attention is"]
    if launcher.world_from_env() is None and args.gpus:
        gpus = launcher.parse_gpus(args.gpus)
        failed = launcher.launch_ranks(gpus, args.rendezvous, argv, restarts=max(0, args.restarts))
        emit(args, {"ranks": len(gpus), "failed": failed}, f"{len(gpus)} ranks finished, {failed} failed")
        return 1 if failed else 0
    return worker.run_rank(worker.parse(argv))


def cmd_calibrate(args, emit) -> int:
    import torch

    from .. import calibrate as cal

    corpus = cal.Corpus.from_toml(_read(args.corpus))
    cost_text = _read(args.out_cost)
    consts = json.loads(core.cost_constants_json(cost_text))
    if args.hardware not in consts["peak_tflops"]:
        raise ValueError(f"no [peak_tflops.{args.hardware}] table in {args.out_cost}")
    eff, drift = {}, {}
    if torch.cuda.is_available():
        eff = cal.calibrate_kernels(corpus, consts["peak_tflops"][args.hardware]["bf16"], consts.get("hbm_gbps", {}).get(args.hardware, 6552.0))
        hbm = consts.get("hbm_gbps", {}).get(args.hardware, 6552.0)
        stream = cal.measure_stream_efficiency(hbm) if "stream_efficiency" in consts else None
        Path(args.out_cost).write_text(cal.write_cost_constants(cost_text, eff, stream_efficiency=stream))
    fitted = {}
    if getattr(args, "fit_step_ms", None) is not None:
        if not (args.fit_plan and args.fit_cluster):
            raise ValueError("--fit-step-ms needs --fit-plan and --fit-cluster")
        pp_ = Path(args.fit_plan)
        plan_text = _read(pp_ / "plan.json") if pp_.is_dir() else _read(pp_)
        cost_now = _read(args.out_cost)
        fitted = cal.fit_fixed_costs(plan_text, _read(args.model), _read(args.fit_cluster), cost_now, args.fit_step_ms, args.fit_kv_tokens)
        Path(args.out_cost).write_text(cal.rewrite_toml_values(cost_now, fitted))
    if args.candidate_artifact:
        from ..compile import parity
        from ..compile.artifact import Artifact
        from ..compile.pipeline import default_parity_prompts
        art = Artifact(args.candidate_artifact)
        ref = Artifact(args.reference_artifact) if args.reference_artifact else Artifact(art.path / "reference_bf16")
        if args.drift_prompts_path:     # JSONL of {"tokens": [...]}: the prompts the drift entries are measured on
            prompts = [json.loads(l)["tokens"] for l in _read(args.drift_prompts_path).splitlines() if l.strip()][:corpus.n_drift_prompts]
        else:
            prompts = default_parity_prompts(art.cfg, min(corpus.n_drift_prompts, 8), seed=corpus.sampling_seed)
        rep = parity.verify(parity.ArtifactForward(art), parity.ArtifactForward(ref), prompts, art.plan, 1.0, consts.get("parity_tolerance_mse", {}))
        drift = cal.calibrate_drift(json.loads(rep.to_json())["layers"], art.plan)
        name = Path(args.model).stem.replace("_config", "")
        dpath = Path(args.out_drift_dir) / f"{name}_drift.toml"
        dpath.write_text(cal.write_drift_table(_read(dpath), drift))
    tuned = {}
    if getattr(args, "autotune", False) and torch.cuda.is_available():
        from ..compile.artifact import Artifact
        from ..models.config import ModelConfig
        art = Artifact(args.candidate_artifact) if args.candidate_artifact else None
        cfg = art.cfg if art is not None else ModelConfig.from_file(args.model)
        tp = int(art.plan["parallelism"]["tp"]) if art is not None else 1
        out = args.autotune_out or (art.path / "cache" / "kernel_configs.json" if art is not None else "kernel_configs.json")
        tuned = cal.autotune_decode_gemms(cfg, tp, args.autotune_batch, out)
    emit(args, {"efficiencies": {f"{k[0]}.{k[1]}": v for k, v in eff.items()}, "drift_entries": len(drift),
                "tuned_gemms": tuned, "fitted": {".".join(x for x in k if x): v for k, v in fitted.items()}},
         f"calibrated {len(eff)} kernel efficiencies, {len(drift)} drift entries, {len(tuned)} tuned GEMM shapes")
    return 0


def bench_collectives(emit, args) -> int:
    """Time the stand-alone all-reduce (publish + peer pull) against the library all-reduce for decode-sized messages.

    Run under `python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m skein_b200 bench
    --collectives`: one process per GPU. CUDA events on the launching stream, 20 launches per sample, max over ranks. Counterpart of the reference's
    SKEIN_ALLREDUCE_BENCH (crates/skein_runtime/src/cuda/nccl.rs: bench_all_reduce)."""
    import datetime

    import torch
    import torch.distributed as dist

    from .. import ops
    from ..parallel.tp import TPComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2 or not torch.cuda.is_available():
        raise ValueError("--collectives needs one process per GPU: launch with torch.distributed.run, 2 or more ranks")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    hidden = 4096
    comm = TPComm(dist.group.WORLD, dev, hidden=hidden, fused_rows=512, mode="fused")
    def timed(fn, n=20):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    rows_out = []
    for rows in (16, 64, 128, 256, 512):
        x = torch.randn(rows, hidden, device=dev).bfloat16()
        y = x.clone()
        fused_us = timed(lambda: comm.all_reduce(x))
        nccl_us = timed(lambda: dist.all_reduce(y))
        # the way the serving path runs it: 20 all-reduces captured into one CUDA graph (no host launch cost)
        comm.all_reduce(x)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                comm.all_reduce(x)
        graph_us = timed(g.replay, n=5) / 20
        rows_out.append({"rows": rows, "bytes": rows * hidden * 2, "fused_eager_us": round(fused_us, 2),
                         "fused_graph_us": round(graph_us, 2), "nccl_eager_us": round(nccl_us, 2)})
    # the other pull collectives at one decode-sized message (64 rows per rank): in a CUDA graph vs the library, eager
    others = {}
    rows = 64 * world
    x = torch.randn(rows, hidden, device=dev).bfloat16()
    shard = x[:64].contiguous()
    lib_out = {"all_gather": torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16),
               "reduce_scatter": torch.empty(64, hidden, device=dev, dtype=torch.bfloat16), "all_to_all": torch.empty_like(x)}
    cases = {"all_gather": (lambda: comm.all_gather(shard), lambda: dist.all_gather_into_tensor(lib_out["all_gather"], shard)),
             "reduce_scatter": (lambda: comm.reduce_scatter(x), lambda: dist.reduce_scatter_tensor(lib_out["reduce_scatter"], x)),
             "all_to_all": (lambda: comm.all_to_all(x), lambda: dist.all_to_all_single(lib_out["all_to_all"], x))}
    for name, (ours, lib) in cases.items():
        ours()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                ours()
        others[name] = {"rows_per_rank": 64, "pull_graph_us": round(timed(g.replay, n=5) / 20, 2),
                        "pull_eager_us": round(timed(ours), 2), "nccl_eager_us": round(timed(lib), 2)}
    torch.cuda.synchronize()
    ops.workspace().check_status()
    if dist.get_rank() == 0:
        emit(args, {"world": world, "hidden": hidden, "all_reduce": rows_out, **others},
             "\n".join([f"{r['rows']:4d} rows ({r['bytes']} B): fused {r['fused_eager_us']} us eager / {r['fused_graph_us']} us "
                        f"in a CUDA graph, nccl {r['nccl_eager_us']} us eager" for r in rows_out]
                       + [f"{k}: pull {v['pull_eager_us']} us eager / {v['pull_graph_us']} us in a CUDA graph, nccl "
                          f"{v['nccl_eager_us']} us eager" for k, v in others.items()]))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def bench_over_http(args, emit) -> int:
    """Replay a trace against a running server (`skein serve`, any number of GPUs behind it) over HTTP with SSE token
    streams: arrival times honoured (scaled by --time-scale), one connection per request, TTFT and inter-token times
    measured at the client. This is how a multi-GPU artifact is benchmarked end to end."""
    import asyncio

    import aiohttp
    import torch

    lines = [json.loads(l) for l in _read(args.workload).splitlines() if l.strip()]
    slo, reqs = lines[0]["slo"], lines[1:]
    if args.max_requests:
        reqs = reqs[:args.max_requests]
    g = torch.Generator().manual_seed(0)
    vocab = args.vocab_size
    max_ctx = args.max_seq_len
    stats = {"ok": 0, "rejected": 0, "failed": 0, "tokens": 0, "ttft": [], "gaps": []}

    async def one(session, r, t0):
        await asyncio.sleep(max(0.0, r["arrival_ms"] / 1000.0 / args.time_scale - (time.monotonic() - t0)))
        n_out = int(r["output_tokens"])
        n_prompt = max(1, min(int(r["prompt_tokens"]), max_ctx - n_out - 1))
        ids = torch.randint(0, vocab, (n_prompt,), generator=g).tolist()
        t_send = time.monotonic()
        try:
            async with session.post(args.url.rstrip("/") + "/v1/completions", json={"prompt": ids, "max_tokens": n_out, "stream": True}) as resp:
                if resp.status == 429:
                    stats["rejected"] += 1
                    return
                if resp.status != 200:
                    stats["failed"] += 1
                    return
                last, n, err = None, 0, False
                async for raw in resp.content:
                    line = raw.decode().strip()
                    if not line.startswith("data: "):
                        continue
                    ev = json.loads(line[6:])
                    now = time.monotonic()
                    if ev.get("error"):
                        err = True
                        break
                    n += 1
                    if last is None:
                        stats["ttft"].append((now - t_send) * 1e3)
                    else:
                        stats["gaps"].append((now - last) * 1e3)
                    last = now
                stats["tokens"] += n
                stats["failed" if err else "ok"] += 1
        except aiohttp.ClientError:
            stats["failed"] += 1

    async def run():
        t0 = time.monotonic()
        conn = aiohttp.TCPConnector(limit=0)
        async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=None)) as session:
            await asyncio.gather(*[one(session, r, t0) for r in reqs])
        return time.monotonic() - t0

    wall = asyncio.run(run())
    q = lambda xs, f: (sorted(xs)[min(len(xs) - 1, int(f * len(xs)))] if xs else None)
    ttft_p50, ttft_p95, tpot_p99 = q(stats["ttft"], 0.5), q(stats["ttft"], 0.95), q(stats["gaps"], 0.99)
    meets = ttft_p95 is not None and ttft_p95 <= slo["ttft_p95_ms"] and (tpot_p99 is None or q(stats["gaps"], 0.95) <= slo["tpot_p95_ms"])
    out = {"url": args.url, "throughput_tok_s": round(stats["tokens"] / wall, 2), "goodput_req_s": round((stats["ok"] if meets else 0) / wall, 3),
           "requests_ok": stats["ok"], "requests_rejected": stats["rejected"], "requests_failed": stats["failed"],
           "ttft_p50_ms": None if ttft_p50 is None else round(ttft_p50, 2), "ttft_p95_ms": None if ttft_p95 is None else round(ttft_p95, 2),
           "tpot_p99_ms": None if tpot_p99 is None else round(tpot_p99, 3), "wall_s": round(wall, 2), "baseline": args.baseline}
    out = _select_metrics(args, out)
    emit(args, out, "\n".join(f"{k:20s} {v}" for k, v in out.items()))
    return 0


def bench_op_profile(args, emit) -> int:
    """One decode step of the artifact's batch size, launched kernel by kernel with CUDA events around every operator:
    the per-operator table (calls, device time, share, host time per launch) of a served step."""
    import torch

    from ..compile.artifact import Artifact
    from ..parallel import worker
    from ..utils.op_profile import OpProfiler

    art = Artifact(args.artifact)
    if art.num_devices != 1 or not torch.cuda.is_available():
        raise ValueError("--op-profile runs a single-GPU artifact on a GPU")
    device = torch.device("cuda", 0)
    eng = worker.build_engine(art, 0, device, None, worker.parse(["--artifact", args.artifact]))
    B = eng.cfg.max_batch
    g = torch.Generator().manual_seed(0)
    n_prompt = max(1, min(64, eng.dec.max_pos // 2))
    for _ in range(B):
        eng.submit(torch.randint(0, art.cfg.vocab_size, (n_prompt,), generator=g).tolist(), 8)
    while eng.batcher.inflight_len and not all(eng.batcher.request_info(i)["phase"] == "decode" for i in eng.batcher.inflight_ids()):
        eng.step()
    ids = eng.batcher.inflight_ids()
    bk = eng.runner.bucket(len(ids))
    eng.runner.stage_decode_inputs(bk, eng.batcher, ids)
    bk.dev_in.copy_(bk.host_in)
    eng.runner._decode_body(bk, False)            # warm-up (descriptor caches, workspaces)
    bk.dev_in.copy_(bk.host_in)
    with OpProfiler() as prof:
        eng.runner._decode_body(bk, False)
    sm = prof.summary()
    emit(args, {"batch": len(ids), "operators": sm}, prof.table())
    return 0


_BENCH_METRIC_KEYS = {"throughput": ("throughput_tok_s",), "goodput": ("goodput_req_s",), "drift_compliance": ("drift_compliance",)}


def _select_metrics(args, out: dict) -> dict:
    """--metrics throughput,goodput,drift_compliance: the headline figures to report; counts, latencies and the wall time
    always come along. An unknown name is an error before anything runs (cmd_bench checks it first)."""
    want = [m.strip() for m in str(getattr(args, "metrics", "") or "").split(",") if m.strip()]
    drop = {k for name, keys in _BENCH_METRIC_KEYS.items() if name not in want for k in keys}
    return {k: v for k, v in out.items() if k not in drop}


def cmd_bench(args, emit) -> int:
    """Replay a trace (arrival times honoured, scaled by --time-scale) against a single-process engine, or with --url
    against a running server over HTTP."""
    import torch

    if getattr(args, "collectives", False):
        return bench_collectives(emit, args)
    unknown = [m.strip() for m in str(getattr(args, "metrics", "") or "").split(",") if m.strip() and m.strip() not in _BENCH_METRIC_KEYS]
    if unknown:
        raise ValueError(f"--metrics: unknown metric(s) {unknown}; known: {sorted(_BENCH_METRIC_KEYS)}")
    if getattr(args, "synth", None):
        # the synthetic workloads of the planner tests and of the serving benchmarks, as a trace file
        n, seed = int(args.synth_requests), int(args.synth_seed)
        text = (core.synth_uniform_trace(n, seed, 128, 2048, 64, 512, 4.0) if args.synth == "uniform"
                else core.synth_burst_trace(n, seed, 50.0, 2.0, 10.0, 600.0, 8192, 32, 1024))
        import tempfile
        path = args.write_trace or tempfile.NamedTemporaryFile("w", suffix=".jsonl", delete=False).name
        Path(path).write_text(text)
        args.workload = path
        if not args.artifact and not getattr(args, "url", None):
            emit(args, {"trace": path, "requests": n, "kind": args.synth, "seed": seed}, f"wrote {n} {args.synth} requests to {path}")
            return 0
    if getattr(args, "url", None):
        if not args.workload:
            raise ValueError("`skein bench --url` needs --workload")
        return bench_over_http(args, emit)
    if getattr(args, "op_profile", False):
        if not args.artifact:
            raise ValueError("`skein bench --op-profile` needs --artifact")
        return bench_op_profile(args, emit)
    if not args.artifact or not args.workload:
        raise ValueError("`skein bench` needs --artifact and --workload (or --collectives under torch.distributed.run)")

    from ..compile.artifact import Artifact
    from ..parallel import worker

    art = Artifact(args.artifact)
    if art.num_devices != 1:
        raise ValueError("this artifact needs several ranks: start it with `skein serve --gpus ...` and run `skein bench --url http://host:port --workload ...`")
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    wargs = worker.parse(["--artifact", args.artifact, "--workload", args.workload])
    eng = worker.build_engine(art, 0, device, None, wargs)
    lines = [json.loads(l) for l in _read(args.workload).splitlines() if l.strip()]
    slo, reqs = lines[0]["slo"], lines[1:]
    if args.max_requests:
        reqs = reqs[:args.max_requests]
    g = torch.Generator().manual_seed(0)
    t0 = time.monotonic()
    pending = list(reqs)
    done_tokens, rejected, first_seen, ttfts = 0, 0, {}, []
    while pending or not eng.idle:
        now = (time.monotonic() - t0) * 1000.0 * args.time_scale
        while pending and pending[0]["arrival_ms"] <= now:
            r = pending.pop(0)
            n_prompt = min(int(r["prompt_tokens"]), eng.dec.max_pos - int(r["output_tokens"]) - 1)
            ids = torch.randint(0, art.cfg.vocab_size, (max(1, n_prompt),), generator=g).tolist()
            rid, d = eng.submit(ids, int(r["output_tokens"]))
            rejected += d.kind == "reject"
            first_seen[rid] = time.monotonic()
        evs = eng.step()
        if not evs:
            time.sleep(0.0005)
        for ev in evs:
            if ev.error is None:
                done_tokens += 1
    wall = time.monotonic() - t0
    text = eng.metrics.render()
    ok = int(next((l.split()[-1] for l in text.splitlines() if l.startswith('skein_requests_total{status="ok"}')), 0))
    ttft_p50, tpot_p99 = eng.metrics.ttft_p50(), eng.metrics.tpot_p99()
    good = ok if (ttft_p50 <= slo["ttft_p95_ms"] and tpot_p99 <= slo["tpot_p95_ms"]) else 0
    rep_path = art.path / "parity_report.json"
    drift_ok = json.loads(rep_path.read_text())["passed"] if rep_path.exists() else None
    out = {"throughput_tok_s": round(done_tokens / wall, 2), "goodput_req_s": round(good / wall, 3), "drift_compliance": drift_ok,
           "requests_ok": ok, "requests_rejected": rejected, "ttft_p50_ms": ttft_p50, "tpot_p99_ms": tpot_p99, "wall_s": round(wall, 2),
           "baseline": args.baseline}
    out = _select_metrics(args, out)
    emit(args, out, "\n".join(f"{k:20s} {v}" for k, v in out.items()))
    return 0
