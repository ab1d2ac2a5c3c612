"""`skein` command line: extract | compile | verify | serve | calibrate | bench.

Flags follow the reference's clap definitions (crates/skein_cli/src/cli.rs:15-239): global `--log-level`
and `--output text|json`; errors are printed to stderr as one JSON object when `--output json`
(crates/skein_cli/src/output.rs:117-190). `bench` is the sub-command the reference's Makefile and a stale
test expect but its CLI never defined (crates/skein_cli/tests/arg_parsing.rs:137-160).
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
from pathlib import Path

log = logging.getLogger("skein")


def _read(p) -> str:
    return Path(p).read_text()


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="skein", description="Blackwell-native LLM serving compiler and runtime")
    ap.add_argument("--log-level", default="info")
    ap.add_argument("--output", default="text", choices=["text", "json"])
    ap.add_argument("--runtime-config", default=None,
                    help="TOML file whose [runtime] table sets the runtime switches (skein_b200/utils/runtime_config.py); "
                         "the environment overrides the file")
    sub = ap.add_subparsers(dest="command", required=True)

    def planner_inputs(p):
        p.add_argument("--model", required=True, help="HuggingFace config.json")
        p.add_argument("--cluster", required=True, help="cluster TOML")
        p.add_argument("--trace", required=True, help="workload trace JSONL (first line: SLO)")
        p.add_argument("--drift", required=True, help="drift table TOML")
        p.add_argument("--cost", required=True, help="cost constants TOML")
        p.add_argument("--objective", default=os.environ.get("SKEIN_OBJECTIVE", "throughput"), choices=["latency", "throughput"],
                       help="throughput (default): least time per generated token among the plans whose decode step meets the "
                            "trace's TPOT SLO, which picks the largest batch that fits; latency: the shortest decode step, "
                            "the reference's objective, which picks batch 1")

    e = sub.add_parser("extract", help="search placement + per-layer dtypes, write plan.json")
    planner_inputs(e)
    e.add_argument("--out", default="plan.json")
    e.add_argument("--disaggregate-decode-devices", type=int, default=0)

    c = sub.add_parser("compile", help="plan, shard weights, write the artifact, run the parity gate")
    planner_inputs(c)
    c.add_argument("--weights", default=None, help="HF safetensors file or directory; omit for seeded random weights")
    c.add_argument("--out", default="artifacts/")
    c.add_argument("--search-budget", type=int, default=100, help="with a GPU present: launch configurations timed per GEMM shape of the decode step; the winners go "
                        "into the artifact's cache/kernel_configs.json (0 = skip the search)")
    c.add_argument("--enforce-parity", action="store_true")
    c.add_argument("--parity-prompts-path", default=None)
    c.add_argument("--n-parity-prompts", type=int, default=8)
    c.add_argument("--seed", type=int, default=0)

    v = sub.add_parser("verify", help="parity of an artifact against its bf16 reference or the dense oracle")
    v.add_argument("--artifact", required=True)
    v.add_argument("--reference", default=None, help="reference artifact (default: <artifact>/reference_bf16)")
    v.add_argument("--sample-from", default=None, help="JSONL of {\"tokens\": [...]} prompts")
    v.add_argument("--n-prompts", type=int, default=50)
    v.add_argument("--cost", default="cluster/cost_constants.toml")
    v.add_argument("--enforce", action="store_true")
    v.add_argument("--hf-reference", action="store_true", help="compare against the cache-free dense oracle on the bf16 weights")
    v.add_argument("--hf-checkpoint", default=None,
                   help="with --hf-reference: checkpoint directory (config.json + safetensors) to run through HuggingFace transformers")
    v.add_argument("--reference-dtype", default="bfloat16")
    v.add_argument("--dump-only", action="store_true")
    v.add_argument("--tokens-file", default=None)
    v.add_argument("--max-accuracy-drift", type=float, default=0.01)
    v.add_argument("--device", default="cpu")

    s = sub.add_parser("serve", help="serve an artifact over HTTP (:8080) or run a generation job")
    s.add_argument("--artifact", required=True)
    s.add_argument("--workload", default=None)
    s.add_argument("--cost", default="cluster/cost_constants.toml")
    s.add_argument("--port", type=int, default=8080)
    s.add_argument("--enable-hot-swap", action="store_true",
                   help="expose POST /admin/hotswap {\"artifact\": path}: verify shapes, drain, mount on every rank")
    s.add_argument("--total-kv-bytes", type=int, default=0, help="0 = size the pool from free device memory")
    s.add_argument("--bytes-per-token", type=int, default=0,
                   help="with --total-kv-bytes: KV bytes one token takes on this rank (0 = derived from the model and the plan)")
    s.add_argument("--gpus", default=None, help="comma-separated device ids; one process per GPU")
    s.add_argument("--prompt", default=None)
    s.add_argument("--max-new-tokens", type=int, default=32)
    s.add_argument("--rendezvous", default="/tmp/skein_rendezvous")
    s.add_argument("--restarts", type=int, default=0,
                   help="with --gpus: start the whole rank group again, up to this many times, after a rank was lost")
    s.add_argument("--batch-demo", action="store_true")
    s.add_argument("--demo-prompts", default=None)
    s.add_argument("--cuda-graphs", action=argparse.BooleanOptionalAction, default=True,
                   help="replay captured decode steps (--no-cuda-graphs launches every kernel eagerly)")
    s.add_argument("--temperature", type=float, default=0.0, help="generation job (--prompt / --demo-prompts): 0 = greedy")
    s.add_argument("--top-k", type=int, default=0)
    s.add_argument("--top-p", type=float, default=1.0)
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--ignore-eos", action="store_true",
                   help="generate max_tokens tokens even when the model emits its end-of-sequence token (benchmarks)")
    s.add_argument("--speculative-draft", default=None, help="artifact of a smaller draft model: speculative decoding in the generation job")
    s.add_argument("--speculative-k", type=int, default=4, help="draft tokens proposed per verification step")
    s.add_argument("--max-batch", type=int, default=0)
    s.add_argument("--max-seq-len", type=int, default=4096)

    k = sub.add_parser("calibrate", help="measure kernel efficiencies / collective bandwidth / dtype drift, rewrite the TOML files")
    k.add_argument("--hardware", required=True)
    k.add_argument("--model", required=True)
    k.add_argument("--corpus", required=True)
    k.add_argument("--drift-prompts-path", default=None)
    k.add_argument("--reference-artifact", default=None)
    k.add_argument("--candidate-artifact", default=None)
    k.add_argument("--out-cost", default="cluster/cost_constants.toml")
    k.add_argument("--out-drift-dir", default="models/")
    k.add_argument("--fit-step-ms", type=float, default=None,
                   help="measured decode-step time of --fit-plan on --fit-cluster: fits the fixed cost it identifies (per kernel "
                        "from a one-GPU plan, per all-reduce from a tensor-parallel one, per exchange from an expert-parallel one)")
    k.add_argument("--fit-plan", default=None, help="plan JSON (or an artifact directory) the step was measured with")
    k.add_argument("--fit-cluster", default=None, help="cluster TOML the step was measured on")
    k.add_argument("--fit-kv-tokens", type=int, default=None, help="context length of the measured step")
    k.add_argument("--autotune", action="store_true",
                   help="also measure GEMM launch configurations for the decode step and store them in the candidate "
                        "artifact's cache/kernel_configs.json (or --autotune-out)")
    k.add_argument("--autotune-out", default=None)
    k.add_argument("--autotune-batch", type=int, default=64)

    b = sub.add_parser("bench", help="replay a workload trace against an artifact and report throughput / goodput / drift compliance")
    b.add_argument("--artifact", default=None)
    b.add_argument("--workload", default=None)
    b.add_argument("--baseline", default=None, help="URL or label of the system the numbers are compared with")
    b.add_argument("--metrics", default="throughput,goodput,drift_compliance")
    b.add_argument("--max-requests", type=int, default=0)
    b.add_argument("--time-scale", type=float, default=1.0, help="divide arrival times by this factor")
    b.add_argument("--collectives", action="store_true", help="micro-benchmark the stand-alone collectives instead")
    b.add_argument("--url", default=None, help="replay the trace against a running server (e.g. http://127.0.0.1:8080) over HTTP/SSE "
                                               "instead of an in-process engine: the way to benchmark `serve --gpus` end to end")
    b.add_argument("--vocab-size", type=int, default=32000, help="with --url: range of the random prompt token ids")
    b.add_argument("--max-seq-len", type=int, default=4096, help="with --url: prompts are clipped so that prompt + output fit")
    b.add_argument("--op-profile", action="store_true", help="print the per-operator table of one decode step (eager launches, CUDA events)")
    b.add_argument("--synth", choices=["uniform", "burst"], default=None,
                   help="generate the trace instead of reading --workload: uniform (prompts 128..2048, outputs 64..512, Poisson 4 req/s) "
                        "or burst (on/off Poisson 50 / 2 req/s every 10 s, log-normal prompts of median 600 capped at 8192, outputs 32..1024)")
    b.add_argument("--synth-requests", type=int, default=256)
    b.add_argument("--synth-seed", type=int, default=0)
    b.add_argument("--write-trace", default=None, help="with --synth: write the generated trace (JSONL) here; without --artifact / --url "
                                                       "the command stops after writing it")
    return ap


def emit(args, payload: dict, text: str) -> None:
    if args.output == "json":
        print(json.dumps(payload, sort_keys=True))
    else:
        print(text)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level.upper(), logging.INFO), format="%(levelname)s %(name)s: %(message)s")
    try:
        if args.runtime_config:
            from ..utils.runtime_config import RuntimeConfig
            rc = RuntimeConfig.resolve(toml_text=_read(args.runtime_config))
            rc.apply_to_env()       # rank processes started by `serve --gpus` inherit it
            log.info("runtime config: %s", rc.describe())
        from . import commands
        return getattr(commands, "cmd_" + args.command)(args, emit)
    except Exception as e:  # one-line JSON error objects, like the reference
        if args.output == "json":
            print(json.dumps({"error": {"kind": type(e).__name__, "message": str(e)}}), file=sys.stderr)
        else:
            print(f"error: {type(e).__name__}: {e}", file=sys.stderr)
        if os.environ.get("SKEIN_TRACEBACK"):
            raise
        return 1


if __name__ == "__main__":
    sys.exit(main())
