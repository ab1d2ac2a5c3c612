#!/usr/bin/env python
"""Headline benchmark: Mixtral-8x7B-shaped decode throughput (tokens/s) at 1/2/4/8 B200.

    python bench.py --gpus 1 --steps 128 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 128 --warmup 8

Workload (the serving config of the headline): random-init bf16 weights N(0, 0.02), 64 concurrent
sequences, prompts of 512 random token ids, 256 generated tokens, paged KV with block size 16,
tensor parallel over all N GPUs. A "step" is one decode step of the whole batch (64 tokens).

Two measurements, both with every kernel of the step (sampling included) inside the timed region:
  value  device-timed (CUDA events, max over ranks): K replays of the captured decode step with the
         sampled tokens fed back on the device.
  e2e    the same step through ModelRunner.decode_step, the call the serving engine makes: every
         step copies its inputs (token ids, positions, lengths, block tables) from pinned host memory
         to the device and reads the sampled tokens back.
The weights (93 GB at N=1) are far larger than L2, so no explicit L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOK_S = 168.0  # the reference's only published number (2x RTX PRO 6000, PP=2)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="mixtral-8x7b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--gen", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree (tensor parallel = gpus / ep)")
    ap.add_argument("--fp8-experts", action="store_true", help="block-scaled e4m3 expert / FFN weights (marks dtype)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--eager", action="store_true",
                    help="launch the step's kernels one by one instead of replaying the captured graph "
                         "(for a per-kernel launch list; the timed loop sits in an NVTX range named 'timed')")
    return ap.parse_args()


def reference_arm(args):
    # The reference is a Rust workspace (cargo, luminal, cudarc). It has no Python package to install
    # (`pip install` of its source tree: "Neither 'setup.py' nor 'pyproject.toml' found") and this image
    # has no Rust toolchain, so it cannot be built or run here.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a Rust/cargo workspace: pip reports no setup.py/pyproject.toml "
                                     "and the image has no cargo/rustc, so it cannot be built offline"}))
    return 0


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled DURING the timed region: NVML reads from a thread every
    10 ms (read-only queries), or `nvidia-smi -lms 100` when NVML cannot be loaded."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                   0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.thread = None
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = False

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.idx < len(ids) and ids[self.idx].isdigit():
                return int(ids[self.idx])
        return self.idx

    def start(self):
        try:
            import threading

            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop:
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        bits = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        for bit, name in self.REASON_BITS.items():
                            if bits & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(0.01)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            sm = self.samples
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(self.reasons), "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    # Libraries (NCCL's version banner, for one) write to file descriptor 1. Keep the real stdout for the one JSON
    # line and send everything else that lands on descriptor 1 to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit_json(obj):
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    import numpy as np
    import torch
    import torch.distributed as dist

    from skein_b200.models import config as mc
    from skein_b200.models.decoder import Decoder, random_weights
    from skein_b200.ops import _lib
    from skein_b200 import ops
    from skein_b200.runtime.runner import ModelRunner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (WORLD_SIZE must equal --gpus)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = {"mixtral-8x7b": mc.mixtral_8x7b, "mixtral-8x22b": mc.mixtral_8x22b, "llama3-70b": mc.llama3_70b}[args.model]()
    if args.layers:
        cfg.num_layers = args.layers
    ep = max(1, args.ep)
    if world % ep != 0 or (ep > 1 and not cfg.is_moe):
        raise SystemExit("--ep must divide the number of GPUs and needs a mixture-of-experts model")
    tp = world // ep
    comm, comm_moe = None, None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
        from skein_b200.parallel.tp import TPComm
        if tp > 1:
            groups = [dist.new_group(list(range(b0, b0 + tp))) for b0 in range(0, world, tp)] if ep > 1 else [dist.group.WORLD]
            comm = TPComm(groups[rank // tp] if ep > 1 else groups[0], dev, hidden=cfg.hidden_size)
        if ep > 1:   # communicator over all tp x ep ranks for the expert-parallel combine
            comm_moe = TPComm(dist.group.WORLD, dev, hidden=cfg.hidden_size)
    lay = mc.ParallelLayout(tp=tp, ep=ep, rank=rank)
    B, P, Gn, ps = args.batch, args.prompt, args.gen, 16
    blocks_per_seq = (P + Gn + ps - 1) // ps + 1
    num_pages = B * blocks_per_seq + 8
    t0 = time.time()
    weights = random_weights(cfg, lay, dev, seed=0, std=0.02)
    if args.fp8_experts:
        from skein_b200.models.decoder import quantize_blocks
        quantize_blocks(weights, range(len(weights.layers)), names=("w13", "w2"))
    dec = Decoder(cfg, weights, lay, num_pages=num_pages, page_size=ps, max_pos=P + Gn + 64, comm=comm, comm_moe=comm_moe)
    fused = all(c is None or c.mode == "fused" for c in (comm, comm_moe))
    use_graphs = fused and not args.eager   # the NCCL baseline mode launches eagerly
    runner = ModelRunner(dec, max_blocks_per_seq=blocks_per_seq, use_graphs=use_graphs, ctx_hint=P + Gn // 2)
    torch.cuda.synchronize()
    t_init = time.time() - t0

    # ---- requests: identical on every rank ---------------------------------------------------------
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).tolist()
    tables = [list(range(1 + s * blocks_per_seq, 1 + (s + 1) * blocks_per_seq)) for s in range(B)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def check_all(where):
        # every rank learns of a device-side error (a peer wait that ran out, a bad index) on any rank
        code = ops.workspace().status[:1].clone()
        if world > 1:
            dist.all_reduce(code, op=dist.ReduceOp.MAX)
        if int(code[0]) != 0:
            if rank == 0:
                emit_json({"error": f"device status {int(code[0])} after {where}", "n_gpus": world})
            if world > 1:
                dist.destroy_process_group()
            sys.exit(3)

    # ---- prefill (chunks of up to 8192 tokens); TTFT of a sequence = time until its chunk finished ----
    per_chunk = max(1, 8192 // P)
    barrier()
    t_start = time.perf_counter()
    first_tokens, ttft = [], []
    for c0 in range(0, B, per_chunk):
        toks = runner.prefill([(prompts[s], tables[s], 0) for s in range(c0, min(B, c0 + per_chunk))])
        torch.cuda.synchronize()
        first_tokens.extend(toks)
        ttft.extend([(time.perf_counter() - t_start) * 1e3] * len(toks))
    check_all("prefill")

    bk = runner.bucket(B)

    def reset_state():
        runner.load_decode_inputs(bk, first_tokens, [P] * B, [P + 1] * B, tables)
        bk.dev_in.copy_(bk.host_in)
        torch.cuda.synchronize()

    K, W = args.steps, max(args.warmup, 3)
    if K + W > Gn - 1:
        raise SystemExit(f"--steps + --warmup must stay below the {Gn} generated tokens of the workload")

    # ---- device-timed loop ---------------------------------------------------------------------------
    reset_state()
    l0 = _lib.launches()
    if use_graphs:
        runner._ensure_graph(bk, True)
    launches_per_step = None
    for i in range(W):
        runner.decode_loop_step(bk)
        if i == 0:
            check_all("the first decode step")
    # kernels per step: count one eager step's launches on a scratch copy of the state
    saved = bk.dev_in.clone()
    torch.cuda.synchronize()
    l1 = _lib.launches()
    runner._decode_body(bk, True)
    torch.cuda.synchronize()
    launches_per_step = _lib.launches() - l1
    bk.dev_in.copy_(saved)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    torch.cuda.nvtx.range_push("timed")
    for _ in range(K):
        runner.decode_loop_step(bk)
    torch.cuda.nvtx.range_pop()
    ev1.record()
    barrier()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    check_all("the timed loop")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    value = B * K / (ms / 1e3)

    # ---- end-to-end loop through the runner's public step call ------------------------------------------
    e2e = None
    if not args.no_e2e:
        reset_state()
        tok_h, pos_h, len_h, _ = bk.views(bk.host_in)
        tok_np, pos_np, len_np = tok_h.numpy(), pos_h.numpy(), len_h.numpy()
        for _ in range(W):
            res = runner.decode_step(bk)
            tok_np[:] = res.numpy(); pos_np += 1; len_np += 1
        barrier()
        step_ms = []
        t_a = time.perf_counter()
        for _ in range(K):
            t_s = time.perf_counter()
            res = runner.decode_step(bk)            # H2D inputs, graph replay, D2H result, stream sync
            tok_np[:] = res.numpy(); pos_np += 1; len_np += 1
            step_ms.append((time.perf_counter() - t_s) * 1e3)
        barrier()
        wall = time.perf_counter() - t_a
        if world > 1:
            t = torch.tensor([wall], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall = float(t[0])
        step_ms.sort()
        e2e = {"value": round(B * K / wall, 2), "unit": "tokens/s", "h2d_bytes_per_step": bk.h2d_bytes,
               "d2h_bytes_per_step": bk.d2h_bytes, "tpot_p50_ms": round(step_ms[len(step_ms) // 2], 3),
               "tpot_p99_ms": round(step_ms[min(len(step_ms) - 1, int(0.99 * len(step_ms)))], 3)}

    if rank == 0:
        ttft.sort()
        out = {
            "metric": args.model.replace("-", "_") + "_decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": round(value / BASELINE_TOK_S, 2) if args.model == "mixtral-8x7b" and not args.layers else None,
            "dtype": "bf16" if not args.fp8_experts else "bf16 activations, fp8 expert weights",
            "data": "synthetic (random-init weights N(0,0.02), random prompt token ids)",
            "config": {"model": cfg.name + ("" if not args.layers else f"-{args.layers}layers-INVALID"),
                       "global_batch": B, "seq_len": P, "gen_len": Gn, "parallelism": f"tp{tp}" + (f"xep{ep}" if ep > 1 else ""),
                       "kv": "paged, block 16", "l2": "inputs (weights) larger than L2, no flush",
                       "cuda_graph": use_graphs, "comm": ((comm or comm_moe).mode if (comm or comm_moe) else "none"),
                       "expert_weights": "fp8 e4m3 1x128" if args.fp8_experts else "bf16"},
            "ttft_p50_ms": round(ttft[len(ttft) // 2], 2),
            "tpot_p99_ms": e2e["tpot_p99_ms"] if e2e else None,
            "e2e": e2e, "gpu_launches": launches_per_step * K, "kernels_per_step": launches_per_step,
            "clocks": clocks, "init_s": round(t_init, 1), "impl": "ours",
        }
        emit_json(out)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
