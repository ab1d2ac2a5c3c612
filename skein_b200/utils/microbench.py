"""Per-kernel micro-benchmarks with roofline fractions against the measured peaks of the machine.

    python -m skein_b200.utils.microbench --op moe_gate_up --tp 1
    python -m skein_b200.utils.microbench --op all --tp 8
    python -m skein_b200.utils.microbench --op moe_gate_up --tp 4 --iters 1 --warmup 1     # a profiler-sized run

Shapes are the decode step of Mixtral-8x7B (64 sequences, top-2 of 8 experts, hidden 4096, ffn 14336,
32/8 heads of 128) divided by --tp the way the tensor-parallel shards divide them; attn_prefill, prefill_qkv,
argmax and quant_fp8 time the prefill-sized launches (16 prompts of --ctx tokens, 8192-token projection). Every op is timed
with CUDA events after warm-up, with a 256 MiB write between iterations so that nothing is served from
L2, and reported as the median. The denominators are the machine's measured copy bandwidth and bf16
GEMM rate when a MEASURED_PEAKS.json sits at the repository root, else the stated fallback.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import ops

_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "kind": "measured"}
    return dict(_FALLBACK, kind="fallback")


def timeit(fn, iters, warmup, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    scr = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    ts = []
    for _ in range(iters):
        if scr is not None:
            scr.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def timeit_graph(make, bytes_per_launch, iters, warmup):
    """In-graph timing: enough independent copies of the op's operands that their total exceeds twice the L2,
    one launch per copy captured into a CUDA graph, launches back to back as in a decode step. Returns the mean
    time per launch (the event timer's ~2 us resolution is amortised over the whole graph)."""
    copies = max(2, min(64, -(-(256 << 20) // max(int(bytes_per_launch), 1))))
    fns = [make()[0] for _ in range(copies)]
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3 / copies)
    ts.sort()
    return ts[len(ts) // 2]


def _report(name, us, bytes_, flops, pk):
    gbs = bytes_ / us * 1e-3
    tfs = flops / us * 1e-6
    fb, ff = gbs / pk["hbm_gbs"], tfs / pk["bf16_tflops"]
    bound = "memory" if fb >= ff else "compute"
    print(json.dumps({"op": name, "us": round(us, 2), "GBps": round(gbs, 1), "TFLOPs": round(tfs, 2),
                      "frac_of_%s_hbm" % pk["kind"]: round(fb, 3), "frac_of_%s_bf16" % pk["kind"]: round(ff, 3),
                      "bound": bound, "MB": round(bytes_ / 1e6, 2)}))


def _bf(*shape, std=0.02):
    return torch.empty(*shape, device="cuda", dtype=torch.bfloat16).normal_(0, std)


def op_moe(which, tp, a):
    E, H, F, per = 8, 4096, 14336 // tp, a.tokens * 2 // 8
    rows = E * per
    cnt = torch.full((E,), per, dtype=torch.int32, device="cuda")
    off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    off[1:] = torch.cumsum(cnt, 0)
    if which == "gate_up":
        xs, w = _bf(rows, H, std=1.0), _bf(E, 2 * F, H)
        out = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops.grouped_linear(xs, w, cnt, off, swiglu=True, out=out)
        fl = 2 * rows * 2 * F * H
    else:
        xs, w = _bf(rows, F, std=1.0), _bf(E, H, F)
        out = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops.grouped_linear(xs, w, cnt, off, swiglu=False, out=out)
        fl = 2 * rows * H * F
    by = w.numel() * 2 + xs.numel() * 2 + out.numel() * 2
    if getattr(a, "fp8", False):   # e4m3 expert weights with 1 x 128 block scales, bf16 activations
        from ..ops import fp8
        wq = fp8.quantize_weight(w)
        del w
        by = wq.nbytes() + xs.numel() * 2 + out.numel() * 2
        return (lambda: fp8.grouped_linear_a16(xs, wq, cnt, off, swiglu=(which == "gate_up"), out=out)), by, fl
    if a.packed:   # tile-packed weights: every 128 x 64 tile the GEMM loads is one contiguous 16 KB block
        wp = ops.pack_weight(w)
        del w
        fn = (lambda: ops.grouped_linear(xs, wp, cnt, off, swiglu=(which == "gate_up"), out=out))
    return fn, by, fl


def op_dense(F, K, a):
    x, w = _bf(a.tokens, K, std=1.0), _bf(F, K)
    out = torch.empty(a.tokens, F, dtype=torch.bfloat16, device="cuda")
    return (lambda: ops.linear(x, w, out=out)), (w.numel() + x.numel() + out.numel()) * 2, 2 * a.tokens * F * K


def op_attn(tp, a):
    B, Hq, Hkv, D, ctx = a.tokens, 32 // tp, max(1, 8 // tp), 128, a.ctx
    nb = (ctx + 15) // 16
    kv = _bf(B * nb + 1, 2, Hkv, 16, D, std=1.0)
    bt = torch.arange(B * nb, dtype=torch.int32, device="cuda").view(B, nb) + 1
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = _bf(B, Hq * D, std=1.0)
    out = torch.empty(B, Hq * D, dtype=torch.bfloat16, device="cuda")
    fn = lambda: ops.attn_decode(q, kv, bt, lens, Hq, Hkv, D, out=out, ctx_hint=ctx)
    return fn, B * ctx * 2 * Hkv * D * 2, 4 * B * Hq * ctx * D


def op_reduce(a):
    B, H = a.tokens, 4096
    res, part, g = _bf(B, H, std=1.0), _bf(1, B, H, std=1.0), _bf(H, std=1.0)
    fn = lambda: ops.reduce_residual_rmsnorm(res, part, g, 1e-5)
    return fn, 4 * B * H * 2, 6 * B * H


def op_reduce_route(a):
    """Post-attention point of a MoE block: partial sum + residual + RMSNorm + router + expert-sorted scatter."""
    B, H = a.tokens, 4096
    res, part, g, wg = _bf(B, H, std=1.0), _bf(1, B, H, std=1.0), _bf(H, std=1.0), _bf(8, H)
    fn = lambda: ops.reduce_norm_route(res, part, g, 1e-5, wg, 2)
    return fn, (6 * B * H + 8 * H) * 2, 2 * B * 8 * H


def op_router(a):
    x, wg = _bf(a.tokens, 4096, std=1.0), _bf(8, 4096)
    fn = lambda: ops.route(x, wg, 2)
    return fn, (x.numel() + wg.numel()) * 2, 2 * a.tokens * 8 * 4096


def op_attn_prefill(tp, a):
    """Causal prefill attention over the paged cache: 16 prompts of --ctx tokens in one launch."""
    S, L, Hq, Hkv, D = 16, a.ctx, 32 // tp, max(1, 8 // tp), 128
    nb = (L + 15) // 16
    kv = _bf(S * nb + 1, 2, Hkv, 16, D, std=1.0)
    bt = torch.arange(S * nb, dtype=torch.int32, device="cuda").view(S, nb) + 1
    q = _bf(S * L, Hq * D, std=1.0)
    out = torch.empty_like(q)
    q_start = torch.arange(S, dtype=torch.int32, device="cuda") * L
    q_len = torch.full((S,), L, dtype=torch.int32, device="cuda")
    fn = lambda: ops.attn_prefill(q, kv, bt, q_start, q_len, q_len, L, Hq, Hkv, D, out=out)
    return fn, (2 * q.numel() + S * L * 2 * Hkv * D) * 2, 4 * Hq * D * S * L * (L + 1) // 2


def op_prefill_gemm(tp, a):
    """The qkv projection at prefill size (8192 tokens): the compute-bound regime of the same GEMM kernel."""
    T, F, K = 8192, (32 + 16) * 128 // tp, 4096
    x, w = _bf(T, K, std=1.0), _bf(F, K)
    out = torch.empty(T, F, dtype=torch.bfloat16, device="cuda")
    return (lambda: ops.linear(x, w, out=out)), (w.numel() + x.numel() + out.numel()) * 2, 2 * T * F * K


def op_argmax(tp, a):
    logits = _bf(a.tokens, 32000 // tp, std=1.0)
    out = torch.empty(a.tokens, dtype=torch.int32, device="cuda")
    return (lambda: ops.sample_argmax(logits, out=out)), logits.numel() * 2, logits.numel()


def op_quant_fp8(a):
    x = _bf(16384, 4096, std=1.0)
    return (lambda: ops.quant_fp8_block128(x)), x.numel() * 3 + x.numel() // 128 * 4, 2 * x.numel()

def op_ep_dispatch(ep, a):
    """Receiving half of the expert-parallel token dispatch (csrc/kernels/ep_dispatch.cu) for one rank of `ep`, with the
    other ranks' published buffers standing in this GPU's memory (one launch reads all of them; their flags are already
    raised): layout from all ranks' expert choices plus the gather of the rows routed to this rank's experts."""
    import ctypes as C
    from ..ops import _lib
    T, k, E, H = a.tokens, 2, 8, 4096
    ep = max(1, min(ep, 8))
    per = max(1, T // ep)
    g = torch.Generator(device="cuda").manual_seed(3)
    rows = [_bf(per, H, std=1.0) for _ in range(ep)]
    ids = [torch.stack([torch.randperm(E, generator=g, device="cuda")[:k] for _ in range(per)]).to(torch.int32) for _ in range(ep)]
    flags = torch.ones(ep, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    n = ep * per * k
    ids_all = torch.empty(n, dtype=torch.int32, device="cuda")
    meta = torch.empty(2 * E + 1 + 2 * n, dtype=torch.int32, device="cuda")
    xs = torch.empty(n, H, dtype=torch.bfloat16, device="cuda")
    VP = C.c_void_p * ep
    rp, ip = VP(*[r.data_ptr() for r in rows]), VP(*[i.data_ptr() for i in ids])
    e_cnt = E // ep
    keep = (rows, ids)

    def fn():
        _lib.check(_lib.lib().skein_ep_dispatch_pull(rp, ip, ep, per, k, E, 0, e_cnt, H, flags.data_ptr(), epoch.data_ptr(),
                                                     ops.workspace().status.data_ptr(), 100, ids_all.data_ptr(), meta.data_ptr(),
                                                     meta[E:].data_ptr(), meta[2 * E + 1:].data_ptr(),
                                                     meta[2 * E + 1 + n:].data_ptr(), xs.data_ptr(), _lib.stream_ptr()), "ep_dispatch")
        return keep
    # bytes: all choices read once per pair CTA from L2, the gathered rows read and written once
    return fn, n // ep * H * 2 * 2 + n * 4, n


def build(name, a):
    tp = a.tp
    if name == "moe_gate_up":
        return op_moe("gate_up", tp, a)
    if name == "moe_down":
        return op_moe("down", tp, a)
    if name == "qkv":
        return op_dense((32 + 16) * 128 // tp, 4096, a)
    if name == "o_proj":
        return op_dense(4096, 32 * 128 // tp, a)
    if name == "lm_head":
        return op_dense(32000 // tp, 4096, a)
    if name == "attn_decode":
        return op_attn(tp, a)
    if name == "reduce_norm":
        return op_reduce(a)
    if name == "router":
        return op_router(a)
    if name == "reduce_route":
        return op_reduce_route(a)
    if name == "attn_prefill":
        return op_attn_prefill(tp, a)
    if name == "prefill_qkv":
        return op_prefill_gemm(tp, a)
    if name == "argmax":
        return op_argmax(tp, a)
    if name == "quant_fp8":
        return op_quant_fp8(a)
    if name == "ep_dispatch":
        return op_ep_dispatch(tp, a)
    raise SystemExit(f"unknown op {name}")


OPS = ("moe_gate_up", "moe_down", "qkv", "o_proj", "lm_head", "attn_decode", "reduce_norm", "reduce_route", "router",
       "attn_prefill", "prefill_qkv", "argmax", "quant_fp8", "ep_dispatch")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--op", default="all", help="one of: all, " + ", ".join(OPS))
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree whose shard shapes are timed")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--packed", action="store_true", help="MoE ops: use tile-packed weights (ops.pack_weight)")
    ap.add_argument("--fp8", action="store_true", help="MoE ops: block-scaled e4m3 expert weights with bf16 activations")
    ap.add_argument("--graph", action="store_true",
                    help="time launches back to back inside a CUDA graph over rotating operand copies (cold L2, "
                         "no per-launch event overhead) instead of one launch per event pair")
    a = ap.parse_args(argv)
    pk = peaks()
    for name in (OPS if a.op == "all" else a.op.split(",")):
        fn, by, fl = build(name, a)
        if a.graph:
            us = timeit_graph(lambda: build(name, a), by, a.iters, a.warmup)
        else:
            us = timeit(fn, a.iters, a.warmup, flush=not a.no_flush)
        _report(f"{name}/tp{a.tp}" + ("/fp8w" if a.fp8 and name.startswith("moe") else "") + ("/graph" if a.graph else ""), us, by, fl, pk)
    ops.workspace().check_status()


if __name__ == "__main__":
    main()
