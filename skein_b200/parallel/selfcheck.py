"""Multi-rank correctness check of the served model: a tiny Mixtral sharded over the live ranks (tensor parallel,
optionally expert parallel), decoded through the same CUDA-graph runner and fused collectives as the real model,
teacher-forced with the tokens of the unsharded CPU reference graph and compared step by step.

Used by the multi-GPU tests and by `bench.py`, which runs it before timing at N > 1 so that a throughput number at
4 or 8 ranks always comes with evidence that those ranks compute the right tokens.

A different greedy token is only accepted at a near-tie of the reference logits, or from the step on at which the
reference routed that sequence on a near-tie between experts (routing is discontinuous: under bf16-level noise such
a token legitimately goes to another expert, and its cache rows differ from then on); a near-tie at one of the
sequence's prompt tokens excuses the sequence from its first token on. The number of differing tokens is capped
either way.

The property is the reference's "TP shards summed equal the full op" (crates/skein_emit/tests/op_numerics.rs:299,371)
taken to the whole served model.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..models import config as mc
from ..models.decoder import BatchInputs, Decoder, random_weights
from ..models.sharding import shard_model
from ..ops import reference as ref
from ..runtime.runner import ModelRunner


def teacher_forced_check(world: int, rank: int, dev, comm=None, comm_moe=None, tp: int | None = None, ep: int = 1,
                         hidden: int = 1024, steps: int = 6, fp8_experts: bool = False, seed: int = 11, dp_attention: bool = False):
    """Runs on every rank of the job (collective). `comm` / `comm_moe` are communicators over this rank's tensor-
    parallel group / all tp x ep ranks, built for `hidden`. Returns a dict of what was compared; raises
    AssertionError on a mismatch that no near-tie explains. dp_attention: pure expert parallelism with every rank
    attending over its own slice of the rows (token dispatch between the ranks); the batch is then 4 rows per rank."""
    tp = tp if tp is not None else world // ep
    heads = max(8, 2 * tp)
    cfg = mc.tiny_mixtral(layers=2, hidden=hidden, inter=512 * tp, heads=heads, kv_heads=max(tp, 2) if tp <= 2 else heads,
                          experts=max(4, 2 * ep), vocab=1024)
    if heads % cfg.num_kv_heads:
        cfg.num_kv_heads = heads
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=seed, std=0.05)
    lay = mc.ParallelLayout(tp=tp, ep=ep, rank=rank)
    w = shard_model(full, cfg, lay, dev, shard_embed=comm is not None and tp > 1)    # vocabulary-parallel embedding
    if fp8_experts:
        from ..models.decoder import quantize_blocks
        quantize_blocks(w, range(len(w.layers)), names=("w13", "w2"))
    dp = dp_attention and ep > 1 and tp == 1 and dev.type == "cuda"
    B, P = (4 * ep if dp else 3), 21
    dec = Decoder(cfg, w, lay, num_pages=4 * B + 8, page_size=16, max_pos=256, comm=comm, comm_moe=comm_moe)
    dec.dp_attention = dp
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).tolist()
    tables = [[1 + 4 * s + i for i in range(4)] for s in range(B)]

    # reference run on CPU (rank 0 decides, everyone follows): tokens plus the top-1/top-2 logit gap per step
    if rank == 0:
        dec_ref = Decoder(cfg, full, num_pages=4 * B + 8, page_size=16, max_pos=256)
        margins = []
        ref_router = ref.router_topk

        def recording_router(x, wg, topk):
            ids, wts, lg_ = ref_router(x, wg, topk)
            srt = torch.sort(lg_, dim=-1, descending=True).values
            margins.append((srt[:, topk - 1] - srt[:, topk]).tolist())
            return ids, wts, lg_

        ref.router_topk = recording_router
        try:
            runner_ref = ModelRunner(dec_ref, max_blocks_per_seq=4, use_graphs=False)
            toks, lg = runner_ref.prefill([(prompts[s], tables[s], 0) for s in range(B)], want_logits=True)
            # a near-tie between experts at one of a sequence's PROMPT tokens can send that token to another expert under
            # bf16-level noise: the sequence's cache rows, and with them its first token and every later one, may then differ
            prefill_tie = [min(min(m[s_ * P:(s_ + 1) * P]) for m in margins) < 0.06 for s_ in range(B)]
            margins.clear()   # from here on: one entry per decode step and layer
            ref_toks, gaps = [toks], []
            top2 = lg.float().topk(2, dim=-1).values
            gaps.append((top2[:, 0] - top2[:, 1]).tolist())
            cached = P
            i32 = lambda x: torch.tensor(x, dtype=torch.int32)
            bt = torch.tensor(tables, dtype=torch.int32)
            for _ in range(steps):
                inp = BatchInputs(token_ids=i32(ref_toks[-1]), positions=i32([cached] * B), block_table=bt,
                                  seq_lens=i32([cached + 1] * B))
                tok, lg = dec_ref.forward(inp)
                top2 = lg.float().topk(2, dim=-1).values
                gaps.append((top2[:, 0] - top2[:, 1]).tolist())
                ref_toks.append(tok.tolist())
                cached += 1
        finally:
            ref.router_topk = ref_router
        n_l = cfg.num_layers
        tie_from = [0 if prefill_tie[s_] else
                    min([t + 1 for t in range(steps) if min(margins[t * n_l + l][s_] for l in range(n_l)) < 0.06], default=steps + 1)
                    for s_ in range(B)]
        payload = [ref_toks, gaps, tie_from]
    else:
        payload = [None, None, None]
    if world > 1:
        dist.broadcast_object_list(payload, src=0)
    ref_toks, gaps, tie_from = payload

    # teacher-forced sharded run through CUDA graphs: every step is fed the reference's previous tokens
    fused = all(c is None or c.mode != "nccl" for c in (comm, comm_moe))
    runner = ModelRunner(dec, max_blocks_per_seq=4, use_graphs=fused)      # library collectives are launched eagerly
    got = [runner.prefill([(prompts[s], tables[s], 0) for s in range(B)])]
    bk = runner.bucket(B)
    cached = P
    for t in range(steps):
        runner.load_decode_inputs(bk, ref_toks[t], [cached] * B, [cached + 1] * B, tables)
        got.append(runner.decode_step(bk)[:B].tolist())
        cached += 1
    if dev.type == "cuda":
        torch.cuda.synchronize()
        ops.workspace().check_status()
        assert runner.graph_replays == (steps if fused else 0)
    diffs = [(t, s_, got[t][s_], ref_toks[t][s_], round(gaps[t][s_], 4))
             for t in range(steps + 1) for s_ in range(B) if got[t][s_] != ref_toks[t][s_]]
    limit = 0.3 if fp8_experts else 0.08        # e4m3 weights move the logits more than bf16 rounding does
    hard = [d for d in diffs if d[4] >= limit and d[0] < tie_from[d[1]]]
    assert not hard and len(diffs) <= (8 if fp8_experts else 4) * max(1, B // 3), \
        ("(step, seq, got, want, reference top-2 gap)", diffs, "router tie from", tie_from)
    return {"tokens_compared": B * (steps + 1), "mismatches_at_near_ties": len(diffs), "tp": tp, "ep": ep, "dp_attention": dp,
            "graph_replays": runner.graph_replays}
