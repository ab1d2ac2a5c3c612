"""Sharded execution on CPU ranks (threads + barrier): TP=2 / TP=4 shards reproduce the unsharded model,
vocabulary-parallel sampling, repeated collectives stay aligned, and host-side failure detection (a rank
that raises, a rank that never arrives) ends the others with an error instead of a hang.

Mirrors crates/skein_emit/tests/op_numerics.rs:299,371 (TP shards sum to the full op), vocab_parallel.rs:38,56,
crates/skein_runtime/src/distributed/barrier_collective.rs:179-220, rank_executor.rs:443-552,
segment_runner.rs:1698-1791 (two-rank pipeline on CPU threads).
"""
import dataclasses
import time

import pytest
import torch

from skein_b200.models import config as mc
from skein_b200.models.decoder import Decoder, ModelWeights, random_weights
from skein_b200.models.sharding import shard_model
from skein_b200.parallel.local import CommError, run_ranks
from skein_b200.runtime.runner import ModelRunner


def _generate(dec, prompts, tables, steps=3):
    runner = ModelRunner(dec, max_blocks_per_seq=4, use_graphs=False)
    toks, lg = runner.prefill([(p, t, 0) for p, t in zip(prompts, tables)], want_logits=True)
    outs, cached = [toks], len(prompts[0])
    bk = runner.bucket(len(prompts))
    for _ in range(steps):
        runner.load_decode_inputs(bk, outs[-1], [cached] * len(prompts), [cached + 1] * len(prompts), tables)
        outs.append(runner.decode_step(bk)[:len(prompts)].tolist())
        cached += 1
    return outs, lg


@pytest.mark.parametrize("tp,cfg", [(2, mc.tiny_mixtral(heads=4, kv_heads=2)), (4, mc.tiny_mixtral(heads=8, kv_heads=4, inter=1024)),
                                    (8, mc.tiny_mixtral(heads=16, kv_heads=8, inter=2048)),
                                    (2, mc.tiny_llama()), (2, dataclasses.replace(mc.tiny_llama(), architecture="Qwen2ForCausalLM", qkv_bias=True))],
                         ids=["mixtral-tp2", "mixtral-tp4", "mixtral-tp8", "llama-tp2", "qwen2-tp2-qkv-bias"])
def test_tp_shards_reproduce_the_unsharded_model(tp, cfg):
    torch.manual_seed(0)
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=5, std=0.05)
    prompts = torch.randint(0, cfg.vocab_size, (2, 19)).tolist()
    tables = [[1, 2, 3, 4], [5, 6, 7, 8]]
    want, want_lg = _generate(Decoder(cfg, full, num_pages=16, page_size=16, max_pos=128), prompts, tables)
    if cfg.qkv_bias:        # the biases matter: without them the model samples other tokens
        assert full.layers[0].bqkv is not None
        bare = ModelWeights(full.embed, [dataclasses.replace(l, bqkv=None) for l in full.layers], full.final_norm, full.lm_head)
        assert _generate(Decoder(cfg, bare, num_pages=16, page_size=16, max_pos=128), prompts, tables)[0] != want

    def rank_fn(r, comm):
        lay = mc.ParallelLayout(tp=tp, rank=r)
        # the embedding table is vocabulary-parallel (each rank holds V / tp rows) except in the last case
        w = shard_model(full, cfg, lay, shard_embed=cfg.is_moe)
        assert w.embed.shape[0] == (cfg.vocab_size // tp if cfg.is_moe else cfg.vocab_size)
        dec = Decoder(cfg, w, lay, num_pages=16, page_size=16, max_pos=128, comm=comm)
        return _generate(dec, prompts, tables)

    results, errors = run_ranks(tp, rank_fn)
    assert not any(errors)
    for outs, lg in results:
        assert outs == want                                   # every rank samples the same tokens as the full model
    # the ranks' logit shards, concatenated, are the full logits
    cat = torch.cat([lg for _, lg in results], dim=1).float()
    assert float((cat - want_lg.float()).norm() / want_lg.float().norm()) < 0.03


def test_repeated_collectives_stay_aligned():
    def rank_fn(r, comm):
        acc = []
        for i in range(20):
            acc.append(float(comm.all_reduce(torch.tensor([[float(r + i)]]))[0, 0]))
        return acc
    results, _ = run_ranks(3, rank_fn)
    assert results[0] == results[1] == results[2] == [float(3 * i + 3) for i in range(20)]


def test_a_failing_rank_ends_the_others_with_an_error():
    seen = {}

    def rank_fn(r, comm):
        comm.all_reduce(torch.ones(1, 1))
        if r == 1:
            raise ValueError("rank 1 lost its GPU (injected)")
        try:
            comm.all_reduce(torch.ones(1, 1))
        except CommError as e:
            seen[r] = str(e)
            raise
    t0 = time.time()
    with pytest.raises(ValueError, match="injected"):
        run_ranks(3, rank_fn, timeout_s=20.0)
    assert time.time() - t0 < 10 and set(seen) == {0, 2}


def test_a_rank_that_never_arrives_times_out():
    def rank_fn(r, comm):
        if r == 0:
            time.sleep(1.0)          # never joins within the collective's budget
            return "late"
        comm.all_reduce(torch.ones(1, 1))
    t0 = time.time()
    with pytest.raises(CommError):
        run_ranks(2, rank_fn, timeout_s=0.2)
    assert time.time() - t0 < 5


@pytest.mark.parametrize("tp,ep", [(1, 2), (1, 4), (2, 2)], ids=["ep2", "ep4", "tp2xep2"])
def test_expert_parallel_ranks_reproduce_the_unsharded_model(tp, ep):
    """Experts owned in blocks by the EP ranks, attention tensor-parallel inside each TP group: the owner-aware
    combine reproduces the single-device model (the reference only tests its dense EP scheme on CPU:
    crates/skein_emit/tests/ep_routing.rs:14,68, topology_emission.rs:57)."""
    cfg = mc.tiny_mixtral(heads=4, kv_heads=2, experts=4)
    torch.manual_seed(0)
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=9, std=0.05)
    prompts = torch.randint(0, cfg.vocab_size, (2, 19)).tolist()
    tables = [[1, 2, 3, 4], [5, 6, 7, 8]]
    want, _ = _generate(Decoder(cfg, full, num_pages=16, page_size=16, max_pos=128), prompts, tables)

    def rank_fn(r, world):
        lay = mc.ParallelLayout(tp=tp, ep=ep, rank=r)
        comm_tp = world.subgroup(lay.tp_group()) if tp > 1 else None
        dec = Decoder(cfg, shard_model(full, cfg, lay), lay, num_pages=16, page_size=16, max_pos=128, comm=comm_tp, comm_moe=world)
        assert dec.w.layers[0].w13.shape[0] == cfg.num_experts // ep
        return _generate(dec, prompts, tables)[0]

    results, errors = run_ranks(tp * ep, rank_fn)
    assert not any(errors)
    assert all(r == want for r in results)


def test_engine_rows_under_data_parallel_attention():
    """Pure expert parallelism with data-parallel attention: the engine gives every decoding sequence to one rank's slice
    of the step's rows for its whole life, pads the slices to one size and runs the same steps on every rank. On CPU
    ranks the decoder attends over all rows, so the tokens must equal the unsharded engine's exactly; the test covers
    the row layout, the padding rows inside a step and the release of a finished sequence's slot."""
    from skein_b200.runtime.engine import Engine, EngineConfig
    cfg = mc.tiny_mixtral(layers=2, hidden=128, inter=256, heads=4, kv_heads=2, experts=4, vocab=256)
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=11, std=0.05)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (5, 9, 7, 3, 6)]
    ecfg = lambda: EngineConfig(max_batch=16, tpot_ms=1e9, ttft_ms=1e9, use_graphs=False, prefix_cache=False)  # noqa: E731
    want = Engine(Decoder(cfg, full, num_pages=96, page_size=16, max_pos=128), ecfg()).generate(prompts, 4)

    def body(rank, comm):
        lay = mc.ParallelLayout(tp=1, ep=2, rank=rank)
        dec = Decoder(cfg, shard_model(full, cfg, lay, "cpu"), lay, num_pages=96, page_size=16, max_pos=128, comm_moe=comm)
        assert dec.dp_ways() == 1
        dec.dp_attention = True
        assert dec.dp_ways() == 2
        eng = Engine(dec, ecfg())
        assert eng._dp == 2 and dec.dp_strict
        out = eng.generate(prompts, 4)
        assert eng._dp_load == [0, 0] and not eng._dp_of          # every finished sequence gave its slot back
        rows = eng._dp_layout([11, 12, 13, 14, 15])               # least loaded slice first, ties to the lower rank
        assert rows == [11, 13, 15, 0, 12, 14, 0, 0]
        eng._dp_release(13)
        assert eng._dp_layout([11, 12, 14, 15, 16]) == [11, 15, 16, 0, 12, 14, 0, 0]    # a sequence keeps its rank
        return out

    results, _ = run_ranks(2, body)
    assert results[0] == want and results[1] == want
    # tensor parallelism beside the experts: attention is not data-parallel, whatever the flag says
    lay = mc.ParallelLayout(tp=2, ep=2, rank=0)
    assert lay.ep == 2

    class _C:       # a communicator is only stored by the constructor
        size = 4
    dec = Decoder(cfg, shard_model(full, cfg, lay, "cpu"), lay, num_pages=8, page_size=16, max_pos=64, comm=_C(), comm_moe=_C())
    dec.dp_attention = True
    assert dec.dp_ways() == 1 and not dec.dp_rows_ok(16)
