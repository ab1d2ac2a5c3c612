"""Pipeline-parallel worker (gloo on CPU, or nccl on GPUs): pp stages reproduce the single-stage model, both
through the plain stage-by-stage step and through the micro-batched pipelined decode."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from skein_b200.models import config as mc  # noqa: E402
from skein_b200.models.decoder import BatchInputs, Decoder, random_weights  # noqa: E402
from skein_b200.models.sharding import shard_model  # noqa: E402
from skein_b200.parallel import launcher, pp  # noqa: E402
from skein_b200.runtime.runner import ModelRunner  # noqa: E402


def main():
    rank, world, rdv = launcher.world_from_env()
    use_cuda = os.environ.get("PP_WORKER_DEVICE", "cpu") == "cuda"
    dev = torch.device("cuda", launcher.local_device_index()) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    launcher.init_process_group(rank, world, rdv, "nccl" if use_cuda else "gloo", timeout_s=60, device=dev if use_cuda else None)
    cfg = mc.tiny_mixtral(layers=5)                      # 5 blocks over 2 stages: 3 + 2
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=21, std=0.05)
    lay = mc.ParallelLayout(pp=world, rank=rank)
    _, pp_ranks, pp_group = pp.make_groups((1, world, 1), rank)
    fb_group = dist.new_group(list(range(world)))
    dec = Decoder(cfg, shard_model(full, cfg, lay, dev), lay, num_pages=32, page_size=16, max_pos=128)
    stage = pp.PipelineStage(dec, lay, pp_ranks, pp_group)
    assert world != 2 or len(dec.w.layers) == (3 if rank == 0 else 2)
    g = torch.Generator().manual_seed(3)
    B = 4
    prompts = torch.randint(0, cfg.vocab_size, (B, 18), generator=g).tolist()
    tables = [[1 + 4 * s + i for i in range(4)] for s in range(B)]

    def gen(model, steps=4):
        runner = ModelRunner(model, max_blocks_per_seq=4, use_graphs=False)
        outs = [runner.prefill([(prompts[s], tables[s], 0) for s in range(B)])]
        bk, cached = runner.bucket(B), 18
        for _ in range(steps):
            runner.load_decode_inputs(bk, outs[-1], [cached] * B, [cached + 1] * B, tables)
            outs.append(runner.decode_step(bk)[:B].tolist())
            cached += 1
        return outs

    got = gen(stage)
    want = gen(Decoder(cfg, full, num_pages=32, page_size=16, max_pos=128)) if rank == 0 else None
    if rank == 0:
        assert got == want, (got, want)

    # micro-batched pipelined decode: 2 micro-batches of 2 sequences, continuing from a fresh prefill
    for kv in dec.kv:
        kv.zero_()
    runner = ModelRunner(stage, max_blocks_per_seq=4, use_graphs=False)
    first = runner.prefill([(prompts[s], tables[s], 0) for s in range(B)])
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    micro = []
    for m in range(2):
        rows = [2 * m, 2 * m + 1]
        bt = torch.zeros(2, 4, dtype=torch.int32, device=dev)
        for i, r in enumerate(rows):
            bt[i] = i32(tables[r])
        micro.append(BatchInputs(token_ids=i32([first[r] for r in rows]), positions=i32([18, 18]), block_table=bt, seq_lens=i32([19, 19])))

    def advance(inp, toks):
        if toks is not None:
            inp.token_ids.copy_(toks)
        inp.positions.add_(1)
        inp.seq_lens.add_(1)

    # in two calls: the second continues where the first stopped (its first step receives the fed-back tokens); the
    # stage compute runs as a captured graph from each micro-batch's second step on when the stages are on GPUs
    out = pp.pipelined_decode(stage, micro, 2, advance, fb_group, more=True)
    out += pp.pipelined_decode(stage, micro, 2, advance, fb_group, resume=True)
    if use_cuda:
        assert all(sg.graph is not None for k, sg in stage._graphs.items() if k[0] == "steady")
    if rank == world - 1:
        piped = [[int(x) for m in range(2) for x in out[t][m].tolist()] for t in range(4)]
    else:
        piped = None
    box = [piped]
    dist.broadcast_object_list(box, src=world - 1)
    if rank == 0:
        assert box[0] == want[1:], (box[0], want[1:])
        print("PP_WORKER_OK world", world)
    # the serving engine with one group of sequences per stage kept in flight across steps: every stage runs the same
    # engine; sequences of different lengths start, finish and arrive while others are on the device
    from skein_b200.runtime.engine import Engine, EngineConfig
    for kv in dec.kv:
        kv.zero_()
    stage.feedback_group = fb_group
    g2 = torch.Generator().manual_seed(5)
    reqs = [(torch.randint(0, cfg.vocab_size, (n,), generator=g2).tolist(), m) for n, m in ((18, 6), (7, 3), (11, 9), (5, 1), (9, 7), (14, 5))]
    late = [(torch.randint(0, cfg.vocab_size, (n,), generator=g2).tolist(), m) for n, m in ((6, 4), (12, 8))]

    def serve(model, continuous):
        eng = Engine(model, EngineConfig(max_batch=8, tpot_ms=1e9, ttft_ms=1e9, use_graphs=False, prefix_cache=False,
                                         pp_continuous=continuous))
        out, n_steps, most = {}, 0, 0
        for p_, m in reqs:
            eng.submit(p_, m)
        while not eng.idle and n_steps < 500:
            if n_steps == 3:
                for p_, m in late:
                    eng.submit(p_, m)
            for ev in eng.step():
                assert ev.error is None, ev
                out.setdefault(ev.request_id, []).append(ev.token)
            most = max(most, len(eng._flights))
            n_steps += 1
        assert eng.idle and not eng._flights and not eng._grp_of and sum(eng._grp_load) == 0
        return [out[i] for i in sorted(out)], most

    def near_tie(prompt, want_seq, got_seq, tol=0.05):
        """True when the two generations part at a step where the single-stage model, given the common prefix, scores the
        two tokens within `tol` of each other (bf16 spacing at these logits is 0.016). The groups of the continuous engine
        are smaller batches than the single-stage engine's, so on GPUs the GEMMs round differently and such a step may
        go either way; on CPU the arithmetic does not depend on the batch and the generations are equal."""
        i = next(j for j, (a_, b_) in enumerate(zip(want_seq, got_seq)) if a_ != b_)
        ref = Decoder(cfg, full if dev.type == "cpu" else shard_model(full, cfg, mc.ParallelLayout(), dev), num_pages=16, page_size=16, max_pos=128)
        _, lg = ModelRunner(ref, max_blocks_per_seq=4, use_graphs=False).prefill([(prompt + want_seq[:i], [1, 2, 3, 4], 0)], want_logits=True)
        row = lg[-1].float().flatten()
        return abs(float(row[want_seq[i]]) - float(row[got_seq[i]])) <= tol and float(row.max()) - float(row[got_seq[i]]) <= tol

    got_c, most = serve(stage, True)
    assert most == world - 1 or world == 1, most       # a step launches every idle group and collects one: pp - 1 stay in flight
    assert [len(x) for x in got_c] == [m for _, m in reqs + late]
    if rank == 0:
        want_c, _ = serve(Decoder(cfg, full, num_pages=32, page_size=16, max_pos=128), False)
        prompts_c = [p_ for p_, _ in reqs + late]
        diff = [i for i, (a_, b_) in enumerate(zip(got_c, want_c)) if a_ != b_]
        if use_cuda:
            assert len(diff) <= 2 and all(near_tie(prompts_c[i], want_c[i], got_c[i]) for i in diff), (got_c, want_c)
        else:
            assert not diff, (got_c, want_c)
        # the excuse itself: the runner-up of a close step passes, an arbitrary token does not
        close = [255, 131, 131, 131, 131, 457]      # parts from the single-stage generation where 457 and 131 score 2.359 / 2.344
        if not use_cuda and want_c[0][:3] == [255, 131, 457]:
            assert near_tie(prompts_c[0], want_c[0], close) and not near_tie(prompts_c[0], want_c[0], [255, 131, 7, 0, 0, 0])
        print("PP_CONTINUOUS_OK world", world)

    # a step that fails (on every stage: the lock-step control plane makes a failure of one rank a failure of all) while
    # groups are on the device: their launches are waited for and dropped, the requests end with an error, and the
    # engine serves the next request as if nothing had happened
    for kv in dec.kv:
        kv.zero_()
    eng = Engine(stage, EngineConfig(max_batch=8, tpot_ms=1e9, ttft_ms=1e9, use_graphs=False, prefix_cache=False, pp_continuous=True))
    for p_, m in reqs[:4]:
        eng.submit(p_, 8)

    def boom(step):
        if step == 3:
            raise RuntimeError("injected")
    eng.failure_injector = boom
    errs, n_steps = [], 0
    while not eng.idle and n_steps < 50:
        errs += [ev for ev in eng.step() if ev.error is not None]
        n_steps += 1
    assert len(errs) == 4 and not eng._flights and not eng._grp_of, (errs, n_steps)
    eng.failure_injector = None
    rid, _ = eng.submit(reqs[2][0], 9)
    after = eng.run_until_done()[rid]
    if rank == 0 and not use_cuda:
        assert after == want_c[2], (after, want_c[2])
        print("PP_CONTINUOUS_FAILURE_OK world", world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
