"""Expert parallelism with data-parallel attention on N GPUs (one process per GPU).

1. Dispatch / combine round trip with identity experts: every rank publishes its own tokens' rows and expert choices,
   the pull kernel gathers the rows routed to this rank's experts, the "experts" return their input, and the
   owner-aware combine with weights that sum to one must give every token back its own row (the reference's
   round-trip property, crates/skein_emit/tests/ep_routing.rs:14,68).
2. A tiny Mixtral served EP = N through the engine with data-parallel attention (each rank runs attention and keeps the
   decode cache for its own slice of the sequences, CUDA-graph decode, token dispatch over peer memory) produces the
   tokens of the unsharded CPU model.
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from skein_b200 import ops  # noqa: E402
from skein_b200.models import config as mc  # noqa: E402
from skein_b200.models.decoder import Decoder, random_weights  # noqa: E402
from skein_b200.models.sharding import shard_model  # noqa: E402
from skein_b200.ops import reference as ref  # noqa: E402
from skein_b200.parallel.tp import PeerPartials, TPComm  # noqa: E402
from skein_b200.runtime.engine import Engine, EngineConfig  # noqa: E402


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-9))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    H, E, k, per = 512, 2 * world, 2, 8
    comm = TPComm(dist.group.WORLD, dev, hidden=H, fused_rows=1024, max_batch=64)
    g = torch.Generator().manual_seed(3)
    T = world * per
    x_all = torch.randn(T, H, generator=g).bfloat16()
    ids_all = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    w_all = torch.rand(T, k, generator=g)
    w_all = w_all / w_all.sum(-1, keepdim=True)
    e_local = E // world
    lo, hi = rank * per, (rank + 1) * per
    for it in range(3):       # several rounds: both buffers and the epochs cycle
        def fill(normed_view, ids_view):
            normed_view.copy_(x_all[lo:hi].to(dev))
            ids_view.copy_(ids_all[lo:hi].to(dev))
        got_ids, counts, offsets, row_of, src_token, xs = comm.ep_dispatch(per, k, E, rank * e_local, e_local, fill)
        c_ref, o_ref, row_ref, src_ref = ref.router_plan(ids_all, E)
        assert torch.equal(got_ids.cpu(), ids_all) and torch.equal(counts.cpu(), c_ref) and torch.equal(offsets.cpu(), o_ref)
        assert torch.equal(row_of.cpu(), row_ref)
        # the rows of this rank's experts hold their tokens' vectors, at the global positions
        r0, r1 = int(o_ref[rank * e_local]), int(o_ref[(rank + 1) * e_local])
        assert torch.equal(src_token[r0:r1].cpu(), src_ref[r0:r1])
        assert torch.equal(xs[r0:r1].cpu(), x_all[src_ref[r0:r1].long()])
        # identity experts: publish the gathered rows unchanged, combine with weights that sum to one
        b = comm.cur
        comm.cur ^= 1
        comm.bufs[b][:T * k].copy_(xs)
        from skein_b200.ops import _lib
        _lib.check(_lib.lib().skein_publish_rows(None, 0, None, comm._push_flag[b], world, comm.epochs[b:b + 1].data_ptr(),
                                                 comm.done[b:b + 1].data_ptr(), _lib.stream_ptr()), "publish")
        part = comm._partials(b, T * k)
        res = torch.zeros(per, H, dtype=torch.bfloat16, device=dev)
        out, _ = ops.reduce_residual_rmsnorm(res, part, None, 0.0, row_of.view(T, k)[lo:hi].contiguous(), w_all[lo:hi].to(dev),
                                             flags=part.flags, epoch=part.epoch, owner_ids=got_ids[lo:hi].contiguous(),
                                             experts_per_owner=e_local, owner_span=1)
        assert rel(out, x_all[lo:hi]) < 1e-2, ("identity round trip", it, rel(out, x_all[lo:hi]))
    torch.cuda.synchronize()
    ops.workspace().check_status()

    # 2. the model through the engine
    cfg = mc.tiny_mixtral(layers=2, hidden=H, inter=512, heads=8, kv_heads=2, experts=E, vocab=1024)
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=11, std=0.05)
    lay = mc.ParallelLayout(tp=1, ep=world, rank=rank)
    dec = Decoder(cfg, shard_model(full, cfg, lay, dev), lay, num_pages=96, page_size=16, max_pos=256, comm_moe=comm)
    dec.dp_attention = True
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 9, 33, 17, 12, 26, 30, 8, 15)]
    eng = Engine(dec, EngineConfig(max_batch=16, tpot_ms=1e9, ttft_ms=1e9, use_graphs=True, prefix_cache=False))
    assert eng._dp == world
    got = eng.generate(prompts, 6)
    torch.cuda.synchronize()
    ops.workspace().check_status()
    assert eng.runner.graph_replays > 0
    if rank == 0:
        want = Engine(Decoder(cfg, full, num_pages=96, page_size=16, max_pos=256),
                      EngineConfig(max_batch=16, tpot_ms=1e9, ttft_ms=1e9, use_graphs=False, prefix_cache=False)).generate(prompts, 6)
        # free-running comparison: a router near-tie may flip a token under bf16 rounding, after which that sequence
        # diverges, so most sequences must agree in full here; the strict check is the teacher-forced one below
        same = sum(a == b for a, b in zip(got, want))
        assert all(a[0] == b[0] for a, b in zip(got, want)) or same >= (2 * len(prompts)) // 3, ("got", got, "want", want)
        assert same >= len(prompts) // 2, ("got", got, "want", want)     # with 2 x ranks experts near-ties are frequent
    dist.barrier()

    # 3. the same layout teacher-forced with the CPU model's tokens, every mismatch explained by a near-tie
    from skein_b200.parallel.selfcheck import teacher_forced_check
    info = teacher_forced_check(world, rank, dev, comm_moe=comm, tp=1, ep=world, hidden=H, dp_attention=True)
    assert info["dp_attention"] and info["graph_replays"] > 0, info
    dist.barrier()
    if rank == 0:
        print("EP_DP_WORKER_OK world", world)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
