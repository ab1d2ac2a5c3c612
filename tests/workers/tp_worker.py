"""Multi-GPU worker (one process per GPU, launched by torch.distributed.run from test_tp_gpu.py).

Checks, on every rank:
  1. stand-alone push all-reduce equals the sum of the ranks' inputs
  2. fused GEMM -> push -> reduce+residual+RMSNorm equals the fp32 reference of the unsharded op
     (dense and grouped / MoE-combine forms): "TP shards summed equal the full op", the property the
     reference tests on CPU in crates/skein_emit/tests/op_numerics.rs:299,371
  3. vocabulary-parallel argmax equals argmax of the gathered logits (vocab_parallel.rs:56)
  4. a tiny Mixtral served TP=N (CUDA-graph decode, fused collectives) produces the same tokens as the
     unsharded CPU reference graph
"""
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
from skein_b200.parallel.tp import TPComm  # noqa: E402
from skein_b200.runtime.runner import ModelRunner  # noqa: E402


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-9))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    H = 1024
    comm = TPComm(dist.group.WORLD, dev, hidden=H, fused_rows=256, max_batch=64,
                  mode=os.environ.get("SKEIN_COMM", "fused"))
    g = torch.Generator().manual_seed(7)

    # 1. stand-alone all-reduce (several rounds so both buffers and epochs cycle)
    for it in range(5):
        xs = [torch.randn(40, H, generator=g).bfloat16() for _ in range(world)]
        y = comm.all_reduce(xs[rank].to(dev))
        want = torch.stack([x.float() for x in xs]).sum(0)
        assert rel(y, want) < 1e-2, ("all_reduce", it, rel(y, want))

    # 2a. dense row-parallel projection
    T, K = 48, 512 * world
    x_full = torch.randn(T, K, generator=g).bfloat16()
    w_full = (torch.randn(H, K, generator=g) / 32).bfloat16()
    res = torch.randn(T, H, generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    ks = slice(rank * 512, (rank + 1) * 512)
    for it in range(3):
        part, flags, epoch = comm.linear_push(x_full[:, ks].contiguous().to(dev), w_full[:, ks].contiguous().to(dev))
        r1, n1 = ops.reduce_residual_rmsnorm(res.to(dev), part, gamma.to(dev), 1e-5, flags=flags, epoch=epoch)
        r2, n2 = ref.reduce_residual_rmsnorm(res, ref.linear(x_full, w_full).unsqueeze(0), gamma, 1e-5)
        assert rel(r1, r2) < 2e-2 and rel(n1, n2) < 2e-2, ("dense", it, rel(r1, r2), rel(n1, n2))

    # 2a'. the same projection through the block-scaled fp8 GEMM with the publish epilogue
    from skein_b200.ops import fp8
    w8 = fp8.quantize_weight(w_full[:, ks].contiguous().to(dev))
    xq, xsc = ops.quant_fp8_block128(x_full[:, ks].contiguous().to(dev))
    for it in range(2):
        part, flags, epoch = comm.linear_push_fp8(xq, xsc, w8)
        r1, n1 = ops.reduce_residual_rmsnorm(res.to(dev), part, gamma.to(dev), 1e-5, flags=flags, epoch=epoch)
        r2, n2 = ref.reduce_residual_rmsnorm(res, ref.linear(x_full, w_full).unsqueeze(0), gamma, 1e-5)
        assert rel(r1, r2) < 6e-2 and rel(n1, n2) < 6e-2, ("fp8 dense", it, rel(r1, r2), rel(n1, n2))

    # 2b. grouped (MoE down projection + top-2 combine)
    E, topk, Kp = 4, 2, 256
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, topk, generator=g)
    counts, offsets, row_of, src = ref.router_plan(ids, E)
    rows = T * topk
    h_full = torch.randn(rows, Kp * world, generator=g).bfloat16()
    w2_full = (torch.randn(E, H, Kp * world, generator=g) / 32).bfloat16()
    kp = slice(rank * Kp, (rank + 1) * Kp)
    part, flags, epoch = comm.linear_push(h_full[:, kp].contiguous().to(dev), w2_full[:, :, kp].contiguous().to(dev),
                                          (counts.to(dev), offsets.to(dev)))
    r1, n1 = ops.reduce_residual_rmsnorm(res.to(dev), part, gamma.to(dev), 1e-5, row_of.view(T, topk).to(dev),
                                         wts.to(dev), flags=flags, epoch=epoch)
    y_full = ref.grouped_linear(h_full, w2_full, counts, offsets)
    r2, n2 = ref.reduce_residual_rmsnorm(res, y_full.unsqueeze(0), gamma, 1e-5, row_of.view(T, topk), wts)
    assert rel(r1, r2) < 2e-2 and rel(n1, n2) < 2e-2, ("grouped", rel(r1, r2), rel(n1, n2))

    # 3. vocabulary-parallel argmax
    V_local = 1000
    logits = torch.randn(world, 16, V_local, generator=g).bfloat16()
    tok = comm.vocab_parallel_argmax(logits[rank].to(dev), V_local)
    want = ref.sample_argmax(torch.cat(list(logits), dim=1))
    assert torch.equal(tok.cpu(), want), "vocab-parallel argmax"

    # 4. tiny Mixtral, TP = world, graph decode with fused collectives vs the CPU reference graph
    from skein_b200.parallel.selfcheck import teacher_forced_check
    info = teacher_forced_check(world, rank, dev, comm=comm, tp=world, hidden=H)
    assert info["tokens_compared"] == 21

    # 5. sequence-parallel dataflow (prefill-sized chunks): reduce-scatter fused with residual + RMSNorm on this rank's
    #    row slice, all-gather of the normalised slices; against the fp32 reference of the unsharded op
    if comm.mode != "nccl":
        T2 = 100                                    # not a multiple of the rank count: the last slice is short
        x2 = torch.randn(T2, K, generator=g).bfloat16()
        res2 = torch.randn(T2, H, generator=g).bfloat16()
        part, _, _ = comm.linear_push(x2[:, ks].contiguous().to(dev), w_full[:, ks].contiguous().to(dev))
        r0, n, per = comm.sp_slice(T2)
        res_loc, normed_loc = comm.reduce_scatter_norm(res2[r0:r0 + n].to(dev), part, gamma.to(dev), 1e-5, T2)
        full = comm.gather_rows(normed_loc, T2)
        r_ref, n_ref = ref.reduce_residual_rmsnorm(res2, ref.linear(x2, w_full).unsqueeze(0), gamma, 1e-5)
        assert res_loc.shape[0] == n and full.shape[0] == T2
        assert rel(res_loc, r_ref[r0:r0 + n]) < 2e-2 and rel(full, n_ref) < 2e-2, ("sp dense", rel(full, n_ref))
        # MoE combine form: partial rows are addressed through row_idx
        part, _, _ = comm.linear_push(h_full[:, kp].contiguous().to(dev), w2_full[:, :, kp].contiguous().to(dev),
                                      (counts.to(dev), offsets.to(dev)))
        r0, n, per = comm.sp_slice(T)
        res_loc, normed_loc = comm.reduce_scatter_norm(res[r0:r0 + n].to(dev), part, gamma.to(dev), 1e-5, T,
                                                       row_of.view(T, topk).to(dev), wts.to(dev))
        full = comm.gather_rows(normed_loc, T)
        assert rel(full, n2) < 2e-2, ("sp grouped", rel(full, n2))
        # the whole model with its prefill on the sequence-parallel path (63 prompt tokens > the threshold below)
        comm.sp_min_rows = 16
        info = teacher_forced_check(world, rank, dev, comm=comm, tp=world, hidden=H, seed=12)
        assert info["tokens_compared"] == 21
        comm.sp_min_rows = 512
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK world", world, "mode", comm.mode, "multimem", int(comm.heap.mc_ptr != 0))
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    if os.environ.get("SKEIN_MULTIMEM") == "1":
        # A rank must not leave while its heap is bound to the multicast object and a peer may still read through the
        # switch: on a failure, stay alive until the peers' bounded waits (10 s) have run out, then report.
        try:
            main()
        except BaseException:
            import time
            import traceback
            traceback.print_exc()
            sys.stdout.flush()
            time.sleep(15)
            os._exit(1)
    else:
        main()
