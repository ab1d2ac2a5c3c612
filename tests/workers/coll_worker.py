"""Stand-alone NVLink collectives on N GPUs: publish + pull all-reduce, all-gather, reduce-scatter and all-to-all
against torch.distributed's results, interleaved and repeated (the two published buffers alternate, the epochs grow),
plus the library fallback for messages larger than the published buffer.

The reference does these exchanges with NCCL calls (crates/skein_runtime/src/cuda/nccl.rs:196-298, 422-445).
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from skein_b200 import ops  # noqa: E402
from skein_b200.ops import _lib  # noqa: E402
from skein_b200.parallel.tp import TPComm  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    H = 1024
    comm = TPComm(dist.group.WORLD, dev, hidden=H, fused_rows=256, max_batch=64, wait_budget_ms=2000)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    launches0 = _lib.launches()
    for it in range(6):
        rows = 8 * world * (it + 1)                      # divisible by the world size; different every round
        x = torch.randn(rows, H, device=dev, generator=g).bfloat16()

        want = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(want, x)
        got = comm.all_gather(x)
        assert torch.equal(got, torch.cat(want)), f"all_gather round {it}"

        full = want[0].float()                           # every rank's x, summed in rank order in fp32
        for w in want[1:]:
            full = full + w.float()
        per = rows // world
        rs = comm.reduce_scatter(x)
        assert rs.shape == (per, H)
        assert torch.equal(rs, full[rank * per:(rank + 1) * per].bfloat16()), f"reduce_scatter round {it}"

        a2a_want = torch.empty_like(x)
        dist.all_to_all_single(a2a_want, x)
        assert torch.equal(comm.all_to_all(x), a2a_want), f"all_to_all round {it}"

        ar = comm.all_reduce(x)
        assert torch.equal(ar, full.bfloat16()), f"all_reduce round {it}"

        ids = torch.arange(rank * 5, rank * 5 + 20, device=dev, dtype=torch.int32).view(4, 5).contiguous()   # 80 bytes
        want_i = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(want_i, ids)
        assert torch.equal(comm.all_gather(ids), torch.cat(want_i)), "all_gather of int32 rows"
    torch.cuda.synchronize()
    ops.workspace().check_status()
    assert _lib.launches() - launches0 >= 6 * 5 * 2, "the peer-memory kernels did not run"

    # larger than the published buffer (256 rows): the library path, same results
    big = torch.randn(64 * world * 8, H, device=dev, generator=g).bfloat16()
    want = [torch.empty_like(big) for _ in range(world)]
    dist.all_gather(want, big)
    assert torch.equal(comm.all_gather(big), torch.cat(want))
    per = big.shape[0] // world
    lib = comm.reduce_scatter(big).float()
    ref = torch.stack(want).float().sum(0)[rank * per:(rank + 1) * per]
    assert (lib - ref).abs().max() <= 0.05 * ref.abs().max()
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        print("COLL_WORKER_OK")


if __name__ == "__main__":
    main()
