"""Two GPUs, one of which stops taking part: the other's bounded peer wait must run out and surface as an error.

Rank 1 stays alive (its memory stays mapped, nothing faults) but skips a decode step. Rank 0 runs the step: its GEMM
publishes as usual, its reduce kernel waits 300 ms for rank 1's flag, records the timeout in the status word and
returns; later kernels of the step give up at once; the host read of the status word raises. No kernel hangs, no rank
exits with work in flight. The reference's shared-memory all-reduce spins forever in this situation
(crates/skein_runtime/src/cuda/shm_allreduce.rs:53).
"""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from skein_b200 import ops  # noqa: E402
from skein_b200.models import config as mc  # noqa: E402
from skein_b200.models.decoder import Decoder, random_weights  # noqa: E402
from skein_b200.models.sharding import shard_model  # noqa: E402
from skein_b200.parallel.tp import TPComm  # noqa: E402
from skein_b200.runtime.runner import ModelRunner  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    # the control plane runs on gloo: nothing on the GPUs depends on a library collective here
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    H = 1024
    comm = TPComm(dist.group.WORLD, dev, hidden=H, fused_rows=256, max_batch=64, wait_budget_ms=300)
    cfg = mc.tiny_mixtral(layers=2, hidden=H, inter=1024, heads=8, kv_heads=2, experts=4, vocab=1024)
    full = random_weights(cfg, mc.ParallelLayout(), "cpu", seed=5, std=0.05)
    lay = mc.ParallelLayout(tp=2, rank=rank)
    dec = Decoder(cfg, shard_model(full, cfg, lay, dev), lay, num_pages=16, page_size=16, max_pos=128, comm=comm)
    runner = ModelRunner(dec, max_blocks_per_seq=4, use_graphs=False)
    B = 2
    prompts = [[3, 5, 7, 9, 11], [2, 4, 6, 8, 10]]
    tables = [[1, 2, 3, 4], [5, 6, 7, 8]]
    toks = runner.prefill([(prompts[s], tables[s], 0) for s in range(B)])
    bk = runner.bucket(B)
    runner.load_decode_inputs(bk, toks, [5] * B, [6] * B, tables)
    first = runner.decode_step(bk)[:B].tolist()          # both ranks: a healthy step
    torch.cuda.synchronize()
    ops.workspace().check_status()
    dist.barrier()

    if rank == 0:
        runner.load_decode_inputs(bk, first, [6] * B, [7] * B, tables)
        t0 = time.monotonic()
        try:
            runner.decode_step(bk)
            torch.cuda.synchronize()
            ops.workspace().check_status()
            raise AssertionError("the step finished although rank 1 never published")
        except RuntimeError as e:
            took = time.monotonic() - t0
            assert "peer flag" in str(e), e
            assert took < 5.0, f"one wait budget expected, the step took {took:.1f} s"
        # the context is still usable: a local kernel runs and the status word is clean again
        y = ops.rmsnorm(torch.ones(4, H, device=dev, dtype=torch.bfloat16), torch.ones(H, device=dev, dtype=torch.bfloat16), 1e-5)
        torch.cuda.synchronize()
        ops.workspace().check_status()
        assert torch.isfinite(y.float()).all()
        print("TP_TIMEOUT_OK", round(took, 2))
    dist.barrier()          # rank 1 only leaves after rank 0 is done with its memory
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
