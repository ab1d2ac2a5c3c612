"""Two CPU ranks (gloo) in lock step through the shared control page: rank 0 leads with an EngineDriver, rank 1
follows. Rank 1's step 2 fails (injected on the host); both ranks must drop the batch, re-arm, and go on serving
the same tokens. The payload broadcast must only happen on iterations that carry requests."""
import os
import sys
import threading

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from skein_b200.models import config as mc  # noqa: E402
from skein_b200.models.decoder import Decoder, random_weights  # noqa: E402
from skein_b200.parallel import launcher  # noqa: E402
from skein_b200.runtime.driver import EngineDriver, SharedControl, follower_loop  # noqa: E402
from skein_b200.runtime.engine import Engine, EngineConfig  # noqa: E402


def main():
    rank, world, rdv = launcher.world_from_env()
    launcher.init_process_group(rank, world, rdv, "gloo", timeout_s=60)
    group = dist.new_group(backend="gloo")
    cfg = mc.tiny_mixtral()
    dec = Decoder(cfg, random_weights(cfg, mc.ParallelLayout(), "cpu", seed=5, std=0.05), num_pages=64, page_size=16, max_pos=256)
    eng = Engine(dec, EngineConfig(max_batch=4, tpot_ms=1e6, use_graphs=False))
    control = SharedControl(str(rdv) + ".control", rank, world, group, wait_s=60)
    bcasts = {"n": 0}
    orig = control._bcast
    control._bcast = lambda p: (bcasts.__setitem__("n", bcasts["n"] + 1), orig(p))[1]
    resyncs = {"n": 0}

    def resync(ctl):
        ctl.barrier()
        resyncs["n"] += 1
        ctl.barrier()
    if rank == 1:
        def boom(step):
            if step == 2:
                raise RuntimeError("injected failure on rank 1")
        eng.failure_injector = boom
        follower_loop(eng, control, rank, resync)
        done = eng.metrics.render()
        assert 'skein_requests_total{status="failed"} 2' in done and 'skein_requests_total{status="ok"} 1' in done, done
    else:
        driver = EngineDriver(eng, control, rank=0, resync=resync).start()
        subs = [driver.submit([3, 4, 5, 6], 6), driver.submit([9, 8, 7], 6)]
        errors = []
        for rid, kind, reason, q in subs:
            while True:
                ev = q.get(timeout=60)
                if ev.is_final:
                    errors.append(ev.error)
                    break
        # rank 0's own step succeeded; it learns of rank 1's failure through the control page
        assert all(e and "another rank" in e for e in errors), errors
        rid, kind, reason, q = driver.submit([1, 2, 3], 4)
        toks = []
        while True:
            ev = q.get(timeout=60)
            assert ev.error is None
            toks.append(ev.token)
            if ev.is_final:
                break
        assert len(toks) == 4
        driver.stop()
        assert driver.error is None
        text = eng.metrics.render()
        assert 'skein_requests_total{status="failed"} 2' in text and "skein_step_failures_total 1" in text, text
    assert resyncs["n"] == 1, resyncs
    # payloads: the two submissions (one or two iterations), the third request, the stop
    assert bcasts["n"] <= 4, bcasts
    assert control.seq >= 8            # ... while the engines stepped many more times than that
    last = torch.tensor([eng._step], dtype=torch.int64)
    both = [torch.zeros_like(last) for _ in range(world)]
    dist.all_gather(both, last, group=group)
    assert int(both[0]) == int(both[1]), both       # the engines ran the same number of steps
    control.close()
    dist.barrier()
    if rank == 0:
        print("CONTROL_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
