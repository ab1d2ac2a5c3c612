"""Prefill / decode disaggregation on two GPUs: rank 0 prefills a prompt and stores its KV pages into rank 1's page
pools over NVLink (PeerKvTransport, one launch per layer), rank 1 decodes from there. The tokens must equal a
single-GPU run of the same model (prefill and decode on one device)."""
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
from skein_b200.parallel.disagg import HeapKvPools, receive_prompt, ship_prompt  # noqa: E402
from skein_b200.runtime.runner import ModelRunner  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    cfg = mc.tiny_mixtral(layers=3, hidden=512, inter=1024, heads=8, kv_heads=2, experts=4, vocab=1024)
    w = random_weights(cfg, mc.ParallelLayout(), dev, seed=31, std=0.05)       # both ranks hold the same model
    pages, ps = 48, 16
    pools = HeapKvPools(dist.group.WORLD, dev, cfg.num_layers, pages, cfg.num_kv_heads, ps, cfg.head_dim)
    dec = Decoder(cfg, w, num_pages=pages, page_size=ps, max_pos=256, kv_pools=pools.pools)
    runner = ModelRunner(dec, max_blocks_per_seq=8, use_graphs=False)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=g).tolist()
    steps = 6
    table_p = [3, 4, 5, 6, 7, 8, 9, 10]            # pages on the prefill rank
    table_d = [20, 21, 22, 30, 31, 32, 33, 34]     # other page ids on the decode rank

    def decode_from(first, table):
        toks, cached = [first], len(prompt)
        bk = runner.bucket(1)
        for _ in range(steps):
            runner.load_decode_inputs(bk, [toks[-1]], [cached], [cached + 1], [table])
            toks.append(int(runner.decode_step(bk)[0]))
            cached += 1
        return toks

    if rank == 0:
        first = ship_prompt(runner, pools, 1, prompt, table_p, table_d)
        want = decode_from(first, table_p)         # the single-GPU run: decode where the prompt was prefilled
        got = [None]
        dist.broadcast_object_list(got, src=1)
        assert got[0] == want, (got[0], want)
    else:
        # poison the target pages first: what the decode reads must be what rank 0 stored
        for p in pools.pools:
            p[table_d[:3]] = float("nan")
        torch.cuda.synchronize()
        first, n = receive_prompt(pools, 0)
        assert n == len(prompt)
        got = decode_from(first, table_d)
        dist.broadcast_object_list([got], src=1)
    torch.cuda.synchronize()
    ops.workspace().check_status()
    dist.barrier()
    if rank == 0:
        print("DISAGG_WORKER_OK")
    pools.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
