"""Decoder graph checks.

CPU: the operator-interface graph (paged KV, prefill chunks + decode steps) against the cache-free
dense reference; decode-with-cache equals full prefill (the reference's kv_cache.rs:14 property).
GPU: the same graph on the CUDA kernels against the CPU oracle, eager and through CUDA graphs.
"""
import pytest
import torch

from skein_b200.models import config as mc
from skein_b200.models.decoder import Decoder, random_weights
from skein_b200.models.dense_reference import forward_full
from skein_b200.runtime.runner import ModelRunner


def _build(cfg, device, num_pages=64, seed=0, std=0.05):
    w = random_weights(cfg, mc.ParallelLayout(), device, seed=seed, std=std)
    dec = Decoder(cfg, w, num_pages=num_pages, page_size=16, max_pos=512)
    return w, dec


def _run_sequence(dec, ids, chunk_sizes, n_decode):
    """Prefill `ids` in chunks, then decode greedily. Returns (logits after prefill, decoded tokens)."""
    runner = ModelRunner(dec, max_blocks_per_seq=8, use_graphs=False)
    table = [3, 7, 1, 9, 12, 20, 33, 40]
    cached, lg = 0, None
    for c in chunk_sizes:
        toks, lg = runner.prefill([(ids[cached:cached + c], table, cached)], want_logits=True)
        cached += c
    out = [toks[0]]
    bk = runner.bucket(1)
    for _ in range(n_decode):
        runner.load_decode_inputs(bk, [out[-1]], [cached], [cached + 1], [table])
        res = runner.decode_step(bk)
        cached += 1
        out.append(int(res[0]))
    return lg, out


@pytest.mark.parametrize("cfg", [mc.tiny_mixtral(), mc.tiny_llama()], ids=["mixtral", "llama"])
def test_graph_matches_dense_reference_cpu(cfg):
    torch.manual_seed(0)
    w, dec = _build(cfg, "cpu")
    ids = torch.randint(0, cfg.vocab_size, (37,)).tolist()
    ref_logits = forward_full(cfg, w, torch.tensor(ids))
    lg, _ = _run_sequence(dec, ids, [37], 0)
    a, b = lg[0].float(), ref_logits[-1]
    assert float((a - b).norm() / b.norm()) < 0.05
    assert int(a.argmax()) == int(b.argmax())


def test_chunked_prefill_and_decode_equal_full_prefill_cpu():
    cfg = mc.tiny_mixtral()
    torch.manual_seed(1)
    w, dec = _build(cfg, "cpu")
    ids = torch.randint(0, cfg.vocab_size, (40,)).tolist()
    lg_full, toks_full = _run_sequence(dec, ids, [40], 3)
    w2, dec2 = _build(cfg, "cpu")
    lg_chunk, toks_chunk = _run_sequence(dec2, ids, [16, 5, 19], 3)
    assert float((lg_full.float() - lg_chunk.float()).abs().max()) < 0.05
    assert toks_full == toks_chunk
    # greedy continuation equals the dense reference's greedy continuation
    seq = list(ids)
    for t in toks_full[:3]:
        nxt = int(forward_full(cfg, w, torch.tensor(seq))[-1].argmax())
        assert nxt == t
        seq.append(t)


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [mc.tiny_mixtral(), mc.tiny_llama()], ids=["mixtral", "llama"])
def test_graph_gpu_matches_cpu(cfg):
    torch.manual_seed(2)
    w_cpu, dec_cpu = _build(cfg, "cpu", seed=3)
    w_gpu, dec_gpu = _build(cfg, "cuda", seed=3)
    # same weights on both devices
    for lc, lg_ in zip(w_cpu.layers, w_gpu.layers):
        for name in ("attn_norm", "wqkv", "wo", "ffn_norm", "router", "w13", "w2"):
            t = getattr(lg_, name)
            if t is not None:
                getattr(lc, name).copy_(t.cpu())
    w_cpu.embed.copy_(w_gpu.embed.cpu()); w_cpu.lm_head.copy_(w_gpu.lm_head.cpu()); w_cpu.final_norm.copy_(w_gpu.final_norm.cpu())
    ids = torch.randint(0, cfg.vocab_size, (70,)).tolist()
    lg_c, toks_c = _run_sequence(dec_cpu, ids, [70], 4)
    lg_g, toks_g = _run_sequence(dec_gpu, ids, [33, 37], 4)
    from skein_b200 import ops
    torch.cuda.synchronize(); ops.workspace().check_status()
    rel = float((lg_g.float().cpu() - lg_c.float()).norm() / lg_c.float().norm())
    assert rel < 0.05, rel
    assert toks_c == toks_g


@pytest.mark.gpu
def test_cuda_graph_decode_equals_eager():
    cfg = mc.tiny_mixtral()
    w, dec = _build(cfg, "cuda", seed=5)
    ids = torch.randint(0, cfg.vocab_size, (3, 20)).tolist()
    tables = [[1, 2, 3], [4, 5, 6], [7, 8, 9]]

    def run(use_graphs):
        for kv in dec.kv:
            kv.zero_()
        runner = ModelRunner(dec, max_blocks_per_seq=4, use_graphs=use_graphs)
        first = runner.prefill([(ids[i], tables[i], 0) for i in range(3)])
        bk = runner.bucket(3)
        outs = [first]
        cached = 20
        for _ in range(5):
            runner.load_decode_inputs(bk, outs[-1], [cached] * 3, [cached + 1] * 3, tables)
            outs.append(runner.decode_step(bk)[:3].tolist())
            cached += 1
        return outs, runner

    eager, _ = run(False)
    graphed, r = run(True)
    assert eager == graphed
    assert r.graph_captures == 1 and r.graph_replays == 5
    # device-side feedback loop gives the same continuation
    for kv in dec.kv:
        kv.zero_()
    runner = ModelRunner(dec, max_blocks_per_seq=4, use_graphs=True)
    first = runner.prefill([(ids[i], tables[i], 0) for i in range(3)])
    bk = runner.bucket(3)
    runner.load_decode_inputs(bk, first, [20] * 3, [21] * 3, tables)
    bk.dev_in.copy_(bk.host_in)
    loop = [first]
    for _ in range(5):
        runner.decode_loop_step(bk)
        loop.append(bk.dev_out[:3].tolist())
    assert loop == eager


def test_fp8_blocks_track_the_bf16_model_cpu():
    """Blocks switched to block-scaled e4m3 weights (and on-the-fly quantised activations) stay close to bf16."""
    from skein_b200.models.decoder import quantize_blocks
    cfg = mc.tiny_mixtral(layers=3)
    torch.manual_seed(4)
    w, dec = _build(cfg, "cpu", seed=8)
    ids = torch.randint(0, cfg.vocab_size, (30,)).tolist()
    lg_bf16, _ = _run_sequence(dec, ids, [30], 0)
    w8, dec8 = _build(cfg, "cpu", seed=8)
    quantize_blocks(w8, [1, 2])
    assert w8.layers[1].w13 is None and "w13" in w8.layers[1].fp8 and not w8.layers[0].fp8
    lg_fp8, _ = _run_sequence(dec8, ids, [30], 0)
    a, b = lg_fp8.float(), lg_bf16.float()
    assert 0 < float((a - b).norm() / b.norm()) < 0.15
