"""HTTP front end and hot swap on CPU: JSON and SSE completions, /metrics, 429 on rejection, 400 on bad bodies,
a step failure closes the stream with an error while the server keeps serving; hot swap rejects incompatible
artifacts, drains under load, and leaves the old artifact mounted when the drain times out.

Mirrors crates/skein_runtime/tests/{serve_driver.rs:43-239, hotswap_drain.rs:55-142, observability_metrics.rs:14}.
"""
import asyncio
import json
import threading
import time
from pathlib import Path

import pytest
import torch

from skein_b200 import core
from skein_b200.compile.artifact import Artifact, build_artifact
from skein_b200.models.decoder import Decoder
from skein_b200.runtime.engine import Engine, EngineConfig
from skein_b200.runtime.hotswap import HotSwap, HotSwapError
from skein_b200.runtime.server import EngineDriver, build_app
from skein_b200.runtime.tokenizer import Tokenizer

ROOT = Path(__file__).resolve().parent.parent
TINY = json.dumps({"architectures": ["LlamaForCausalLM"], "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
                   "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 300, "rope_theta": 5e5,
                   "rms_norm_eps": 1e-5, "max_position_embeddings": 256})
INPUTS = ((ROOT / "cluster/b200_1x.toml").read_text(), (ROOT / "cluster/sample_trace.jsonl").read_text(),
          (ROOT / "models/llama3_70b_drift.toml").read_text(), (ROOT / "cluster/cost_constants.toml").read_text())


def make_artifact(tmp_path, seed=0, batch=4, cfg=TINY):
    from skein_b200.compile.artifact import WeightSource
    from skein_b200.models.config import ModelConfig
    plan = core.extract_plan(cfg, *INPUTS, {"force_batch": batch}, [["bf16", "bf16", "bf16"]])["plan_json"]
    c = ModelConfig.from_hf_dict(json.loads(cfg))
    return Artifact(build_artifact(plan, cfg, tmp_path, WeightSource(c, seed=seed, std=0.05)))


def make_engine(art, **kw):
    dec = Decoder(art.cfg, art.load_weights(0, "cpu"), art.layout(0), num_pages=64, page_size=16, max_pos=256)
    return Engine(dec, EngineConfig(max_batch=4, tpot_ms=1e6, use_graphs=False, **kw))


def test_tokenizer_fallback():
    t = Tokenizer(300)
    assert t.is_fallback and t.encode("hi") == [104, 105] and t.decode([104, 105]) == "hi"
    assert Tokenizer(50).encode("hi") == [104 % 50, 105 % 50]


def test_streamed_text_is_decoded_incrementally(tmp_path):
    """The pieces of a stream add up to the decode of the whole: the space in front of a sentencepiece token and a
    character spread over several byte tokens are not lost."""
    from tokenizers import Tokenizer as HFTokenizer
    from tokenizers import decoders
    from tokenizers.models import WordLevel

    from skein_b200.runtime.tokenizer import IncrementalDecoder
    hf = HFTokenizer(WordLevel({"\u2581hello": 0, "\u2581wor": 1, "ld": 2, "<unk>": 3}, unk_token="<unk>"))
    hf.decoder = decoders.Metaspace()
    f = tmp_path / "tokenizer.json"
    hf.save(str(f))
    t = Tokenizer(4, f)
    assert t.decode([1]) == "wor"                                # one token at a time the space is gone
    d = IncrementalDecoder(t)
    assert [d.push(i) for i in (0, 1, 2, 0)] == ["hello", " wor", "ld", " hello"]
    fb = IncrementalDecoder(Tokenizer(300))                       # byte tokens: "h", then the two bytes of e-acute, then "!"
    assert [fb.push(b) for b in "h\u00e9!".encode()] == ["h", "", "\u00e9", "!"]


def test_http_completions_stream_metrics_and_errors(tmp_path):
    from aiohttp.test_utils import TestClient, TestServer

    art = make_artifact(tmp_path)
    eng = make_engine(art)
    driver = EngineDriver(eng).start()

    async def scenario():
        async with TestClient(TestServer(build_app(driver, Tokenizer(300)))) as c:
            r = await c.post("/v1/completions", json={"prompt": "hello", "max_tokens": 3})
            assert r.status == 200
            body = await r.json()
            assert len(body["tokens"]) == 3 and isinstance(body["text"], str)
            r = await c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 4, "stream": True})
            assert r.status == 200 and r.headers["Content-Type"].startswith("text/event-stream")
            events = [json.loads(l[6:]) for l in (await r.text()).splitlines() if l.startswith("data: ")]
            assert len(events) == 4 and events[-1]["is_final"] and not events[0]["is_final"] and all("token" in e for e in events)
            assert (await c.post("/v1/completions", json={"max_tokens": 3})).status == 400
            assert (await c.post("/v1/completions", data=b"not json")).status == 400
            r = await c.post("/v1/completions", json={"prompt": [5, 300, 7], "max_tokens": 2})      # vocabulary is 300
            assert r.status == 400 and "token ids" in (await r.json())["error"]["message"]
            assert (await c.post("/v1/completions", json={"prompt": [-1], "max_tokens": 2})).status == 400
            r = await c.post("/v1/completions", json={"prompt": [1] * 250, "max_tokens": 100})
            assert r.status == 429                               # prompt + max_tokens beyond the position limit
            m = await (await c.get("/metrics")).text()
            assert 'skein_requests_total{status="ok"} 2' in m and "skein_steps_total" in m and "skein_kv_pages_in_use" in m
            assert (await (await c.get("/healthz")).json())["ok"]
            # a failing step: the stream ends with an error event, the next request is served
            eng.failure_injector = lambda step: (_ for _ in ()).throw(RuntimeError("boom"))
            r = await c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 3})
            assert r.status == 503 and "boom" in (await r.json())["error"]["message"]
            eng.failure_injector = None
            assert (await c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 2})).status == 200

    try:
        asyncio.run(asyncio.wait_for(scenario(), 120))
    finally:
        driver.stop()


def test_generation_ends_at_the_models_end_of_sequence_token(tmp_path):
    """`eos_token_id` of the checkpoint's config ends a generation (finish_reason "stop") when the artifact ships the
    model's tokenizer; an artifact without one (byte tokens, random weights) has no such token, and --ignore-eos
    switches it off."""
    from aiohttp.test_utils import TestClient, TestServer
    from tokenizers import Tokenizer as HFTokenizer
    from tokenizers.models import WordLevel

    from skein_b200.compile.artifact import WeightSource
    from skein_b200.models.config import ModelConfig
    from skein_b200.parallel import worker

    art = make_artifact(tmp_path / "plain")
    free = make_engine(art).generate([[5, 6, 7]], 5)[0]
    cfg_eos = json.dumps({**json.loads(TINY), "eos_token_id": [free[2], 299]})          # several end tokens: the first counts
    assert ModelConfig.from_hf_dict(json.loads(cfg_eos)).eos_token_id == free[2] and ModelConfig.from_hf_dict(json.loads(TINY)).eos_token_id == -1
    tok_file = tmp_path / "tokenizer.json"
    HFTokenizer(WordLevel({f"t{i}": i for i in range(300)}, unk_token="t0")).save(str(tok_file))
    plan = core.extract_plan(cfg_eos, *INPUTS, {"force_batch": 4}, [["bf16", "bf16", "bf16"]])["plan_json"]
    c = ModelConfig.from_hf_dict(json.loads(cfg_eos))
    with_tok = Artifact(build_artifact(plan, cfg_eos, tmp_path / "tok", WeightSource(c, seed=0, std=0.05), tokenizer_json=tok_file))
    no_tok = Artifact(build_artifact(plan, cfg_eos, tmp_path / "notok", WeightSource(c, seed=0, std=0.05)))
    dev = torch.device("cpu")
    args = lambda a, *extra: worker.parse(["--artifact", str(a.path), "--cpu", "--max-seq-len", "256", *extra])  # noqa: E731
    eng = worker.build_engine(with_tok, 0, dev, None, args(with_tok))
    assert eng.cfg.eos_token == free[2]
    assert worker.build_engine(no_tok, 0, dev, None, args(no_tok)).cfg.eos_token == -1
    assert worker.build_engine(with_tok, 0, dev, None, args(with_tok, "--ignore-eos")).cfg.eos_token == -1
    assert eng.generate([[5, 6, 7]], 5)[0] == free[:3]                                  # ends with the end token, which is delivered
    driver = EngineDriver(eng).start()

    async def scenario():
        async with TestClient(TestServer(build_app(driver, Tokenizer(300)))) as cl:
            body = await (await cl.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 5})).json()
            assert body["tokens"] == free[:3] and body["finish_reason"] == "stop"
            body = await (await cl.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 2})).json()
            assert body["tokens"] == free[:2] and body["finish_reason"] == "length"
            r = await cl.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 5, "stream": True})
            events = [json.loads(l[6:]) for l in (await r.text()).splitlines() if l.startswith("data: ")]
            assert [e["token"] for e in events] == free[:3] and events[-1]["finish_reason"] == "stop" and "finish_reason" not in events[0]

    try:
        asyncio.run(asyncio.wait_for(scenario(), 120))
    finally:
        driver.stop()


def test_hot_swap_reject_drain_and_timeout(tmp_path):
    a = make_artifact(tmp_path / "a", seed=0)
    b = make_artifact(tmp_path / "b", seed=1, batch=8)           # same shapes, other weights and batch policy
    wide = json.loads(TINY); wide["intermediate_size"] = 1024
    c = make_artifact(tmp_path / "c", cfg=json.dumps(wide))
    eng = make_engine(a)
    driver = EngineDriver(eng).start()
    try:
        hs = HotSwap(driver, a, drain_timeout_s=30.0)
        with pytest.raises(HotSwapError, match="rejected"):
            hs.swap(c.path)
        # drain under load: requests in flight finish, then the weights change
        subs = [driver.submit([3, 4, 5], 6) for _ in range(3)]
        t = threading.Thread(target=lambda: hs.swap(b.path, tmp_path))
        t.start()
        done = []
        for rid, kind, reason, q in subs:
            while True:
                ev = q.get(timeout=60)
                if ev.is_final:
                    done.append(ev.error)
                    break
        t.join(60)
        assert done == [None, None, None] and hs.mounted.path == b.path and not driver.draining
        assert (tmp_path / "LATEST").is_symlink()
        w_new = b.load_weights(0, "cpu")
        assert torch.equal(eng.dec.w.layers[0].wqkv, w_new.layers[0].wqkv)
        # drain timeout: a long request keeps the old artifact mounted and admission resumes
        hs2 = HotSwap(driver, b, drain_timeout_s=0.01)
        rid, kind, reason, q = driver.submit([1, 2, 3], 200)
        with pytest.raises(HotSwapError, match="timed out"):
            hs2.swap(a.path)
        assert hs2.mounted.path == b.path and not driver.draining
        assert driver.submit([9], 1)[1] in ("admit", "delay")
    finally:
        driver.stop()


def test_hot_swap_over_http_forgets_cached_prefixes_and_swaps_fp8_weights(tmp_path):
    """POST /admin/hotswap (serve --enable-hot-swap): after the swap the same prompt is answered by the new weights
    from scratch, although its prefix was cached under the old ones; block-scaled fp8 tensors are swapped too."""
    from aiohttp.test_utils import TestClient, TestServer

    a = make_artifact(tmp_path / "a", seed=0)
    b = make_artifact(tmp_path / "b", seed=1)
    eng = make_engine(a, prefix_cache=True)
    driver = EngineDriver(eng).start()
    prompt = list(range(3, 43))                                    # 40 tokens: two full pages are cacheable
    fresh_b = make_engine(b, prefix_cache=False).generate([prompt], 5)[0]

    async def scenario():
        async with TestClient(TestServer(build_app(driver, Tokenizer(300), HotSwap(driver, a), tmp_path))) as c:
            r1 = await (await c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 5})).json()
            r1b = await (await c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 5})).json()
            assert r1["tokens"] == r1b["tokens"] and eng.kv.prefix_hit_tokens_total == 32
            bad = await c.post("/admin/hotswap", json={"artifact": str(tmp_path / "nope")})
            assert bad.status == 409
            ok = await c.post("/admin/hotswap", json={"artifact": str(b.path)})
            assert ok.status == 200 and (await ok.json())["mounted"] == str(b.path)
            assert eng.kv.try_prefix_reuse(prompt) == 0            # KV computed with the old weights is unreachable
            r2 = await (await c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 5})).json()
            assert r2["tokens"] == fresh_b and r2["tokens"] != r1["tokens"]
            # sampling parameters travel through the API; a seed fixes the stream
            s1 = await (await c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 5, "temperature": 1.3, "top_k": 40, "seed": 5})).json()
            s2 = await (await c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 5, "temperature": 1.3, "top_k": 40, "seed": 5})).json()
            assert s1["tokens"] == s2["tokens"] and s1["tokens"] != r2["tokens"]
            assert (await c.post("/v1/completions", json={"prompt": prompt, "temperature": 1.0, "top_p": 1.5})).status == 400

    try:
        asyncio.run(asyncio.wait_for(scenario(), 120))
    finally:
        driver.stop()
    assert (tmp_path / "LATEST").is_symlink()
    # fp8 blocks are copied in place as well
    from skein_b200.models.decoder import quantize_blocks
    from skein_b200.runtime.hotswap import _copy_into
    wa, wb = a.load_weights(0, "cpu"), b.load_weights(0, "cpu")
    quantize_blocks(wa, [0], names=("w13",)); quantize_blocks(wb, [0], names=("w13",))
    q_before = wa.layers[0].fp8["w13"].q.clone()
    wa.layers[0].fp8["w13"].copy_(wb.layers[0].fp8["w13"])
    assert not torch.equal(q_before.view(torch.uint8), wa.layers[0].fp8["w13"].q.view(torch.uint8))
    assert torch.equal(wa.layers[0].fp8["w13"].q.view(torch.uint8), wb.layers[0].fp8["w13"].q.view(torch.uint8))
    with pytest.raises(HotSwapError):
        _copy_into(None, wb.layers[0].wqkv)
