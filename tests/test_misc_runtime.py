"""Speculative decoding loop, heartbeat watchdog, profiling switches (CPU)."""
import time

import pytest

from skein_b200.parallel.watchdog import Heartbeat, Monitor
from skein_b200.runtime import speculative as sp


def test_speculative_equals_target_greedy_when_draft_is_the_target():
    V = 7

    def dist_for(seq):                      # deterministic "model": next token = (last + 2) mod V
        p = [0.0] * V
        p[(seq[-1] + 2) % V] = 1.0
        return p
    target = lambda seq, draft: [dist_for(seq + draft[:i]) for i in range(len(draft) + 1)]
    out, st = sp.generate([1], 9, 3, dist_for, target, seed=0)
    assert out == [(1 + 2 * (i + 1)) % V for i in range(9)]
    assert st["accepted"] == st["proposed"] and st["target_calls"] <= 3      # every draft token accepted: 4 tokens per call


def test_speculative_with_a_bad_draft_still_follows_the_target():
    V = 5
    target_next = lambda seq: (seq[-1] + 1) % V

    def target(seq, draft):
        ps = []
        for i in range(len(draft) + 1):
            p = [0.0] * V
            p[target_next(seq + draft[:i])] = 1.0
            ps.append(p)
        return ps
    draft = lambda seq: [1.0 / V] * V        # uniform draft: mostly rejected
    out, st = sp.generate([0], 8, 4, draft, target, seed=1)
    assert out == [(i + 1) % V for i in range(8)]
    assert st["accepted"] < st["proposed"]


def test_watchdog_flags_a_rank_that_stops_beating(tmp_path):
    a = Heartbeat(str(tmp_path), 0, 0.02).start()
    b = Heartbeat(str(tmp_path), 1, 0.02).start()
    mon = Monitor(str(tmp_path), 2, interval_s=0.02, missed_beats=5)
    time.sleep(0.1)
    assert mon.dead_ranks() == []
    b.stop()                                 # rank 1 "dies" on the host
    deadline = time.time() + 3
    while time.time() < deadline and mon.dead_ranks() != [1]:
        time.sleep(0.05)
    assert mon.dead_ranks() == [1]
    a.stop()
    assert Monitor(str(tmp_path), 3, 0.01, 1).dead_ranks(now=0.0) == [] and Monitor(str(tmp_path / "none"), 1, 0.01, 1).dead_ranks(0.0) == []


def test_profiling_is_a_no_op_by_default():
    from skein_b200.utils import profiling
    with profiling.region("x"):
        pass
    assert profiling.report() == {} or "x" in profiling.report()
    profiling.count_h2d(10); profiling.count_d2h(4)
    assert profiling.host_bytes()["h2d"] >= 10


def test_packed_weight_round_trip_and_in_place_update():
    """Tile-packed weights keep the logical tensor: unpack / cpu give it back, copy_ re-packs in place (hot swap)."""
    import torch

    from skein_b200 import ops

    g = torch.Generator().manual_seed(0)
    for shape in ((256, 128), (3, 384, 192)):
        w = torch.randn(*shape, generator=g).bfloat16()
        p = ops.pack_weight(w)
        assert p.shape == tuple(shape) and torch.equal(p.unpack(), w) and torch.equal(p.cpu(), w)
        storage = p.data.data_ptr()
        w2 = torch.randn(*shape, generator=g).bfloat16()
        p.copy_(w2)
        assert p.data.data_ptr() == storage and torch.equal(p.unpack(), w2)
        p.copy_(ops.pack_weight(w))
        assert torch.equal(p.unpack(), w)
        # the CPU operators accept the packed form
        x = torch.randn(5, shape[-1], generator=g).bfloat16()
        if len(shape) == 2:
            assert torch.equal(ops.linear(x, p), ops.linear(x, w))
    import pytest
    with pytest.raises(ValueError):
        ops.pack_weight(torch.zeros(100, 64))


def test_heartbeat_stops_while_a_step_is_stuck(tmp_path):
    """The beat follows the step loop: a rank that has been inside one step for longer than the limit looks dead to
    the monitor although its process (and the beating thread) is alive; an idle rank keeps beating."""
    started = {"t": None}
    hb = Heartbeat(str(tmp_path), 0, 0.02, step_started_at=lambda: started["t"], stall_limit_s=0.1).start()
    mon = Monitor(str(tmp_path), 1, interval_s=0.02, missed_beats=5)
    try:
        time.sleep(0.3)
        assert mon.dead_ranks() == []                   # idle: beats
        time.sleep(0.15)
        assert mon.dead_ranks() == []
        started["t"] = time.monotonic()                 # a step begins and never ends
        time.sleep(0.5)
        mon.dead_ranks()
        time.sleep(0.2)
        assert mon.dead_ranks() == [0]
        started["t"] = None                             # the step finished after all
        time.sleep(0.2)
        assert mon.dead_ranks() == []
    finally:
        hb.stop()


def test_speculative_decoding_with_a_draft_model_equals_target_greedy():
    """A draft Decoder proposes, the target Decoder verifies k + 1 positions in one chunk over its paged KV cache: with
    temperature 0 the output is the target's greedy decode for a good and for a useless draft."""
    from skein_b200.models import config as mc
    from skein_b200.models.decoder import Decoder, random_weights
    from skein_b200.runtime.engine import Engine, EngineConfig

    cfg = mc.tiny_mixtral()
    mk = lambda c, seed: Decoder(c, random_weights(c, mc.ParallelLayout(), "cpu", seed=seed, std=0.05), num_pages=32, page_size=16, max_pos=256)
    prompt = list(range(5, 25))
    want = Engine(mk(cfg, 0), EngineConfig(max_batch=1, tpot_ms=1e6, use_graphs=False, prefix_cache=False)).generate([prompt], 12)[0]
    out, st = sp.SpeculativeDecoder(mk(cfg, 0), mk(cfg, 0), k=3).generate(prompt, 12)
    assert out == want and st["accepted"] == st["proposed"] and st["target_steps"] <= 5      # 4 tokens per target step
    small = mc.tiny_mixtral(layers=1)
    out, st = sp.SpeculativeDecoder(mk(cfg, 0), mk(small, 3), k=3).generate(prompt, 12)
    assert out == want and st["accepted"] < st["proposed"]
    # with a temperature the rule samples from the target: same seed, same tokens; the draft being the target
    # itself, every proposal is accepted
    a, sa = sp.SpeculativeDecoder(mk(cfg, 0), mk(cfg, 0), k=3).generate(prompt, 10, temperature=0.9, seed=4)
    b, _ = sp.SpeculativeDecoder(mk(cfg, 0), mk(cfg, 0), k=3).generate(prompt, 10, temperature=0.9, seed=4)
    assert a == b and len(a) == 10 and sa["accepted"] == sa["proposed"]


def test_spans_are_exported_as_otlp_http_json(monkeypatch):
    """With SKEIN_OTLP_ENDPOINT set the engine ships one span per step and one per finished request to <endpoint>/v1/traces
    (OTLP/HTTP JSON); a collector that is down costs nothing but dropped spans."""
    import http.server
    import json
    import threading

    from skein_b200.models import config as mc
    from skein_b200.models.decoder import Decoder, random_weights
    from skein_b200.runtime.engine import Engine, EngineConfig
    from skein_b200.utils import otlp

    got = []

    class Collector(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            body = self.rfile.read(int(self.headers["Content-Length"]))
            got.append((self.path, self.headers["Content-Type"], json.loads(body)))
            self.send_response(200)
            self.end_headers()
            self.wfile.write(b"{}")

        def log_message(self, *a):
            pass

    srv = http.server.HTTPServer(("127.0.0.1", 0), Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        otlp.shutdown()
        monkeypatch.setenv("SKEIN_OTLP_ENDPOINT", f"http://127.0.0.1:{srv.server_address[1]}")
        monkeypatch.setenv("SKEIN_OTLP_SERVICE", "skein-test")
        cfg = mc.tiny_mixtral(layers=1, hidden=128, inter=128, heads=2, kv_heads=1, experts=4, vocab=64)
        dec = Decoder(cfg, random_weights(cfg, mc.ParallelLayout(), "cpu", seed=0), num_pages=16, page_size=16, max_pos=64)
        eng = Engine(dec, EngineConfig(max_batch=4, use_graphs=False, prefix_cache=False))
        assert eng._otlp is not None
        out = eng.generate([[1, 2, 3], [4, 5]], 4)
        assert [len(o) for o in out] == [4, 4]
        otlp.shutdown()                       # flushes
    finally:
        srv.shutdown()
    assert got and all(p == "/v1/traces" and ct == "application/json" for p, ct, _ in got)
    spans = [s for _, _, b in got for rs in b["resourceSpans"] for ss in rs["scopeSpans"] for s in ss["spans"]]
    res = got[0][2]["resourceSpans"][0]["resource"]["attributes"]
    assert {"key": "service.name", "value": {"stringValue": "skein-test"}} in res
    names = [s["name"] for s in spans]
    assert names.count("request") == 2 and names.count("engine.step") >= 4
    req = next(s for s in spans if s["name"] == "request")
    attrs = {a["key"]: a["value"] for a in req["attributes"]}
    assert attrs["output_tokens"] == {"intValue": "4"} and "ttft_ms" in attrs and len(req["traceId"]) == 32 and len(req["spanId"]) == 16
    assert int(req["endTimeUnixNano"]) >= int(req["startTimeUnixNano"])
    # no endpoint: no exporter, no thread
    monkeypatch.delenv("SKEIN_OTLP_ENDPOINT")
    assert otlp.exporter() is None
    # a dead collector: posts fail quietly, a full queue drops
    ex = otlp.SpanExporter("http://127.0.0.1:9", max_queue=2, flush_s=0.05, timeout_s=0.2)
    for i in range(50):
        ex.span("x", 1, 2)
    ex.close()
    assert ex.sent == 0 and (ex.dropped > 0 or ex.failed_posts > 0)
