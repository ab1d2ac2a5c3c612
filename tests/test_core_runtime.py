"""C++ runtime pieces on CPU: paged-KV block manager + radix prefix cache, continuous batcher, parity math,
drift monitor, speculative acceptance, CPU collectives, metrics.

Mirrors crates/skein_runtime/tests/{kv_allocator,radix_reuse,batcher_admission,runtime_traits,
observability_metrics}.rs and the unit tests in drift_monitor.rs, speculative.rs, comparison.rs.
"""
import math

import pytest

from skein_b200 import core


# ---- KV manager ---------------------------------------------------------------------------------------------------
def test_admit_advance_release_accounting():
    kv = core.KvBlockManager(8, 16, False)
    pt = kv.admit(1, list(range(40)))                  # 3 pages
    assert len(pt.pages) == 3 and kv.in_use_pages == 3 and kv.available_pages == 5
    assert kv.advance(1, 8) == []                      # 48 tokens still fit 3 pages
    added = kv.advance(1, 1)                           # token 49 needs a 4th
    assert len(added) == 1 and kv.pages_for(1)[-1] == added[0]
    kv.admit(2, list(range(16 * 4)))
    assert kv.in_use_pages == 8 and abs(kv.utilization - 1.0) < 1e-12
    with pytest.raises(Exception, match="exhausted"):
        kv.admit(3, [1, 2, 3])
    kv.release(1)
    assert kv.in_use_pages == 4 and kv.pages_for(1) is None
    with pytest.raises(Exception, match="unknown request"):
        kv.release(1)
    with pytest.raises(Exception, match="already admitted"):
        kv.admit(2, [1])
    big = core.KvBlockManager.with_capacity(268435456, 524288, 16)
    assert big.total_pages == 32


def test_prefix_reuse_refcounts_and_lru_eviction():
    kv = core.KvBlockManager(6, 4, True)
    a = list(range(10))                                # 2 full pages + 2 tokens
    pa = kv.admit(1, a)
    assert pa.prefix_hit_tokens == 0 and pa.registered_pages == 0
    # pages that are reserved but not computed yet are invisible to other requests
    assert kv.try_prefix_reuse(a) == 0
    assert kv.mark_computed(1, a, 5) == 1 and kv.try_prefix_reuse(a) == 4
    assert kv.mark_computed(1, a, 10) == 2
    pb = kv.admit(2, a[:8] + [99, 98, 97])             # shares the two full pages
    assert pb.prefix_hit_tokens == 8 and pb.pages[:2] == pa.pages[:2] and pb.pages[2] != pa.pages[2]
    assert kv.in_use_pages == 4 and kv.prefix_hit_tokens_total == 8
    # an identical prompt may reuse at most len-1 tokens' worth of full pages
    assert kv.try_prefix_reuse(a[:8]) == 4
    kv.release(1)
    assert kv.in_use_pages == 3                        # shared pages stay referenced by request 2
    kv.release(2)
    assert kv.in_use_pages == 0 and kv.available_pages == 6
    # cached pages survive release and are found again
    assert kv.try_prefix_reuse(a) == 8
    gen_before = kv.generation_of(pa.pages[0])
    # filling the cache evicts the LRU cached pages and bumps their generation: the trie entry goes stale
    kv.admit(3, list(range(100, 124)))                 # 6 pages: needs every page
    assert kv.generation_of(pa.pages[0]) == gen_before + 1
    kv.release(3)
    assert kv.try_prefix_reuse(a) == 0


def test_radix_hit_rate_on_shared_system_prompt():
    kv = core.KvBlockManager(64, 16, True)
    system = list(range(1000, 1064))                   # 4 pages
    hits = 0
    for i in range(8):
        pt = kv.admit(i, system + [i, i + 1, i + 2])
        hits += pt.prefix_hit_tokens
        kv.mark_computed(i, system + [i, i + 1, i + 2], 67)
        kv.release(i)
    assert hits == 7 * 64


def test_failed_request_and_cleared_cache_leave_no_stale_prefix():
    kv = core.KvBlockManager(8, 4, True)
    a = list(range(12))
    kv.admit(1, a)
    kv.mark_computed(1, a, 8)                          # two pages computed, then the step fails
    kv.release(1, True)
    assert kv.try_prefix_reuse(a) == 0 and kv.available_pages == 8
    # a page shared with a live request survives the failure of the other one
    kv.admit(2, a); kv.mark_computed(2, a, 12)
    pb = kv.admit(3, a + [50])
    assert pb.prefix_hit_tokens == 12
    kv.release(3, True)
    assert kv.try_prefix_reuse(a + [50]) == 12
    kv.release(2)
    # new weights: everything cached is forgotten, the pages are free again
    kv.clear_prefix_cache()
    assert kv.try_prefix_reuse(a + [50]) == 0 and kv.available_pages == 8
    kv.admit(4, a); kv.mark_computed(4, a, 12)
    assert kv.try_prefix_reuse(a + [50]) == 12


# ---- batcher --------------------------------------------------------------------------------------------------------
def test_slo_admission_decisions():
    b = core.ContinuousBatcher(max_batch=2, ttft_ms=500, tpot_ms=50, decode_us_at_b1=8000, batch_exponent=0.7, prefill_per_token_us=25)
    assert b.decide(1, [0] * 100, 8, 0).kind == "admit"
    d = b.decide(2, [0] * 30000, 8, 0)                 # 750 ms predicted prefill > 500 ms TTFT SLO
    assert d.kind == "reject" and d.reason == "prompt_too_long"
    assert b.submit(1, [0] * 10, 4, 0).kind == "admit" and b.submit(2, [0] * 10, 4, 0).kind == "admit"
    d = b.submit(3, [0] * 10, 4, 100)
    assert d.kind == "delay" and d.reason == "batch_full" and d.until_ms > 100 and b.queued_len == 1
    # TPOT SLO: 8 ms * n^0.7 > 50 ms for n >= 14
    big = core.ContinuousBatcher(max_batch=64, tpot_ms=50)
    for i in range(13):
        assert big.submit(i, [0] * 8, 4, 0).kind == "admit"
    assert big.submit(99, [0] * 8, 4, 0).reason == "tpot_slo"
    assert b.submit(4, [0] * 30000, 4, 0).kind == "reject" and b.rejected == 1


def test_batch_life_cycle_with_kv_and_chunked_prefill():
    kv = core.KvBlockManager(32, 16, True)
    b = core.ContinuousBatcher(max_batch=4, chunk_tokens=32, kv=kv, tpot_ms=1000, max_prefill_tokens=48)
    assert b.submit(1, list(range(70)), 3, 0).kind == "admit"
    assert b.submit(2, list(range(500, 520)), 2, 0).kind == "admit"
    assert kv.in_use_pages == 5 + 2
    pre, dec = b.next_step_batch()
    assert pre == [(1, 0, 32, False), (2, 0, 16, False)] and dec == []      # 48-token budget shared in order
    # a request with the same prompt arriving now shares only what request 1 has computed so far
    assert kv.try_prefix_reuse(list(range(70))) == 0
    b.prefill_advanced(1, 32); b.prefill_advanced(2, 16)
    assert kv.try_prefix_reuse(list(range(70))) == 32
    pre, dec = b.next_step_batch()
    assert pre == [(1, 32, 64, False), (2, 16, 20, True)]
    b.prefill_advanced(1, 64); b.prefill_advanced(2, 20)
    assert b.accept_token(2, 7, 10) == (False, 1)                            # first token: request 2 now decodes
    assert b.request_info(2)["phase"] == "decode" and b.request_info(2)["first_token_ms"] == 10
    pre, dec = b.next_step_batch()
    assert pre == [(1, 64, 70, True)] and dec == [2]
    b.prefill_advanced(1, 70)
    assert b.accept_token(1, 5, 20) == (False, 1)
    assert b.accept_token(2, 8, 20) == (True, 2)                             # max_new_tokens reached
    assert b.current_sequence(2) == list(range(500, 520)) + [7, 8]
    b.retire(2)
    assert kv.pages_for(2) is None and b.inflight_len == 1 and b.retired == 1
    pre, dec = b.next_step_batch()
    assert pre == [] and dec == [1]
    assert b.accept_token(1, 6, 30, eos_token=6) == (True, 2)                # EOS ends the request early
    b.retire(1)
    assert kv.in_use_pages == 0
    assert b.accept_token(1, 0, 40) is None


def test_kv_pressure_delays_then_promotes():
    kv = core.KvBlockManager(4, 16, False)
    b = core.ContinuousBatcher(max_batch=8, kv=kv, tpot_ms=1000)
    assert b.submit(1, [0] * 40, 8, 0).kind == "admit"                       # 3 pages
    d = b.submit(2, [0] * 30, 8, 0)
    assert d.kind == "delay" and d.reason == "kv_full"
    b.promote_ready(d.until_ms)
    assert b.queued_len == 1                                                  # still no room
    b.retire(1)
    b.promote_ready(10**6)
    assert b.queued_len == 0 and b.inflight_ids() == [2]
    assert sorted(b.retire_all()) == [2] and kv.in_use_pages == 0           # failure path retires everything


# ---- parity math ------------------------------------------------------------------------------------------------------
def test_mse_and_kl():
    assert core.mse([1.0, 2.0, 3.0], [1.0, 2.0, 5.0]) == pytest.approx(4.0 / 3.0)
    assert core.kl_divergence([1.0, 2.0, 3.0], [1.0, 2.0, 3.0]) == pytest.approx(0.0, abs=1e-12)
    assert core.kl_divergence([0.0, 0.0], [0.0, math.log(3.0)]) == pytest.approx(0.5 * math.log(0.5 / 0.25) + 0.5 * math.log(0.5 / 0.75))
    # stable at extreme logits
    k = core.kl_divergence([1e4, -1e4, 0.0], [1e4, -1e4, 1.0])
    assert math.isfinite(k) and k >= 0
    assert sum(math.exp(v) for v in core.log_softmax([1e4, 1e4 - 1.0])) == pytest.approx(1.0)
    with pytest.raises(Exception, match="mismatch"):
        core.mse([1.0], [1.0, 2.0])


def test_drift_monitor():
    m = core.DriftMonitor([100] * 64, 0.05)
    kl, drifted, n = m.assess([100] * 64)
    assert kl == pytest.approx(0.0, abs=1e-12) and not drifted and n == 64
    kl, drifted, _ = m.assess([3000] * 64)
    assert kl > 0.05 and drifted
    assert m.assess([3000] * 10)[1] is False                                  # below MIN_SAMPLES never flags


def test_speculative_accept_reject_and_bonus():
    p = [[0.1, 0.9], [0.5, 0.5], [0.2, 0.8]]                                  # target, k + 1 rows
    q = [[0.5, 0.5], [0.5, 0.5]]
    # token 1 at step 0: ratio min(1, .9/.5) = 1 -> accept; token 0 at step 1: ratio 1 -> accept; bonus from p[2]
    acc, corr = core.speculative_verify([1, 0], q, p, [0.99, 0.99, 0.1])
    assert acc == [1, 0] and corr == 0
    # token 0 at step 0: ratio .1/.5 = .2 < u -> reject; residual = max(0, p - q) = [0, .4] -> token 1
    acc, corr = core.speculative_verify([0, 0], q, p, [0.5, 0.0, 0.3])
    assert acc == [] and corr == 1
    with pytest.raises(Exception, match="shape"):
        core.speculative_verify([0], q, p, [0.1, 0.1])
    with pytest.raises(Exception, match="out of range"):
        core.speculative_verify([5, 0], q, p, [0.1, 0.1, 0.1])


def test_cpu_collectives():
    bufs = [[1.0, 2.0, 3.0, 4.0], [10.0, 20.0, 30.0, 40.0]]
    assert core.cpu_collective("ring_allreduce", bufs) == [[11.0, 22.0, 33.0, 44.0]] * 2
    assert core.cpu_collective("allgather", [[1.0], [2.0]]) == [[1.0, 2.0]] * 2
    assert core.cpu_collective("reducescatter", bufs) == [[11.0, 22.0], [33.0, 44.0]]
    assert core.cpu_collective("alltoall", bufs) == [[1.0, 2.0, 10.0, 20.0], [3.0, 4.0, 30.0, 40.0]]
    assert core.cpu_collective("broadcast", bufs, 1) == [bufs[1], bufs[1]]
    # repeated all-to-all is its own inverse for 2 ranks
    assert core.cpu_collective("alltoall", core.cpu_collective("alltoall", bufs)) == bufs
    with pytest.raises(Exception, match="unsupported"):
        core.cpu_collective("gossip", bufs)


def test_metrics_text():
    m = core.MetricsRegistry(4)
    for s in range(6):
        m.record_step(s, 8, 1000.0, 50.0, 12)
    m.record_request(1, "ok", 120.0, 9.0, 64, 20)
    m.record_request(2, "rejected", 0.0, 0.0, 0, 0)
    m.count("skein_graph_replays_total", 5)
    text = m.render()
    for name in ("skein_steps_total 6", "skein_step_compute_us_total 6000", "skein_step_comm_us_total 300", "skein_kv_pages_in_use 12",
                 'skein_batch_size_histogram_bucket{le="8"} 6', 'skein_requests_total{status="ok"} 1', 'skein_requests_total{status="rejected"} 1',
                 'skein_ttft_ms_histogram_bucket{le="250"} 1', 'skein_tpot_ms_histogram_bucket{le="10"} 1',
                 "skein_prefix_cache_hit_tokens_total 64", "skein_graph_replays_total 5"):
        assert name in text, name
    assert m.steps_buffered == 4 and m.requests_buffered == 2                 # ring buffer capacity
    assert m.ttft_p50() == 120.0
