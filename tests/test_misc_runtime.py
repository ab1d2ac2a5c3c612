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
