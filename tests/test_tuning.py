"""Kernel-configuration cache: keys, persistence, invalidation by kernel build; device tuning on a GPU.

The reference tests its search cache the same way: a key that changes with every input that can invalidate the result,
round trip through the file, miss on a different device (crates/skein_compile/src/search_cache.rs:36-55, tests 152-260).
"""
import json

import pytest
import torch

from skein_b200.ops import tuning


def test_keys_cover_everything_that_invalidates_a_result():
    k = tuning.make_key("gemm", (0, 1, 6144, 4096, 64), "bf16", "sm_100", "abc")
    assert k == "gemm|0x1x6144x4096x64|bf16|sm_100|abc"
    others = [tuning.make_key("gemm", (0, 1, 6144, 4096, 80), "bf16", "sm_100", "abc"),
              tuning.make_key("gemm", (0, 1, 6144, 4096, 64), "fp8", "sm_100", "abc"),
              tuning.make_key("gemm", (0, 1, 6144, 4096, 64), "bf16", "sm_90", "abc"),
              tuning.make_key("gemm", (0, 1, 6144, 4096, 64), "bf16", "sm_100", "abd"),
              tuning.make_key("attn", (0, 1, 6144, 4096, 64), "bf16", "sm_100", "abc")]
    assert len({k, *others}) == 6
    assert tuning.gemm_shape_key(2, 8, 4096, 1792, 120) == (2, 8, 4096, 1792, 128)   # rows round up to 16


def test_round_trip_and_stale_pruning(tmp_path):
    path = tmp_path / "cache" / "kernel_configs.json"
    c = tuning.KernelConfigCache(path)
    c.put("gemm", (0, 1, 768, 4096, 64), {"n_tile": 64, "grid": 0, "line_cut_only": 0}, arch="sm_100", build="b1")
    c.put("gemm", (0, 1, 768, 4096, 64), {"n_tile": 32, "grid": 0, "line_cut_only": 1}, arch="sm_100", build="b0")
    c.save()
    doc = json.loads(path.read_text())
    assert doc["version"] == 1 and len(doc["entries"]) == 2
    d = tuning.KernelConfigCache(path)
    assert d.get("gemm", (0, 1, 768, 4096, 64), arch="sm_100", build="b1")["n_tile"] == 64
    assert d.get("gemm", (0, 1, 768, 4096, 64), arch="sm_100", build="other") is None
    assert (d.hits, d.misses) == (1, 1)
    assert d.prune_stale(build="b1") == 1 and len(d.entries) == 1
    path.write_text(json.dumps({"version": 7, "entries": {}}))
    with pytest.raises(ValueError):
        tuning.KernelConfigCache(path)
    # a corrupt file: strict loading raises, the serving path falls back to an empty cache and says why
    path.write_text("{ not json")
    with pytest.raises(ValueError):
        tuning.KernelConfigCache(path)
    lenient = tuning.KernelConfigCache(path, strict=False)
    assert lenient.entries == {} and "JSONDecodeError" in lenient.load_error
    lenient.put("gemm", (0, 1, 128, 64, 16), {"n_tile": 16, "grid": 0, "line_cut_only": 0}, arch="sm_100", build="b1")
    lenient.save()
    assert tuning.KernelConfigCache(path).get("gemm", (0, 1, 128, 64, 16), arch="sm_100", build="b1")["n_tile"] == 16


def test_candidates_respect_the_epilogue_limits():
    dense = tuning.gemm_candidates(0, 1, 6144, 64, 148)
    dual = tuning.gemm_candidates(1, 8, 14336, 128, 148)
    assert dense and dual
    assert all(c["n_tile"] <= 128 for c in dual) and all(c["n_tile"] % 16 == 0 for c in dense + dual)
    assert any(c["grid"] > 0 for c in dual)            # 896 tiles on 148 SMs: a whole-tile grid is among them
    assert {c["line_cut_only"] for c in dense} == {0, 1}


@pytest.mark.gpu
def test_tuned_configuration_is_used_and_exact():
    from skein_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(48, 1024, device="cuda").bfloat16()
    w = (torch.randn(640, 1024, device="cuda") / 32).bfloat16()
    want = ops.linear(x, w)
    cache = tuning.KernelConfigCache()
    best, results = ops.tune_linear(x, w, cache=cache)
    assert best is not None and len(results) >= 2
    assert cache.get("gemm", tuning.gemm_shape_key(0, 1, 640, 1024, 48))["n_tile"] == best["n_tile"]
    tuning.activate(cache)
    try:
        got = ops.linear(x, w)
        torch.cuda.synchronize()
        ops.workspace().check_status()
        assert cache.hits >= 2
    finally:
        tuning.activate(None)
    assert float((got.float() - want.float()).abs().max()) < 2e-2 * float(want.float().abs().max())


def test_heuristic_grid_whole_tiles_only_when_they_waste_little():
    # expert down projection of Mixtral (8 experts x 32 feature tiles = 256 tiles) on 148 SMs
    assert tuning.heuristic_grid(256, 28, 148) == 128      # 8 ranks, K = 1792: two whole tiles per CTA
    assert tuning.heuristic_grid(256, 56, 148) == 128
    assert tuning.heuristic_grid(256, 112, 148) == 0       # 2 ranks: the idle SM time costs more than the fix-up
    assert tuning.heuristic_grid(256, 224, 148) == 0       # 1 GPU, K = 14336
    assert tuning.heuristic_grid(250, 64, 148) == 125      # lm_head, 32000 x 4096
    assert tuning.heuristic_grid(224, 64, 148) == 0        # 31 idle K-blocks per CTA ...
    assert tuning.heuristic_grid(224, 64, 148, dual=True) == 112   # ... but the two-accumulator kernel keeps whole tiles
    assert tuning.heuristic_grid(100, 64, 148) == 0 and tuning.heuristic_grid(896, 64, 148) == 0   # outside (SMs, 2 SMs]
