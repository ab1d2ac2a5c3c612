"""Hot swap: replace the mounted artifact without dropping requests.

    1. verify_shape_compatibility   io.json of every device must be equal (names, shard shapes, dtypes)
    2. drain                        the engine driver stops admitting and keeps stepping until the in-flight
                                    requests have finished; on time-out the old artifact stays mounted and
                                    admission resumes
    3. mount                        between two steps, on every rank in the same iteration (the driver announces
                                    it through the control plane): the new weights are copied into the live
                                    tensors (bf16, tile-packed and block-scaled fp8 alike, so captured CUDA graphs
                                    keep pointing at valid storage) and the prefix cache is emptied, because KV
                                    pages computed with the old weights must not be matched any more
    4. atomic symlink swap          LATEST is renamed over

The server exposes it as POST /admin/hotswap (serve --enable-hot-swap).

Counterpart of crates/skein_runtime/src/hotswap/{mod.rs:20-42, mount.rs:13, symlink.rs:10-48, drain.rs} and
of the server life cycle that calls it (crates/skein_runtime/src/server/lifecycle.rs:22-124).
"""
from __future__ import annotations

import torch

from ..compile.artifact import Artifact, ArtifactError, update_latest_symlink, verify_shape_compatibility


class HotSwapError(RuntimeError):
    pass


def _copy_into(old, new) -> None:
    """In-place update of one weight slot, whatever its storage form."""
    if old is None or new is None:
        if (old is None) != (new is None):
            raise HotSwapError("the artifacts store a weight in different forms (one has it, the other does not)")
        return
    old.copy_(new)


def mount_weights(engine, artifact_path, rank: int) -> None:
    """Copy rank `rank`'s shard of the artifact into the engine's live weights and forget cached prefixes."""
    new = Artifact(artifact_path)
    dec = engine.dec
    inner = getattr(dec, "dec", dec)          # a pipeline stage wraps its decoder
    fresh = new.load_weights(rank, inner.device)
    with torch.no_grad():
        for old_l, new_l in zip(inner.w.layers, fresh.layers):
            for name in ("attn_norm", "wqkv", "wo", "ffn_norm", "router", "w13", "w2", "bqkv"):
                _copy_into(getattr(old_l, name), getattr(new_l, name))
            if set(old_l.fp8) != set(new_l.fp8):
                raise HotSwapError("the artifacts quantise different projections of a block")
            for name, w8 in old_l.fp8.items():
                w8.copy_(new_l.fp8[name])
        for name in ("embed", "final_norm", "lm_head"):
            _copy_into(getattr(inner.w, name), getattr(fresh, name))
    engine.kv.clear_prefix_cache()
    if inner.device.type == "cuda":
        torch.cuda.synchronize(inner.device)


class HotSwap:
    def __init__(self, driver, mounted: Artifact, rank: int = 0, drain_timeout_s: float = 60.0):
        self.driver, self.mounted, self.rank, self.drain_timeout_s = driver, mounted, rank, drain_timeout_s

    def swap(self, new_path, out_root=None) -> Artifact:
        try:
            new = Artifact(new_path)
            verify_shape_compatibility(self.mounted, new)
        except ArtifactError as e:
            raise HotSwapError(f"rejected: {e}") from e
        ok, msg = self.driver.swap(new.path, self.drain_timeout_s)
        if not ok:
            if "timed out" in msg:
                raise HotSwapError(f"drain timed out after {self.drain_timeout_s:g} s; the old artifact stays mounted")
            raise HotSwapError(msg)
        if out_root is not None:
            update_latest_symlink(out_root, new.path)
        self.mounted = new
        return new
