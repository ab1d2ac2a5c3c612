"""Hot swap: replace the mounted artifact without dropping requests.

    1. verify_shape_compatibility   io.json of every device must be equal (names, shard shapes, dtypes)
    2. drain                        stop admitting, wait (bounded) for in-flight requests to finish; on
                                    timeout the old artifact stays mounted and admission resumes
    3. load + atomic symlink swap   new weights are copied into the live tensors, LATEST is renamed over

Counterpart of crates/skein_runtime/src/hotswap/{mod.rs:20-42, mount.rs:13, symlink.rs:10-48, drain.rs}.
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..compile.artifact import Artifact, ArtifactError, update_latest_symlink, verify_shape_compatibility


class HotSwapError(RuntimeError):
    pass


class HotSwap:
    def __init__(self, driver, mounted: Artifact, rank: int = 0, drain_timeout_s: float = 60.0):
        self.driver, self.mounted, self.rank, self.drain_timeout_s = driver, mounted, rank, drain_timeout_s

    def swap(self, new_path, out_root=None) -> Artifact:
        new = Artifact(new_path)
        try:
            verify_shape_compatibility(self.mounted, new)
        except ArtifactError as e:
            raise HotSwapError(f"rejected: {e}") from e
        if not self.driver.drain(self.drain_timeout_s):
            raise HotSwapError(f"drain timed out after {self.drain_timeout_s:g} s; the old artifact stays mounted")
        try:
            self._mount(new)
            if out_root is not None:
                update_latest_symlink(out_root, new.path)
            self.mounted = new
        finally:
            self.driver.draining = False
        return new

    def _mount(self, new: Artifact) -> None:
        dec = self.driver.engine.dec
        fresh = new.load_weights(self.rank, dec.device)
        with torch.no_grad():
            for old_l, new_l in zip(dec.w.layers, fresh.layers):
                for name in ("attn_norm", "wqkv", "wo", "ffn_norm", "router", "w13", "w2"):
                    o, n = getattr(old_l, name), getattr(new_l, name)
                    if o is not None:
                        o.copy_(n)      # in place: captured CUDA graphs keep pointing at the same storage
            for name in ("embed", "final_norm", "lm_head"):
                o, n = getattr(dec.w, name), getattr(fresh, name)
                if o is not None:
                    o.copy_(n)
