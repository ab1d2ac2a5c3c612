"""Compiled artifact: a content-addressed directory that `serve` and `verify` load without re-planning.

    <out>/<blake3(plan.json)>/
        plan.json  topology.json  metadata.json  model_config.json  [tokenizer.json]
        device_<N>/segments.json   per-device segments + schedule (the lowering recipe's result)
        device_<N>/io.json         weight manifest (name, shard shape, dtype, axis/start/len)
        device_<N>/weights.safetensors   this device's shard, HuggingFace parameter names
        cache/                      kernel-configuration cache (autotune results)
        reference_bf16/             the same placement with every dtype bf16 (parity oracle)
        parity_report.json
    <out>/LATEST -> <hash>          swapped atomically (tmp symlink + rename)

Same layout and hash rule as the reference (crates/skein_compile/src/artifact.rs:285-369; LATEST update in
crates/skein_cli/src/cmd/compile.rs:256, crates/skein_runtime/src/hotswap/symlink.rs:10). The reference's
`graph_segments.bin` (bincode of a luminal re-lowering recipe) becomes `segments.json`: lowering is
deterministic (C++ core, byte-stable), so the file can be regenerated and is checked on load.

Weights: a block whose plan dtype is fp8_e4m3 is stored as e4m3 bytes plus fp32 scales per 1 x 128 block
(`<name>.scale`); nothing is clamped back to bf16.
"""
from __future__ import annotations

import datetime
import json
import os
import shutil
from pathlib import Path

import torch

from .. import core
from ..models.config import ModelConfig, ParallelLayout
from ..models.decoder import LayerWeights, ModelWeights
from ..ops import reference as ref

FP8_DTYPES = ("fp8_e4m3",)


class ArtifactError(RuntimeError):
    pass


# ---- checkpoint access ------------------------------------------------------------------------------------------
class WeightSource:
    """Parameters by HuggingFace name. Backed by a safetensors file / sharded checkpoint directory, or by a
    seeded random generator (benchmarks and tests: N(0, std), norm gains 1)."""

    def __init__(self, cfg: ModelConfig, path: str | None = None, seed: int = 0, std: float = 0.02):
        self.cfg, self.path, self.seed, self.std = cfg, path, seed, std
        self._files = {}
        self._index = None
        if path is not None:
            p = Path(path)
            if p.is_dir():
                idx = p / "model.safetensors.index.json"
                if idx.exists():
                    self._index = {k: p / v for k, v in json.loads(idx.read_text())["weight_map"].items()}
                elif (p / "model.safetensors").exists():
                    self._single = p / "model.safetensors"
                else:
                    raise ArtifactError(f"{p} holds neither model.safetensors nor model.safetensors.index.json")
            else:
                self._single = p

    def get(self, name: str, shape) -> torch.Tensor:
        if self.path is None:
            return _random_param(name, shape, self.seed, self.std)
        from safetensors import safe_open

        if self._index is not None and name not in self._index:
            raise ArtifactError(f"checkpoint has no tensor `{name}`")
        f = self._index[name] if self._index is not None else self._single
        if f not in self._files:
            self._files[f] = safe_open(str(f), framework="pt")
        if name not in self._files[f].keys():
            raise ArtifactError(f"checkpoint has no tensor `{name}`")
        t = self._files[f].get_tensor(name)
        if list(t.shape) != list(shape):
            raise ArtifactError(f"`{name}` has shape {list(t.shape)}, the model expects {list(shape)}")
        return t.to(torch.bfloat16)


def _stable_name_seed(name: str) -> int:
    # hash() of str is salted per process; use BLAKE3 so that random weights are reproducible across ranks
    return int(core.blake3_hex(name.encode())[:8], 16)


def _random_param(name, shape, seed, std):
    if name.endswith("layernorm.weight") or name == "model.norm.weight":
        return torch.ones(*shape, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(_stable_name_seed(name) ^ (seed * 1000003))
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)


# ---- build ----------------------------------------------------------------------------------------------------------
def _slice(t: torch.Tensor, entry: dict) -> torch.Tensor:
    if entry["axis"] < 0:
        return t
    return t.narrow(entry["axis"], entry["start"], entry["len"]).contiguous()


def build_artifact(plan_json: str, config_json: str, out_root: str | Path, source: WeightSource | None = None,
                   tokenizer_json: str | Path | None = None, write_weights: bool = True, hardware: str = "b200") -> Path:
    """Lower the plan, shard (and quantise) the weights, write the artifact directory. Returns its path."""
    plan = json.loads(plan_json)
    core.plan_validate(plan_json)
    if json.loads(config_json).get("tie_word_embeddings") and plan["parallelism"]["pp"] > 1:
        # the output projection reads the embedding table, which the lowering places on the first stage only
        raise ArtifactError("tied input / output embeddings are not supported with pipeline parallelism")
    h = core.plan_hash(plan_json)
    root = Path(out_root) / h
    tmp = Path(out_root) / (h + ".partial")
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    (tmp / "plan.json").write_text(core.plan_roundtrip(plan_json))
    (tmp / "topology.json").write_text(core.emit_topology(plan_json, config_json))
    (tmp / "model_config.json").write_text(config_json)
    (tmp / "metadata.json").write_text(json.dumps({
        "skein_b200_version": "0.1.0", "hardware": hardware, "arch": "sm_100a",
        "timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds")}))
    (tmp / "cache").mkdir()
    if tokenizer_json is not None and Path(tokenizer_json).exists():
        shutil.copy(tokenizer_json, tmp / "tokenizer.json")
    cfg = ModelConfig.from_hf_dict(json.loads(config_json))
    source = source or WeightSource(cfg)
    par = plan["parallelism"]
    n_dev = par["tp"] * par["pp"] * par["ep"]
    for d in range(n_dev):
        dd = tmp / f"device_{d}"
        dd.mkdir()
        (dd / "segments.json").write_text(core.lower_device(plan_json, config_json, d))
        io = core.io_manifest(plan_json, config_json, d)
        (dd / "io.json").write_text(io)
        if not write_weights:
            continue
        from safetensors.torch import save_file

        tensors = {}
        for e in json.loads(io)["tensors"]:
            full_shape = _full_shape(cfg, e["name"])
            t = source.get(e["name"], full_shape)
            t = _slice(t, e)
            if e["dtype"] in FP8_DTYPES and t.dim() == 2 and t.shape[1] % 128 == 0:
                q, s = ref.quant_fp8_block128(t, pow2_scales=True)     # weights: exact in-kernel rescaling (ops/fp8.py)
                tensors[e["name"]] = q.view(torch.uint8)
                tensors[e["name"] + ".scale"] = s
            else:
                tensors[e["name"]] = t.contiguous()
        save_file(tensors, str(dd / "weights.safetensors"))
    if root.exists():
        shutil.rmtree(root)
    os.replace(tmp, root)
    return root


def _full_shape(cfg: ModelConfig, name: str):
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    if name in ("model.embed_tokens.weight", "lm_head.weight"):
        return (cfg.vocab_size, H)
    if name.endswith("layernorm.weight") or name == "model.norm.weight":
        return (H,)
    if name.endswith("q_proj.bias"):
        return (cfg.num_heads * D,)
    if name.endswith("k_proj.bias") or name.endswith("v_proj.bias"):
        return (cfg.num_kv_heads * D,)
    if "q_proj" in name:
        return (cfg.num_heads * D, H)
    if "k_proj" in name or "v_proj" in name:
        return (cfg.num_kv_heads * D, H)
    if "o_proj" in name:
        return (H, cfg.num_heads * D)
    if "block_sparse_moe.gate" in name:
        return (cfg.num_experts, H)
    if ".w1." in name or ".w3." in name or "gate_proj" in name or "up_proj" in name:
        return (I, H)
    if ".w2." in name or "down_proj" in name:
        return (H, I)
    raise ArtifactError(f"unknown parameter `{name}`")


def update_latest_symlink(out_root: str | Path, artifact_dir: Path) -> None:
    """Atomic LATEST -> <hash>: create a temporary symlink, rename it over the old one."""
    out_root = Path(out_root)
    tmp = out_root / f".LATEST.{os.getpid()}.tmp"
    if tmp.is_symlink() or tmp.exists():
        tmp.unlink()
    os.symlink(artifact_dir.name, tmp)
    os.replace(tmp, out_root / "LATEST")


# ---- load -------------------------------------------------------------------------------------------------------------
class Artifact:
    def __init__(self, path: str | Path):
        self.path = Path(path).resolve()
        for f in ("plan.json", "topology.json", "model_config.json", "metadata.json"):
            if not (self.path / f).exists():
                raise ArtifactError(f"{self.path} is not an artifact: {f} is missing")
        self.plan_json = (self.path / "plan.json").read_text()
        self.plan = json.loads(self.plan_json)
        self.config_json = (self.path / "model_config.json").read_text()
        self.cfg = ModelConfig.from_hf_dict(json.loads(self.config_json))
        want = core.plan_hash(self.plan_json)
        if self.path.name != want and not self.path.name.startswith("reference"):
            raise ArtifactError(f"artifact directory {self.path.name} does not match its plan hash {want}")
        par = self.plan["parallelism"]
        self.layout_dims = (par["tp"], par["pp"], par["ep"])
        self.num_devices = par["tp"] * par["pp"] * par["ep"]

    def check_lowering(self, device: int) -> None:
        """The stored segments must equal what the current lowering produces for this plan."""
        stored = (self.path / f"device_{device}" / "segments.json").read_text()
        if stored != core.lower_device(self.plan_json, self.config_json, device):
            raise ArtifactError(f"device_{device}/segments.json does not match the plan (stale or corrupt artifact)")

    def io_manifest(self, device: int) -> dict:
        return json.loads((self.path / f"device_{device}" / "io.json").read_text())

    def tokenizer_path(self):
        p = self.path / "tokenizer.json"
        return p if p.exists() else None

    def layout(self, rank: int) -> ParallelLayout:
        tp, pp, ep = self.layout_dims
        return ParallelLayout(tp=tp, pp=pp, ep=ep, rank=rank)

    def load_weights(self, device_idx: int, device) -> ModelWeights:
        """Read device_<N>/weights.safetensors and assemble the fused tensors the decoder uses
        (q/k/v stacked, experts stacked with gate rows before up rows). fp8 blocks are dequantised to bf16
        here when the runtime has no fp8 kernel for them (W8A16 numerics: exactly the stored values)."""
        from safetensors import safe_open

        f = self.path / f"device_{device_idx}" / "weights.safetensors"
        if not f.exists():
            raise ArtifactError(f"{f} is missing (artifact was built without weights)")
        with safe_open(str(f), framework="pt") as sf:
            keys = set(sf.keys())

            def get(name):
                if name not in keys:
                    raise ArtifactError(f"device_{device_idx}/weights.safetensors lacks `{name}`")
                t = sf.get_tensor(name)
                if name + ".scale" in keys:
                    t = ref.dequant_fp8_block128(t.view(torch.float8_e4m3fn), sf.get_tensor(name + ".scale")).to(torch.bfloat16)
                return t.to(device)

            return self._assemble(get, self.layout(device_idx))

    def load_full_weights(self, device) -> ModelWeights:
        """Reassemble the unsharded model from every device's shard (inverse of the sharder): used by the
        in-process parity gate and as a round-trip check of the slicing."""
        from safetensors import safe_open

        full = {}
        for d in range(self.num_devices):
            f = self.path / f"device_{d}" / "weights.safetensors"
            if not f.exists():
                raise ArtifactError(f"{f} is missing (artifact was built without weights)")
            with safe_open(str(f), framework="pt") as sf:
                keys = set(sf.keys())
                for e in self.io_manifest(d)["tensors"]:
                    name = e["name"]
                    t = sf.get_tensor(name)
                    if name + ".scale" in keys:
                        t = ref.dequant_fp8_block128(t.view(torch.float8_e4m3fn), sf.get_tensor(name + ".scale")).to(torch.bfloat16)
                    if e["axis"] < 0:
                        full.setdefault(name, t)
                        continue
                    if name not in full:
                        full[name] = torch.zeros(*_full_shape(self.cfg, name), dtype=t.dtype)
                    full[name].narrow(e["axis"], e["start"], e["len"]).copy_(t)

        def get(name):
            if name not in full:
                raise ArtifactError(f"no device holds `{name}`")
            return full[name].to(device)

        return self._assemble(get, ParallelLayout())

    def _assemble(self, get, lay: ParallelLayout) -> ModelWeights:
        cfg = self.cfg
        layers = []
        e_local = cfg.num_experts // lay.ep if cfg.is_moe else 0
        e0 = lay.ep_rank * e_local
        for b in lay.stage_layers(cfg.num_layers):
            pre = f"model.layers.{b}."
            wqkv = torch.cat([get(pre + f"self_attn.{p}_proj.weight") for p in "qkv"], dim=0).contiguous()
            if cfg.is_moe:
                w13 = torch.stack([torch.cat([get(pre + f"block_sparse_moe.experts.{e}.w1.weight"),
                                              get(pre + f"block_sparse_moe.experts.{e}.w3.weight")], dim=0)
                                   for e in range(e0, e0 + e_local)]).contiguous()
                w2 = torch.stack([get(pre + f"block_sparse_moe.experts.{e}.w2.weight") for e in range(e0, e0 + e_local)]).contiguous()
                router = get(pre + "block_sparse_moe.gate.weight")
            else:
                w13 = torch.cat([get(pre + "mlp.gate_proj.weight"), get(pre + "mlp.up_proj.weight")], dim=0).contiguous()
                w2 = get(pre + "mlp.down_proj.weight").contiguous()
                router = None
            bqkv = (torch.cat([get(pre + f"self_attn.{p}_proj.bias") for p in "qkv"]).contiguous() if cfg.qkv_bias else None)
            layers.append(LayerWeights(attn_norm=get(pre + "input_layernorm.weight"), wqkv=wqkv,
                                       wo=get(pre + "self_attn.o_proj.weight").contiguous(),
                                       ffn_norm=get(pre + "post_attention_layernorm.weight"), router=router, w13=w13, w2=w2,
                                       bqkv=bqkv))
        first, last = lay.pp_rank == 0, lay.pp_rank == lay.pp - 1
        embed = get("model.embed_tokens.weight") if first else None
        # tied embeddings: the output projection is the embedding table (under tensor parallelism both are split by
        # vocabulary rows the same way, so a rank's table shard is its shard of the output projection)
        lm_head = (embed if cfg.tie_word_embeddings else get("lm_head.weight")) if last else None
        return ModelWeights(embed=embed, layers=layers, final_norm=get("model.norm.weight") if last else None, lm_head=lm_head)


def verify_shape_compatibility(old: Artifact, new: Artifact) -> None:
    """Hot swap precondition: both artifacts expose the same weight manifest per device (names, shapes, dtypes)."""
    if old.num_devices != new.num_devices:
        raise ArtifactError(f"device count differs: {old.num_devices} vs {new.num_devices}")
    for d in range(old.num_devices):
        a = [(t["name"], t["shape"], t["dtype"]) for t in old.io_manifest(d)["tensors"]]
        b = [(t["name"], t["shape"], t["dtype"]) for t in new.io_manifest(d)["tensors"]]
        if a != b:
            raise ArtifactError(f"io.json of device {d} differs between the mounted and the new artifact")
