"""Model and parallel-layout descriptions used by the decoder graph.

ModelConfig is read from a HuggingFace ``config.json`` (MixtralForCausalLM, LlamaForCausalLM and
the Llama-shaped Mistral / Qwen2 families). The reference imports Mixtral only
(crates/skein_ir/src/model/mod.rs:33-47, model/mixtral.rs:74-372) and rejects the rest; here the
dense Llama-style block is a Mixtral block with a plain SwiGLU MLP instead of routed experts.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path

MOE_ARCHS = {"MixtralForCausalLM"}
DENSE_ARCHS = {"LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM"}


class ImportError_(ValueError):
    """A config.json that cannot be turned into a consistent model."""


@dataclass
class ModelConfig:
    architecture: str = "MixtralForCausalLM"
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-5
    rope_theta: float = 1e6
    num_experts: int = 8          # 0 = dense MLP
    top_k: int = 2
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    name: str = "mixtral-8x7b"
    qkv_bias: bool = False        # the q / k / v projections carry a bias each (Qwen2)
    eos_token_id: int = -1        # token that ends a generation (-1: none known)
    rope_scaling: dict | None = None   # the checkpoint's RoPE frequency scaling ("linear" or "llama3"), None = plain RoPE

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def validate(self) -> None:
        if self.num_heads % self.num_kv_heads != 0:
            raise ImportError_("num_attention_heads must be a multiple of num_key_value_heads")
        if self.is_moe and not (1 <= self.top_k <= self.num_experts):
            raise ImportError_("num_experts_per_tok must be in [1, num_local_experts]")
        if self.head_dim % 2 != 0:
            raise ImportError_("head_dim must be even (RoPE rotates pairs)")

    def param_count(self) -> int:
        H, I, D = self.hidden_size, self.intermediate_size, self.head_dim
        attn = H * (self.num_heads * D) * 2 + H * (self.num_kv_heads * D) * 2
        if self.qkv_bias:
            attn += (self.num_heads + 2 * self.num_kv_heads) * D
        ffn = 3 * H * I * max(self.num_experts, 1) + (H * self.num_experts if self.is_moe else 0)
        per_block = attn + ffn + 2 * H
        emb = self.vocab_size * H
        return self.num_layers * per_block + emb + H + (0 if self.tie_word_embeddings else emb)

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_hf_dict(d: dict, name: str | None = None) -> "ModelConfig":
        archs = d.get("architectures") or []
        if not archs:
            raise ImportError_("config.json has no `architectures`")
        arch = archs[0]
        if arch not in MOE_ARCHS | DENSE_ARCHS:
            raise ImportError_(f"architecture {arch} is not supported")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ImportError_(f"hidden_act {act!r} is not supported (only silu)")
        H = int(d["hidden_size"])
        nh = int(d["num_attention_heads"])
        hd = d.get("head_dim") or (H // nh)
        if d.get("head_dim") is None and H % nh != 0:
            raise ImportError_("hidden_size is not divisible by num_attention_heads and head_dim is absent")
        # newer checkpoints nest theta and the scaling scheme in `rope_parameters`; older ones have `rope_theta` and
        # `rope_scaling` at the top level
        rp = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rp.get("rope_theta", 1e4))
        scaling = d.get("rope_scaling") or ({k: v for k, v in rp.items() if k != "rope_theta"} if rp else None)
        kind = (scaling or {}).get("rope_type") or (scaling or {}).get("type") or "default"
        if kind == "default":
            scaling = None
        elif kind not in ("linear", "llama3"):
            raise ImportError_(f"rope scaling {kind!r} is not supported (plain, linear and llama3 are)")
        if float(d.get("partial_rotary_factor", rp.get("partial_rotary_factor", 1.0)) or 1.0) != 1.0:
            raise ImportError_("partial rotary embeddings are not supported")
        if d.get("mlp_bias"):
            raise ImportError_("mlp_bias = true is not supported")
        cfg = ModelConfig(
            architecture=arch, hidden_size=H, intermediate_size=int(d["intermediate_size"]),
            num_layers=int(d["num_hidden_layers"]), num_heads=nh,
            num_kv_heads=int(d.get("num_key_value_heads", nh)), head_dim=int(hd), vocab_size=int(d["vocab_size"]),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)), rope_theta=float(theta),
            num_experts=int(d.get("num_local_experts", 0)) if arch in MOE_ARCHS else 0,
            top_k=int(d.get("num_experts_per_tok", 0)) if arch in MOE_ARCHS else 0,
            max_position_embeddings=int(d.get("max_position_embeddings", 8192)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            name=name or d.get("_name_or_path") or d.get("model_type", "model"),
            qkv_bias=arch == "Qwen2ForCausalLM", rope_scaling=dict(scaling) if scaling else None)
        eos = d.get("eos_token_id")
        if isinstance(eos, (list, tuple)):      # several end tokens: the engine stops on one, the first listed
            eos = eos[0] if eos else None
        cfg.eos_token_id = int(eos) if eos is not None else -1
        # Sliding-window attention (Mistral v0.1; Qwen2 only with use_sliding_window): the attention kernels attend over the
        # whole context, which is the same function as long as a sequence is no longer than the window, so the window
        # becomes the position limit and longer requests are refused instead of being answered differently.
        sw = d.get("sliding_window")
        if sw and (arch != "Qwen2ForCausalLM" or d.get("use_sliding_window")) and int(sw) < cfg.max_position_embeddings:
            cfg.max_position_embeddings = int(sw)
        if d.get("attention_bias") and not cfg.qkv_bias:
            raise ImportError_(f"attention_bias = true (biases on q, k, v and o_proj) is not supported for {arch}")
        cfg.validate()
        return cfg

    def to_hf_dict(self) -> dict:
        """The HuggingFace config.json fields that describe this model (what the planner and the lowering read)."""
        d = {"architectures": [self.architecture], "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
             "num_hidden_layers": self.num_layers, "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
             "head_dim": self.head_dim, "vocab_size": self.vocab_size, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
             "max_position_embeddings": self.max_position_embeddings, "tie_word_embeddings": self.tie_word_embeddings,
             "hidden_act": "silu"}
        if self.is_moe:
            d.update(num_local_experts=self.num_experts, num_experts_per_tok=self.top_k)
        if self.rope_scaling:
            d["rope_scaling"] = dict(self.rope_scaling)
        return d

    @staticmethod
    def from_file(path) -> "ModelConfig":
        p = Path(path)
        return ModelConfig.from_hf_dict(json.loads(p.read_text()), name=p.stem.replace("_config", ""))


def mixtral_8x7b() -> ModelConfig:
    return ModelConfig()


def mixtral_8x22b() -> ModelConfig:
    return ModelConfig(hidden_size=6144, intermediate_size=16384, num_layers=56, num_heads=48, num_kv_heads=8,
                       head_dim=128, vocab_size=32768, rope_theta=1e6, num_experts=8, top_k=2,
                       max_position_embeddings=65536, name="mixtral-8x22b")


def llama3_70b() -> ModelConfig:
    return ModelConfig(architecture="LlamaForCausalLM", hidden_size=8192, intermediate_size=28672, num_layers=80,
                       num_heads=64, num_kv_heads=8, head_dim=128, vocab_size=128256, rms_norm_eps=1e-5,
                       rope_theta=5e5, num_experts=0, top_k=0, max_position_embeddings=8192, name="llama3-70b")


def tiny_mixtral(layers=2, hidden=256, inter=512, heads=4, kv_heads=2, experts=4, vocab=512) -> ModelConfig:
    """A small Mixtral-shaped model for tests (head_dim stays 128: the attention kernels require it)."""
    return ModelConfig(hidden_size=hidden, intermediate_size=inter, num_layers=layers, num_heads=heads,
                       num_kv_heads=kv_heads, head_dim=128, vocab_size=vocab, num_experts=experts, top_k=2,
                       max_position_embeddings=4096, name="tiny-mixtral")


def tiny_llama(layers=2, hidden=256, inter=512, heads=4, kv_heads=2, vocab=512) -> ModelConfig:
    return ModelConfig(architecture="LlamaForCausalLM", hidden_size=hidden, intermediate_size=inter,
                       num_layers=layers, num_heads=heads, num_kv_heads=kv_heads, head_dim=128, vocab_size=vocab,
                       rope_theta=5e5, num_experts=0, top_k=0, max_position_embeddings=4096, name="tiny-llama")


@dataclass
class ParallelLayout:
    """Where this rank sits in the TP x PP x EP grid (device coordinates are lexicographic in
    (pp, ep, tp), tp fastest, as in the reference's Placement: crates/skein_cost/src/cluster.rs:100-169)."""
    tp: int = 1
    pp: int = 1
    ep: int = 1
    rank: int = 0

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.ep

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def ep_rank(self) -> int:
        return (self.rank // self.tp) % self.ep

    @property
    def pp_rank(self) -> int:
        return self.rank // (self.tp * self.ep)

    def tp_group(self) -> list[int]:
        base = self.rank - self.tp_rank
        return [base + i for i in range(self.tp)]

    def ep_group(self) -> list[int]:
        base = self.pp_rank * self.tp * self.ep + self.tp_rank
        return [base + i * self.tp for i in range(self.ep)]

    def pp_group(self) -> list[int]:
        inner = self.rank % (self.tp * self.ep)
        return [inner + s * self.tp * self.ep for s in range(self.pp)]

    def stage_layers(self, num_layers: int) -> range:
        """Blocks of this pipeline stage; the remainder is spread over the first stages."""
        base, rem = divmod(num_layers, self.pp)
        s = self.pp_rank
        start = s * base + min(s, rem)
        return range(start, start + base + (1 if s < rem else 0))
