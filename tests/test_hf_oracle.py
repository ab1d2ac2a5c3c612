"""The runtime's decoder against HuggingFace `transformers` on tiny random models of every supported family (CPU):
Mixtral, Llama, Mistral, Qwen2 (q / k / v biases) and a Llama with tied input / output embeddings.

The checkpoint is written by transformers, compiled into an artifact by this framework's own pipeline (HF tensor
names, expert stacking, q/k/v fusion), and both sides run the same prompts. This is the one oracle that is not
written by the same hand as the kernels, the role of the reference's Python subprocess
(crates/skein_parity/src/reference.rs:65-104, crates/skein_parity/reference/verify_reference.py)."""
import json
from pathlib import Path

import pytest
import torch

transformers = pytest.importorskip("transformers")

from skein_b200 import core  # noqa: E402
from skein_b200.compile import parity  # noqa: E402
from skein_b200.compile.artifact import Artifact, WeightSource, build_artifact  # noqa: E402
from skein_b200.models.config import ModelConfig  # noqa: E402

ROOT = Path(__file__).resolve().parent.parent
INPUTS = ((ROOT / "cluster/b200_1x.toml").read_text(), (ROOT / "cluster/sample_trace.jsonl").read_text(),
          (ROOT / "models/llama3_70b_drift.toml").read_text(), (ROOT / "cluster/cost_constants.toml").read_text())


def _hf_model(kind):
    torch.manual_seed(0)
    common = dict(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=128, max_position_embeddings=256, rms_norm_eps=1e-5, tie_word_embeddings=False)
    if kind == "mixtral":
        cfg = transformers.MixtralConfig(num_local_experts=4, num_experts_per_tok=2, rope_theta=1e6, **common)
        m = transformers.MixtralForCausalLM(cfg)
    elif kind == "qwen2":        # q / k / v projections carry biases
        cfg = transformers.Qwen2Config(rope_theta=1e6, use_sliding_window=False, **{k: v for k, v in common.items() if k != "head_dim"},)
        m = transformers.Qwen2ForCausalLM(cfg)
    elif kind == "mistral":
        cfg = transformers.MistralConfig(rope_theta=1e4, sliding_window=None, **common)
        m = transformers.MistralForCausalLM(cfg)
    elif kind == "llama-rope-llama3":      # Llama 3.1-style frequency scaling
        cfg = transformers.LlamaConfig(rope_theta=5e5, rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
                                       **common)
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "llama-rope-linear":
        cfg = transformers.LlamaConfig(rope_theta=5e5, rope_scaling={"rope_type": "linear", "factor": 4.0}, **common)
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "llama-tied":   # the output projection is the embedding table
        cfg = transformers.LlamaConfig(rope_theta=5e5, **{**common, "tie_word_embeddings": True})
        m = transformers.LlamaForCausalLM(cfg)
    else:
        cfg = transformers.LlamaConfig(rope_theta=5e5, **common)
        m = transformers.LlamaForCausalLM(cfg)
    with torch.no_grad():
        for name, p in m.named_parameters():      # larger than the default init so that attention and routing matter; bf16-exact
            if p.dim() > 1:
                p.normal_(0.0, 0.06)
            elif "bias" in name:
                p.normal_(0.0, 0.5)
            p.copy_(p.to(torch.bfloat16).float())
    return m.eval()


@pytest.mark.parametrize("kind", ["mixtral", "llama", "mistral", "qwen2", "llama-tied", "llama-rope-llama3", "llama-rope-linear"])
def test_decoder_matches_huggingface_transformers(kind, tmp_path):
    hf = _hf_model(kind)
    ckpt = tmp_path / "ckpt"
    hf.save_pretrained(ckpt, safe_serialization=True)
    cfg_json = (ckpt / "config.json").read_text()
    d = json.loads(cfg_json)      # as transformers wrote it: recent versions nest theta and the scaling in `rope_parameters`
    cfg = ModelConfig.from_hf_dict(d)
    assert (cfg.rope_scaling is not None) == ("rope" in kind) and cfg.rope_theta == (1e6 if kind in ("mixtral", "qwen2") else 1e4 if kind == "mistral" else 5e5)
    plan = core.extract_plan(cfg_json, *INPUTS, {"force_batch": 4}, [["bf16", "bf16", "bf16"]])["plan_json"]
    art = Artifact(build_artifact(plan, cfg_json, tmp_path / "art", WeightSource(cfg, str(ckpt))))
    ours = parity.ArtifactForward(art, "cpu")
    oracle = parity.HFForward(ckpt, "float32")
    dense = parity.DenseForward(art.cfg, art.load_full_weights("cpu"))     # the in-process oracle of the parity gate
    g = torch.Generator().manual_seed(1)
    agree, flipped = 0, 0
    for n in (5, 23, 40):
        prompt = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        hid, lg = ours.run(prompt)
        hid_hf, lg_hf = oracle.run(prompt)
        hid_d, lg_d = dense.run(prompt)
        assert len(hid) == len(hid_hf) == len(hid_d) == cfg.num_layers
        for a, b, c in zip(hid, hid_hf, hid_d):
            # the straight-line fp32 model is the same function as transformers, to rounding
            assert (c - b).pow(2).mean() / b.pow(2).mean() < 1e-9
            # the runtime's decoder keeps activations in bf16: relative MSE per token of the residual stream; a
            # token whose router scores are nearly tied may take another expert under that rounding
            tok = (a - b).pow(2).mean(-1) / b.pow(2).mean(-1)
            flipped += int((tok > 1e-3).sum())
            assert tok.median() < 2e-4, tok
        assert core.kl_divergence(lg_hf.tolist(), lg_d.tolist()) < 1e-9
        assert core.kl_divergence(lg_hf.tolist(), lg.tolist()) < 1e-3
        agree += int(torch.argmax(lg)) == int(torch.argmax(lg_hf))
    assert agree >= 2 and flipped <= (2 if kind == "mixtral" else 0)
