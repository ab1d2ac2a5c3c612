"""Straight-line, cache-free PyTorch implementation of the same decoder math (fp32 compute on bf16
weights), independent of the operator interface. It follows the HuggingFace Mixtral / Llama
modelling code step by step (RMSNorm -> attention with NeoX RoPE and causal mask -> residual ->
RMSNorm -> top-k softmax-routed SwiGLU experts or SwiGLU MLP -> residual) and serves as the
"HF-style" oracle of the parity gate and of the graph tests, in the role of the reference's Python
subprocess oracle (crates/skein_parity/reference/verify_reference.py).
"""
from __future__ import annotations

import math

import torch

from ..ops.reference import rope_inv_freq
from .config import ModelConfig
from .decoder import ModelWeights


def _rms(x, g, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)) * g.float()


def _rope(x, pos, theta, scaling=None):
    # x: [T, heads, D]
    D = x.shape[-1]
    half = D // 2
    inv = rope_inv_freq(D, theta, scaling).to(x.device)
    ang = pos.double().unsqueeze(1) * inv.unsqueeze(0)
    cos, sin = ang.cos().float().unsqueeze(1), ang.sin().float().unsqueeze(1)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)


@torch.no_grad()
def forward_full(cfg: ModelConfig, w: ModelWeights, token_ids: torch.Tensor, capture_hidden: list | None = None):
    """Full-sequence forward of ONE sequence (unsharded weights). Returns fp32 logits [T, V]."""
    T = token_ids.shape[0]
    H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    x = w.embed[token_ids.long()].float()
    pos = torch.arange(T, device=x.device)
    mask = torch.triu(torch.full((T, T), float("-inf"), device=x.device), diagonal=1)
    for lw in w.layers:
        h = _rms(x, lw.attn_norm, cfg.rms_norm_eps)
        qkv = h @ lw.wqkv.float().t()
        if getattr(lw, "bqkv", None) is not None:
            qkv = qkv + lw.bqkv.float()
        q = _rope(qkv[:, :Hq * D].view(T, Hq, D), pos, cfg.rope_theta, cfg.rope_scaling)
        k = _rope(qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D), pos, cfg.rope_theta, cfg.rope_scaling)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        G = Hq // Hkv
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D) + mask
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), v).reshape(T, Hq * D)
        x = x + a @ lw.wo.float().t()
        h = _rms(x, lw.ffn_norm, cfg.rms_norm_eps)
        # a Decoder on the same weights may have re-laid the expert matrices tile by tile: read the logical view
        w13 = lw.w13.unpack() if hasattr(lw.w13, "unpack") else lw.w13
        w2 = lw.w2.unpack() if hasattr(lw.w2, "unpack") else lw.w2
        if cfg.is_moe:
            logits = h @ lw.router.float().t()
            probs = torch.softmax(logits, dim=-1)
            topv, topi = probs.topk(cfg.top_k, dim=-1)
            topv = topv / topv.sum(-1, keepdim=True)
            y = torch.zeros_like(x)
            I = w13.shape[1] // 2
            for e in range(cfg.num_experts):
                sel = (topi == e)
                rows = sel.any(-1).nonzero().squeeze(-1)
                if rows.numel() == 0:
                    continue
                he = h[rows]
                g = he @ w13[e, :I].float().t()
                u = he @ w13[e, I:].float().t()
                o = (torch.nn.functional.silu(g) * u) @ w2[e].float().t()
                y[rows] += o * (topv[rows] * sel[rows].float()).sum(-1, keepdim=True)
            x = x + y
        else:
            I = w13.shape[0] // 2
            g = h @ w13[:I].float().t()
            u = h @ w13[I:].float().t()
            x = x + (torch.nn.functional.silu(g) * u) @ w2.float().t()
        if capture_hidden is not None:
            capture_hidden.append(x.clone())
    h = _rms(x, w.final_norm, cfg.rms_norm_eps)
    return h @ w.lm_head.float().t()
