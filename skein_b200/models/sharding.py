"""Slice a full set of weights into one rank's shard.

Roles follow the reference's shard_role table (crates/skein_emit/src/shard_role.rs:35-166: pipeline
stage first, then expert ownership, then tensor parallelism; column-parallel q/k/v/w1/w3/lm_head,
row-parallel o/w2), with two differences: experts are owned in contiguous blocks
(expert e lives on ep rank e // (E / ep)) so that a rank's experts form one slice of the stacked
weight. The embedding table is vocabulary-sharded on request (`shard_embed`; the decoder then sums the ranks'
lookups inside its first RMSNorm) and replicated otherwise.
"""
from __future__ import annotations

import torch

from .config import ModelConfig, ParallelLayout
from .decoder import LayerWeights, ModelWeights, shard_shapes


def _rows(t: torch.Tensor, start: int, n: int) -> torch.Tensor:
    return t[start:start + n]


def shard_layer(lw: LayerWeights, cfg: ModelConfig, lay: ParallelLayout) -> LayerWeights:
    sh = shard_shapes(cfg, lay)
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size
    r = lay.tp_rank
    q = _rows(lw.wqkv, r * sh["Hq"] * D, sh["Hq"] * D)
    k = _rows(lw.wqkv, Hq * D + r * sh["Hkv"] * D, sh["Hkv"] * D)
    v = _rows(lw.wqkv, (Hq + Hkv) * D + r * sh["Hkv"] * D, sh["Hkv"] * D)
    wqkv = torch.cat([q, k, v], dim=0).contiguous()
    bqkv = None
    if lw.bqkv is not None:       # the bias rows follow their weight rows
        bqkv = torch.cat([_rows(lw.bqkv, r * sh["Hq"] * D, sh["Hq"] * D), _rows(lw.bqkv, Hq * D + r * sh["Hkv"] * D, sh["Hkv"] * D),
                          _rows(lw.bqkv, (Hq + Hkv) * D + r * sh["Hkv"] * D, sh["Hkv"] * D)]).contiguous()
    wo = lw.wo[:, r * sh["Hq"] * D:(r + 1) * sh["Hq"] * D].contiguous()
    Il = sh["I"]
    if cfg.is_moe:
        e0 = lay.ep_rank * sh["E_local"]
        w13 = lw.w13[e0:e0 + sh["E_local"]]
        w13 = torch.cat([w13[:, r * Il:(r + 1) * Il], w13[:, I + r * Il:I + (r + 1) * Il]], dim=1).contiguous()
        w2 = lw.w2[e0:e0 + sh["E_local"], :, r * Il:(r + 1) * Il].contiguous()
        router = lw.router
    else:
        w13 = torch.cat([lw.w13[r * Il:(r + 1) * Il], lw.w13[I + r * Il:I + (r + 1) * Il]], dim=0).contiguous()
        w2 = lw.w2[:, r * Il:(r + 1) * Il].contiguous()
        router = None
    return LayerWeights(attn_norm=lw.attn_norm, wqkv=wqkv, wo=wo, ffn_norm=lw.ffn_norm, router=router, w13=w13, w2=w2, bqkv=bqkv)


def shard_model(full: ModelWeights, cfg: ModelConfig, lay: ParallelLayout, device=None, shard_embed: bool = False) -> ModelWeights:
    """full holds every block (pp = tp = ep = 1 shapes). Returns the shard of `lay.rank`, moved to `device`.
    shard_embed: vocabulary-parallel embedding table (this rank's rows, zero-padded to the common shard size), whose
    lookups the decoder sums inside its first RMSNorm; otherwise the table is replicated."""
    sh = shard_shapes(cfg, lay)
    stage = lay.stage_layers(cfg.num_layers)
    first, last = lay.pp_rank == 0, lay.pp_rank == lay.pp - 1

    def mv(t):
        return t if (t is None or device is None) else t.to(device)

    layers = []
    for i in stage:
        s = shard_layer(full.layers[i], cfg, lay)
        layers.append(LayerWeights(**{k: mv(getattr(s, k)) for k in
                                      ("attn_norm", "wqkv", "wo", "ffn_norm", "router", "w13", "w2", "bqkv")}))
    v0 = lay.tp_rank * sh["V_local"]
    lm = full.lm_head[v0:v0 + sh["V_local"]].contiguous() if last else None
    emb = full.embed
    if shard_embed and lay.tp > 1 and first:
        emb = torch.zeros(sh["V_local"], full.embed.shape[1], dtype=full.embed.dtype)
        rows = full.embed[v0:v0 + sh["V_local"]]
        emb[:rows.shape[0]] = rows
    return ModelWeights(embed=mv(emb) if first else None, layers=layers,
                        final_norm=mv(full.final_norm) if last else None, lm_head=mv(lm))
