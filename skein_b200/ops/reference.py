"""Plain PyTorch (fp32 math) reference of every operator in skein_b200.ops.

These are the oracles the CUDA kernels are tested against, the implementation used on CPU-only
machines, and the math of the bf16 parity reference. Shapes and conventions are identical to the
CUDA operators; see skein_b200/ops/functional.py.
"""
from __future__ import annotations

import math

import torch


def linear(x, w, residual=None):
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def swiglu_linear(x, w13):
    """w13 = [gate rows; up rows] stacked along dim 0."""
    inter = w13.shape[0] // 2
    g = x.float() @ w13[:inter].float().t()
    u = x.float() @ w13[inter:].float().t()
    return (torch.nn.functional.silu(g) * u).to(x.dtype)


def grouped_linear(xs, w, counts, offsets, swiglu=False):
    """xs: [rows, K] expert-sorted; w: [E, F(or 2I), K]; rows of expert e are offsets[e] : offsets[e]+counts[e]."""
    E = w.shape[0]
    F = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.zeros(xs.shape[0], F, dtype=xs.dtype, device=xs.device)
    counts = counts.tolist()
    offsets = offsets.tolist()
    for e in range(E):
        c, o = counts[e], offsets[e]
        if c == 0:
            continue
        out[o:o + c] = swiglu_linear(xs[o:o + c], w[e]) if swiglu else linear(xs[o:o + c], w[e])
    return out


def reduce_residual_rmsnorm(residual, partial, gamma, eps, row_idx=None, row_w=None, owner_ids=None, experts_per_owner=1,
                            owner_span=1):
    """partial: [n_src, rows, H] or None. Returns (residual_out bf16-rounded, normed_out or None)."""
    acc = residual.float() if residual is not None else None
    if partial is not None:
        p = partial.float()
        if row_idx is None:
            contrib = p.sum(0)
        else:
            B, topk = row_idx.shape
            contrib = torch.zeros(B, p.shape[-1], dtype=torch.float32, device=p.device)
            for j in range(topk):
                idx = row_idx[:, j].long().clamp(min=0)
                wj = row_w[:, j].float().unsqueeze(1)
                valid = (row_idx[:, j] >= 0).float().unsqueeze(1)
                for s in range(p.shape[0]):
                    mine = 1.0
                    if owner_ids is not None:
                        lo = (owner_ids[:, j].long() // experts_per_owner) * owner_span
                        mine = ((s >= lo) & (s < lo + owner_span)).float().unsqueeze(1)
                    contrib = contrib + mine * valid * wj * p[s][idx]
        acc = contrib if acc is None else acc + contrib
    dt = residual.dtype if residual is not None else partial.dtype
    res_out = acc.to(dt)
    if gamma is None:
        return res_out, None
    xf = res_out.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    normed = (xf * inv).to(dt).float() * gamma.float()
    return res_out, normed.to(dt)


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None = None):
    """The head_dim / 2 rotation frequencies (float64), with the checkpoint's frequency scaling applied: none, "linear"
    (every frequency divided by `factor`) or "llama3" (Llama 3.1 and later: wavelengths beyond the original context
    are stretched by `factor`, short ones kept, the band in between blended). Other schemes are refused by the importer."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim))
    kind = (scaling or {}).get("rope_type") or (scaling or {}).get("type") or "default"
    if kind == "default":
        return inv
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv / factor
    if kind == "llama3":
        lo, hi = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - lo) / (hi - lo)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > orig / lo, inv / factor, inv)
        medium = ~(wavelen < orig / hi) & ~(wavelen > orig / lo)
        return torch.where(medium, blended, out)
    raise ValueError(f"rope scaling {kind!r} is not supported")


def rope_cos_sin_table(max_pos: int, head_dim: int, theta: float, device=None, scaling: dict | None = None):
    """[max_pos, head_dim/2, 2] fp32 (cos, sin), the table the RoPE kernel reads."""
    inv_freq = rope_inv_freq(head_dim, theta, scaling)
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv_freq.unsqueeze(0)
    tab = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32)
    return tab.to(device) if device is not None else tab


def rope_kv_append(qkv, positions, seq_of_token, block_table, cos_sin, kv_cache, Hq, Hkv, D):
    """In-place on qkv (q rotated) and kv_cache (k rotated + v written). positions < 0 rows are skipped."""
    T = qkv.shape[0]
    page_size = kv_cache.shape[3]
    half = D // 2
    v = qkv.view(T, Hq + 2 * Hkv, D)
    pos = positions.long()
    ok = pos >= 0
    cs = cos_sin[pos.clamp(min=0)]  # [T, half, 2]
    cos, sin = cs[..., 0].unsqueeze(1), cs[..., 1].unsqueeze(1)
    qk = v[:, :Hq + Hkv].float()
    x0, x1 = qk[..., :half], qk[..., half:]
    rot = torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1).to(qkv.dtype)
    v[:, :Hq + Hkv][ok] = rot[ok]
    seqs = seq_of_token.long() if seq_of_token is not None else torch.arange(T, device=qkv.device)
    for t in range(T):
        if not bool(ok[t]):
            continue
        p = int(pos[t])
        page = int(block_table[int(seqs[t]), p // page_size])
        kv_cache[page, 0, :, p % page_size] = v[t, Hq:Hq + Hkv]
        kv_cache[page, 1, :, p % page_size] = v[t, Hq + Hkv:]


def _gather_kv(kv_cache, block_table_row, length):
    page_size = kv_cache.shape[3]
    n_pages = (length + page_size - 1) // page_size
    pages = block_table_row[:n_pages].long()
    k = kv_cache[pages, 0].permute(1, 0, 2, 3).reshape(kv_cache.shape[2], -1, kv_cache.shape[4])[:, :length]
    v = kv_cache[pages, 1].permute(1, 0, 2, 3).reshape(kv_cache.shape[2], -1, kv_cache.shape[4])[:, :length]
    return k.float(), v.float()  # [Hkv, L, D]


def attn_decode(q, kv_cache, block_table, seq_lens, Hq, Hkv, D, scale=None):
    """q: [B, >= Hq*D] (first Hq*D columns are the query heads). Returns [B, Hq*D]."""
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq * D, dtype=q.dtype, device=q.device)
    G = Hq // Hkv
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        k, v = _gather_kv(kv_cache, block_table[b], L)
        qb = q[b, :Hq * D].float().view(Hkv, G, D)
        s = torch.einsum("hgd,hld->hgl", qb, k) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hgl,hld->hgd", p, v).reshape(-1).to(q.dtype)
    return out


def attn_prefill(q, kv_cache, block_table, q_start, q_len, kv_len, Hq, Hkv, D, scale=None):
    """Causal attention of each sequence's chunk (rows q_start : q_start+q_len of q) over its cache."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros(q.shape[0], Hq * D, dtype=q.dtype, device=q.device)
    G = Hq // Hkv
    for s_i in range(len(q_len)):
        ql, kl, qs = int(q_len[s_i]), int(kv_len[s_i]), int(q_start[s_i])
        if ql == 0:
            continue
        k, v = _gather_kv(kv_cache, block_table[s_i], kl)
        qb = q[qs:qs + ql, :Hq * D].float().view(ql, Hkv, G, D)
        s = torch.einsum("thgd,hld->thgl", qb, k) * scale
        pos = torch.arange(ql, device=q.device) + (kl - ql)
        mask = torch.arange(kl, device=q.device).unsqueeze(0) > pos.unsqueeze(1)  # [ql, kl]
        s = s.masked_fill(mask[:, None, None, :], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qs + ql] = torch.einsum("thgl,hld->thgd", p, v).reshape(ql, -1).to(q.dtype)
    return out


def router_topk(x, wg, topk):
    logits = (x.float() @ wg.float().t()).to(x.dtype).float()
    # ties -> lower expert index: stable descending sort
    order = torch.sort(logits, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :topk].to(torch.int32)
    w = torch.softmax(order.values[:, :topk], dim=-1)
    return ids, w, logits


def router_plan(expert_ids, E, e_first=0, e_count=None):
    """Stable expert-sorted layout: returns counts[E], offsets[E+1], row_of[T*topk], src_token[rows]."""
    e_count = E if e_count is None else e_count
    flat = expert_ids.reshape(-1).long()
    topk = expert_ids.shape[1]
    n = flat.numel()
    mine = (flat >= e_first) & (flat < e_first + e_count)
    counts = torch.zeros(E, dtype=torch.int32, device=flat.device)
    for e in range(e_first, e_first + e_count):
        counts[e] = int(((flat == e)).sum())
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=flat.device)
    offsets[1:] = torch.cumsum(counts, 0)
    row_of = torch.full((n,), -1, dtype=torch.int32, device=flat.device)
    src_token = torch.zeros(max(int(offsets[-1]), 1), dtype=torch.int32, device=flat.device)
    nxt = offsets[:-1].clone().tolist()
    fl = flat.tolist()
    ml = mine.tolist()
    for i in range(n):
        if ml[i]:
            e = fl[i]
            row_of[i] = nxt[e]
            src_token[nxt[e]] = i // topk
            nxt[e] += 1
    return counts, offsets, row_of, src_token


def sample_argmax(logits):
    lf = logits.float()
    mx = lf.max(dim=-1, keepdim=True).values
    V = lf.shape[-1]
    idx = torch.where(lf == mx, torch.arange(V, device=lf.device).expand_as(lf), torch.full_like(lf, V, dtype=torch.long))
    return idx.min(dim=-1).values.to(torch.int32)


_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def sample(logits, temperature, top_k, top_p, seeds, step):
    """Temperature / top-k / top-p sampling with the counter-based generator of csrc/kernels/sample.cu: the
    candidate list is the top_k (at most 64) largest logits in (value descending, index ascending) order, top_p
    keeps its shortest prefix whose probability reaches p, and one uniform draw from splitmix64(seed ^
    splitmix64(step + 1)) selects the token. Rows with temperature <= 0 are greedy."""
    import numpy as np
    lf = logits.float()
    B, V = lf.shape
    steps = [0] * B if step is None else ([int(step.reshape(-1)[0])] * B if step.numel() == 1 else [int(x) for x in step[:B]])
    out = []
    f32 = np.float32
    for b in range(B):
        T = float(temperature[b]) if temperature is not None else 0.0
        K = 1 if T <= 0 else (int(top_k[b]) if top_k is not None else 64)
        if K <= 0 or K > 64:
            K = 64
        K = min(K, V)
        row = lf[b]
        order = sorted(range(V), key=lambda i: (-float(row[i]), i))[:K]
        if K == 1:
            out.append(order[0])
            continue
        vals = [f32(row[i]) for i in order]
        pr = [f32(np.exp((v - vals[0]) / f32(T), dtype=f32)) for v in vals]
        den = f32(0)
        for x in pr:
            den = f32(den + x)
        P = f32(top_p[b]) if top_p is not None else f32(1)
        keep, cum = K, f32(0)
        for k in range(K):
            cum = f32(cum + f32(pr[k] / den))
            if cum >= P:
                keep = k + 1
                break
        kept = f32(0)
        for k in range(keep):
            kept = f32(kept + pr[k])
        seed = (int(seeds[b]) & _M64) if seeds is not None else 0x1234
        s64 = _splitmix64(seed ^ _splitmix64((steps[b] + 1) & _M64))
        u = f32(f32(f32((s64 >> 40) & 0xFFFFFF) / f32(16777216.0)) * kept)
        run, pick = f32(0), order[keep - 1]
        for k in range(keep):
            run = f32(run + pr[k])
            if u < run:
                pick = order[k]
                break
        out.append(pick)
    return torch.tensor(out, dtype=torch.int32)


def embed(ids, table, vocab_start=0):
    loc = ids.long() - vocab_start
    ok = (loc >= 0) & (loc < table.shape[0])
    out = table[loc.clamp(0, table.shape[0] - 1)]
    return out * ok.unsqueeze(1).to(out.dtype)


def quant_fp8_block128(x, pow2_scales: bool = False):
    """Returns (q float8_e4m3fn [rows, K], scales fp32 [rows, K/128]). pow2_scales: every scale is the smallest power
    of two that brings the block's largest magnitude inside the e4m3 range (used for weights)."""
    rows, K = x.shape
    xb = x.float().view(rows, K // 128, 128)
    amax = xb.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    if pow2_scales:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (xb / scale.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(rows, K)
    return q, scale


def dequant_fp8_block128(q, scale):
    rows, K = q.shape
    return (q.float().view(rows, K // 128, 128) * scale.unsqueeze(-1)).view(rows, K)
