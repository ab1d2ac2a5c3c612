"""Decoder-only transformer (Mixtral MoE blocks or Llama dense blocks) over the operator interface.

The graph is the same for prefill and decode; only the attention operator differs. Per block:

    normed -> fused q/k/v projection -> RoPE + paged-KV append -> attention -> o_proj
           -> [sum partials + residual + RMSNorm]                      (one fused kernel)
           -> MoE: router top-k -> expert-sorted gather -> grouped gate/up GEMM with SwiGLU epilogue
                   -> grouped down GEMM            | dense: gate/up GEMM with SwiGLU -> down GEMM
           -> [top-k weighted combine + sum partials + residual + next block's RMSNorm] (one kernel)

Under tensor parallelism the two row-parallel projections (o_proj, down) store their partial output
straight into every peer's buffer from the GEMM epilogue and the fused reduce kernel that follows
waits on the peers' flags, so a block has no stand-alone collective launch.

This is the role of the reference's op wiring (crates/skein_emit/src/op_wiring.rs:740-902 wire_block,
:904 attention, :1153-1304 MoE variants, :1787 rms_norm, :2431-2472 RoPE), with PyTorch holding
the graph instead of luminal and hand-written kernels instead of searched ones.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field

import torch

from .. import ops
from ..ops import fp8
from ..ops import reference as ref
from .config import ModelConfig, ParallelLayout


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor            # [H]
    wqkv: torch.Tensor                 # [(Hq + 2 Hkv) / tp * D, H]   q rows, then k rows, then v rows
    wo: torch.Tensor                   # [H, Hq / tp * D]
    ffn_norm: torch.Tensor             # [H]
    router: torch.Tensor | None        # [E, H]
    w13: torch.Tensor                  # MoE: [E_local, 2 I / tp, H] (gate rows first); dense: [2 I / tp, H]
    w2: torch.Tensor                   # MoE: [E_local, H, I / tp];                     dense: [H, I / tp]
    # block-scaled fp8 copies (present when the plan's dtype map selects fp8 for this block)
    fp8: dict = field(default_factory=dict)


@dataclass
class ModelWeights:
    embed: torch.Tensor | None         # [V, H] (first pipeline stage)
    layers: list                       # LayerWeights of this stage's blocks
    final_norm: torch.Tensor | None    # [H] (last stage)
    lm_head: torch.Tensor | None       # [V / tp, H] (last stage)


def shard_shapes(cfg: ModelConfig, lay: ParallelLayout):
    if cfg.num_heads % lay.tp or cfg.num_kv_heads % lay.tp:
        raise ValueError(f"tp={lay.tp} must divide the query heads ({cfg.num_heads}) and kv heads ({cfg.num_kv_heads})")
    if cfg.intermediate_size % lay.tp:
        raise ValueError("tp must divide intermediate_size")
    if cfg.is_moe and cfg.num_experts % lay.ep:
        raise ValueError("ep must divide the number of experts")
    if not cfg.is_moe and lay.ep != 1:
        raise ValueError("expert parallelism needs a MoE model")
    return dict(Hq=cfg.num_heads // lay.tp, Hkv=cfg.num_kv_heads // lay.tp, I=cfg.intermediate_size // lay.tp,
                E_local=(cfg.num_experts // lay.ep) if cfg.is_moe else 0,
                V_local=(cfg.vocab_size + lay.tp - 1) // lay.tp)


def random_weights(cfg: ModelConfig, lay: ParallelLayout, device, seed: int = 0, std: float = 0.02,
                   dtype=torch.bfloat16, shard_embed: bool = False) -> ModelWeights:
    """Random-init weights N(0, std) of this rank's shard shapes (norm gains are 1, as HF initialises them).
    shard_embed: the embedding table holds only this rank's vocabulary rows (tensor parallelism)."""
    sh = shard_shapes(cfg, lay)
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1000003 + lay.rank)
    H, D = cfg.hidden_size, cfg.head_dim

    def rnd(*shape):
        t = torch.empty(*shape, dtype=dtype, device=device)
        t.normal_(0.0, std, generator=g)
        return t

    layers = []
    for _ in lay.stage_layers(cfg.num_layers):
        if cfg.is_moe:
            router, w13, w2 = rnd(cfg.num_experts, H), rnd(sh["E_local"], 2 * sh["I"], H), rnd(sh["E_local"], H, sh["I"])
        else:
            router, w13, w2 = None, rnd(2 * sh["I"], H), rnd(H, sh["I"])
        layers.append(LayerWeights(
            attn_norm=torch.ones(H, dtype=dtype, device=device), wqkv=rnd((sh["Hq"] + 2 * sh["Hkv"]) * D, H),
            wo=rnd(H, sh["Hq"] * D), ffn_norm=torch.ones(H, dtype=dtype, device=device), router=router, w13=w13, w2=w2))
    first, last = lay.pp_rank == 0, lay.pp_rank == lay.pp - 1
    return ModelWeights(
        embed=rnd(sh["V_local"] if (shard_embed and lay.tp > 1) else cfg.vocab_size, H) if first else None, layers=layers,
        final_norm=torch.ones(H, dtype=dtype, device=device) if last else None,
        lm_head=rnd(sh["V_local"], H) if last else None)


def quantize_blocks(weights: ModelWeights, blocks, names=("wqkv", "wo", "w13", "w2"), drop_bf16: bool = True) -> None:
    """Replace the named projections of the listed blocks (indices into weights.layers) by block-scaled e4m3
    copies, as the plan's per-layer dtype map asks. With drop_bf16 the bf16 tensors are released."""
    for b in blocks:
        lw = weights.layers[b]
        for name in names:
            w = getattr(lw, name)
            if w is None or name in lw.fp8 or w.shape[-1] % 128 != 0:
                continue
            lw.fp8[name] = fp8.quantize_weight(w)
            if drop_bf16:
                setattr(lw, name, None)


@dataclass
class BatchInputs:
    """Device-side description of one step (prefill chunk or decode step)."""
    token_ids: torch.Tensor            # [T] int32
    positions: torch.Tensor            # [T] int32, -1 marks a padding row
    block_table: torch.Tensor          # [S, max_blocks] int32
    seq_lens: torch.Tensor             # [S] int32: cache length of each sequence after this step
    is_prefill: bool = False
    seq_of_token: torch.Tensor | None = None   # [T] int32 (prefill); decode: token t belongs to sequence t
    q_start: torch.Tensor | None = None        # [S] int32 (prefill)
    q_len: torch.Tensor | None = None          # [S] int32 (prefill)
    max_q_len: int = 0                         # host int (prefill)
    logit_rows: torch.Tensor | None = None     # [S] int64 rows of the hidden state that produce logits (prefill)
    ctx_hint: int = 1024                       # host-side typical context length (chooses split-KV)


@dataclass
class SamplingInputs:
    """Per-row sampling parameters of a step (device tensors): rows with temperature <= 0 are greedy."""
    temperature: torch.Tensor          # [B] fp32
    top_k: torch.Tensor                # [B] int32 (0: the kernel's maximum of 64 candidates)
    top_p: torch.Tensor                # [B] fp32 in (0, 1]
    seeds: torch.Tensor                # [B] int64: one random stream per request
    step: torch.Tensor                 # [B] int32: counter of each row's random stream (the token's position)


class Decoder:
    """One rank's share of the model: weights, KV cache and the step function.

    The decoder takes ownership of `weights`: on a GPU the expert matrices are replaced in place by their tile-packed
    form (`ops.PackedWeight`: `.shape`, `.cpu()`, `.unpack()`, `.copy_()`), so that no second copy stays alive."""

    def __init__(self, cfg: ModelConfig, weights: ModelWeights, layout: ParallelLayout | None = None,
                 num_pages: int = 0, page_size: int = 16, max_pos: int | None = None, comm=None, comm_moe=None,
                 pack_moe: bool | None = None, kv_pools=None):
        # pack_moe: tile-pack the FFN / expert weights. kv_pools: per-layer page pools allocated by the caller
        # (peer-mapped pools of a prefill/decode pair, parallel/disagg.py) instead of pools allocated here
        self.cfg, self.w, self.layout = cfg, weights, layout or ParallelLayout()
        self.comm = comm          # tensor-parallel communicator over this rank's TP group, or None
        self.comm_moe = comm_moe  # communicator over all tp x ep ranks of the stage (expert parallelism), or None
        self._owner = None
        if self.layout.ep > 1 and comm_moe is None:
            raise ValueError("expert parallelism needs a communicator over the stage's tp x ep ranks (comm_moe)")
        self.sh = shard_shapes(cfg, self.layout)
        self.page_size = page_size
        dev = (weights.embed if weights.embed is not None else weights.layers[0].attn_norm).device
        self.device = dev
        self.max_pos = max_pos or cfg.max_position_embeddings
        self.cos_sin = ref.rope_cos_sin_table(self.max_pos, cfg.head_dim, cfg.rope_theta, dev)
        self.num_pages = num_pages
        if kv_pools is not None:
            want = (num_pages, 2, self.sh["Hkv"], page_size, cfg.head_dim)
            if len(kv_pools) != len(weights.layers) or any(tuple(p.shape) != want for p in kv_pools):
                raise ValueError(f"kv_pools must be {len(weights.layers)} tensors of shape {want}")
            self.kv = list(kv_pools)
        else:
            self.kv = [torch.zeros(num_pages, 2, self.sh["Hkv"], page_size, cfg.head_dim, dtype=torch.bfloat16, device=dev)
                       for _ in weights.layers] if num_pages > 0 else []
        self.capture_hidden = None  # set to a list to record the residual stream after every block (parity gate)
        # vocabulary-parallel embedding: when the table holds only this rank's rows (models/sharding.py, random_weights
        # with shard_embed), the first row it owns; None for a replicated table
        self.embed_vocab_start = None
        if (weights.embed is not None and comm is not None and comm.size > 1 and weights.embed.shape[0] != cfg.vocab_size):
            if weights.embed.shape[0] > self.sh["V_local"]:      # the last rank's shard may be short
                raise ValueError("the embedding table is neither whole nor this rank's vocabulary shard")
            self.embed_vocab_start = self.layout.tp_rank * self.sh["V_local"]
        if pack_moe is None:
            pack_moe = os.environ.get("SKEIN_PACK_MOE", "1") == "1"
        if pack_moe and dev.type == "cuda":
            # expert weights re-laid tile by tile (ops.pack_weight): each 128 x 64 tile the GEMM streams is one
            # contiguous 16 KB block instead of 128 rows that are a whole K apart. Measured in-graph on B200:
            # gate/up 80.4 -> 71.2 us at the TP=4 shard shape, 43.2 -> 40.4 us at TP=8, unchanged at TP=1 (HBM-bound)
            for lw in weights.layers:
                for name in ("w13", "w2"):
                    w = getattr(lw, name)
                    if not isinstance(w, torch.Tensor) or w.dim() not in (2, 3):
                        continue
                    rows, K = w.shape[-2], w.shape[-1]
                    half_ok = name != "w13" or (rows // 2) % 128 == 0     # the up half starts on a tile boundary
                    if rows % 128 == 0 and K % 64 == 0 and half_ok:
                        setattr(lw, name, ops.pack_weight(w))

    # ---- pieces ---------------------------------------------------------------------------------
    def _attention(self, li: int, normed, inp: BatchInputs):
        cfg, sh, lw = self.cfg, self.sh, self.w.layers[li]
        qkv = self._col_linear(normed, lw, "wqkv")
        if not inp.is_prefill and inp.seq_of_token is None and ops.can_fuse_rope(self.kv[li], sh["Hq"], sh["Hkv"]):
            # decode: RoPE and the cache append ride in the attention kernel
            return ops.attn_decode_rope(qkv, inp.positions, inp.block_table, self.cos_sin, self.kv[li], inp.seq_lens,
                                        sh["Hq"], sh["Hkv"], cfg.head_dim, ctx_hint=inp.ctx_hint)
        ops.rope_kv_append(qkv, inp.positions, inp.seq_of_token, inp.block_table, self.cos_sin, self.kv[li],
                           sh["Hq"], sh["Hkv"], cfg.head_dim)
        if inp.is_prefill:
            return ops.attn_prefill(qkv, self.kv[li], inp.block_table, inp.q_start, inp.q_len, inp.seq_lens,
                                    inp.max_q_len, sh["Hq"], sh["Hkv"], cfg.head_dim)
        return ops.attn_decode(qkv, self.kv[li], inp.block_table, inp.seq_lens, sh["Hq"], sh["Hkv"], cfg.head_dim,
                               ctx_hint=inp.ctx_hint)

    def _col_linear(self, x, lw, name, swiglu=False, grouped=None, rows_hint=None):
        """Column-parallel (local) projection through the block's bf16 weight or, when the plan's dtype map
        selected fp8 for this block, its block-scaled e4m3 copy (activations quantised on the fly)."""
        w8 = lw.fp8.get(name)
        if w8 is not None:
            # weights e4m3 with 1 x 128 block scales, activations bf16: the GEMM streams the e4m3 tiles and rescales them
            # to bf16 in shared memory (ops/fp8.py)
            if grouped is not None:
                return fp8.grouped_linear_a16(x, w8, *grouped, swiglu=swiglu, rows_hint=rows_hint)
            return fp8.linear_a16(x, w8, swiglu=swiglu)
        w = getattr(lw, name)
        if grouped is not None:
            return ops.grouped_linear(x, w, *grouped, swiglu=swiglu, rows_hint=rows_hint)
        return ops.swiglu_linear(x, w) if swiglu else ops.linear(x, w)

    def _row_parallel(self, x, lw, name, grouped=None):
        """Row-parallel projection. Returns (partial [n_src, rows, H], flags, epoch) for the fused reduce."""
        single = self.comm is None or self.comm.size == 1
        w8 = lw.fp8.get(name)
        if w8 is not None and single:
            return self._col_linear(x, lw, name, grouped=grouped).unsqueeze(0), None, None
        if w8 is not None and x.is_cuda and hasattr(self.comm, "linear_push_fp8"):
            return self.comm.linear_push_fp8(x, None, w8, grouped)
        w = getattr(lw, name)
        if w is None:
            w = w8.dequant()      # CPU ranks (reference operators): dequantise, then the bf16 path
        if single:
            y = ops.grouped_linear(x, w, *grouped) if grouped is not None else ops.linear(x, w)
            return y.unsqueeze(0), None, None
        return self.comm.linear_push(x, w, grouped)

    def _ffn(self, li: int, normed, routed=None):
        """Returns (partial, flags, epoch, row_idx, row_w) feeding the fused combine/reduce. `routed` carries the
        router's outputs and the expert-sorted activations when the preceding reduce kernel already made them."""
        cfg, lw = self.cfg, self.w.layers[li]
        if not cfg.is_moe:
            h = self._col_linear(normed, lw, "w13", swiglu=True)
            part, flags, epoch = self._row_parallel(h, lw, "w2")
            return part, flags, epoch, None, None
        T = normed.shape[0]
        e_local = self.sh["E_local"]
        first = self.layout.ep_rank * e_local
        if self.layout.ep > 1:
            # Expert parallel: every rank of the stage routes all tokens the same way (global expert-sorted
            # layout), computes only the rows of the experts it owns, and its down projection stores those rows
            # into every rank's receive slot; the combine then reads each (token, slot) pair from the ranks that
            # own its expert. Row positions are global, so no index exchange is needed.
            if routed is None:
                ids, wts, counts, offsets, row_of, src_token = ops.route(normed, lw.router, cfg.top_k)
                xs = ops.gather_rows(normed, src_token, n_rows_dev=offsets[cfg.num_experts:])
            else:
                ids, wts, counts, offsets, row_of, src_token, xs = routed
            cnt_l, off_l = counts[first:first + e_local], offsets[first:first + e_local]
            h = self._col_linear(xs, lw, "w13", swiglu=True, grouped=(cnt_l, off_l), rows_hint=T * cfg.top_k // self.layout.ep)
            w8 = lw.fp8.get("w2")
            if w8 is not None and h.is_cuda and hasattr(self.comm_moe, "linear_push_fp8"):
                part, flags, epoch = self.comm_moe.linear_push_fp8(h, None, w8, (cnt_l, off_l))
            else:
                w2 = lw.w2 if lw.w2 is not None else w8.dequant()
                part, flags, epoch = self.comm_moe.linear_push(h, w2, (cnt_l, off_l))
            self._owner = (ids, e_local, self.layout.tp)
            return part, flags, epoch, row_of.view(T, cfg.top_k), wts
        if routed is None:
            ids, wts, counts, offsets, row_of, src_token = ops.route(normed, lw.router, cfg.top_k, first, e_local)
            xs = ops.gather_rows(normed, src_token, n_rows_dev=offsets[cfg.num_experts:])
        else:
            ids, wts, counts, offsets, row_of, src_token, xs = routed
        cnt_l, off_l = counts[first:first + e_local], offsets[first:first + e_local]
        h = self._col_linear(xs, lw, "w13", swiglu=True, grouped=(cnt_l, off_l), rows_hint=T * cfg.top_k)
        part, flags, epoch = self._row_parallel(h, lw, "w2", (cnt_l, off_l))
        return part, flags, epoch, row_of.view(T, cfg.top_k), wts

    # ---- the step ---------------------------------------------------------------------------------
    def forward_hidden(self, inp: BatchInputs, hidden_in: torch.Tensor | None = None):
        """Runs this stage's blocks. Returns (residual stream [T, H], normed [T, H]) where `normed` is the final
        norm on the last stage and the next stage's first attn_norm input otherwise (None)."""
        cfg = self.cfg
        layers = self.w.layers
        if hidden_in is None and self.embed_vocab_start is not None:
            # table sharded by vocabulary rows: the ranks' lookups are summed inside the first RMSNorm
            residual, normed = self.comm.embed_reduce(inp.token_ids, self.w.embed, self.embed_vocab_start,
                                                      layers[0].attn_norm, cfg.rms_norm_eps)
        else:
            residual = ops.embed(inp.token_ids, self.w.embed) if hidden_in is None else hidden_in
            normed = ops.rmsnorm(residual, layers[0].attn_norm, cfg.rms_norm_eps)
        last_stage = self.w.final_norm is not None
        T = residual.shape[0]
        if (inp.is_prefill and self.comm is not None and self.comm.size > 1 and self.layout.ep == 1 and residual.is_cuda
                and hasattr(self.comm, "sp_ok") and self.comm.sp_ok(T, T * max(1, cfg.top_k if cfg.is_moe else 1))):
            return self._forward_hidden_sp(inp, residual, normed, last_stage)
        for li, lw in enumerate(layers):
            attn = self._attention(li, normed, inp)
            part, flags, epoch = self._row_parallel(attn, lw, "wo")
            routed = None
            if cfg.is_moe and residual.is_cuda and ops.can_fuse_route(residual.shape[0], cfg.top_k, residual.device):
                # decode-sized batches: the router and the expert-sorted scatter ride in the reduce kernel
                ep = self.layout.ep > 1
                e_first = 0 if ep else self.layout.ep_rank * self.sh["E_local"]
                e_cnt = cfg.num_experts if ep else self.sh["E_local"]
                out = ops.reduce_norm_route(residual, part, lw.ffn_norm, cfg.rms_norm_eps, lw.router, cfg.top_k,
                                            e_first, e_cnt, flags=flags, epoch=epoch)
                residual, normed, routed = out[0], out[1], out[2:]
            else:
                residual, normed = ops.reduce_residual_rmsnorm(residual, part, lw.ffn_norm, cfg.rms_norm_eps,
                                                               flags=flags, epoch=epoch)
            self._owner = None
            part, flags, epoch, row_idx, row_w = self._ffn(li, normed, routed)
            if li + 1 < len(layers):
                next_gamma = layers[li + 1].attn_norm
            else:
                next_gamma = self.w.final_norm if last_stage else None
            own = {} if self._owner is None else dict(owner_ids=self._owner[0], experts_per_owner=self._owner[1],
                                                      owner_span=self._owner[2])
            residual, normed = ops.reduce_residual_rmsnorm(residual, part, next_gamma, cfg.rms_norm_eps, row_idx,
                                                           row_w, flags=flags, epoch=epoch, **own)
            if self.capture_hidden is not None:
                self.capture_hidden.append(residual.detach().float().cpu())
        return residual, normed

    def _forward_hidden_sp(self, inp: BatchInputs, residual, normed, last_stage: bool):
        """Prefill-sized chunks under tensor parallelism: sequence-parallel between the projections. The row-parallel
        GEMMs (o_proj, down) publish their partials; every rank reduces, adds the residual and normalises only its
        own slice of the token rows (reduce-scatter fused with residual + RMSNorm, peer loads or the in-switch
        reduction), the residual stream stays sharded by rows from layer to layer, and the normalised slices are
        gathered into local memory for the next column-parallel GEMM (parallel/tp.py). No library collective runs.
        The reference keeps activations replicated and all-reduces twice per block through NCCL
        (crates/skein_emit/src/handoff.rs:104-211, crates/skein_runtime/src/cuda/nccl.rs:196-245)."""
        cfg, comm, layers = self.cfg, self.comm, self.w.layers
        T = residual.shape[0]
        r0, n, _ = comm.sp_slice(T)
        res_loc = residual[r0:r0 + n].contiguous()
        for li, lw in enumerate(layers):
            attn = self._attention(li, normed, inp)
            part, _, _ = self._row_parallel(attn, lw, "wo")
            res_loc, normed_loc = comm.reduce_scatter_norm(res_loc, part, lw.ffn_norm, cfg.rms_norm_eps, T)
            normed = comm.gather_rows(normed_loc, T)
            part, _, _, row_idx, row_w = self._ffn(li, normed, None)
            if li + 1 < len(layers):
                next_gamma = layers[li + 1].attn_norm
            else:
                next_gamma = self.w.final_norm if last_stage else None
            res_loc, normed_loc = comm.reduce_scatter_norm(res_loc, part, next_gamma, cfg.rms_norm_eps, T, row_idx, row_w)
            normed = comm.gather_rows(normed_loc, T) if next_gamma is not None else None
            if self.capture_hidden is not None:
                self.capture_hidden.append(self._gather_residual(res_loc, T).float().cpu())
        residual = self._gather_residual(res_loc, T) if not last_stage else None
        return residual, normed

    def _gather_residual(self, res_loc, T):
        """The full residual stream from its row slices (only where a whole copy is needed: the hand-off to the next
        pipeline stage, the parity gate's per-layer capture)."""
        _, n, per = self.comm.sp_slice(T)
        pad = torch.zeros(per, res_loc.shape[1], dtype=res_loc.dtype, device=res_loc.device)
        pad[:n] = res_loc
        return self.comm.gather_rows(pad, T)

    def logits(self, normed, inp: BatchInputs):
        """Logits of this rank's vocabulary shard for the rows that need them."""
        if inp.is_prefill and inp.logit_rows is not None:
            normed = normed.index_select(0, inp.logit_rows).contiguous()
        return ops.linear(normed, self.w.lm_head)

    def forward(self, inp: BatchInputs, hidden_in=None, sampling: SamplingInputs | None = None):
        """Full step on a single stage: returns (next tokens int32 [rows], logits shard). Greedy unless `sampling`
        is given."""
        _, normed = self.forward_hidden(inp, hidden_in)
        lg = self.logits(normed, inp)
        return self.sample(lg, sampling), lg

    def sample(self, lg, sampling: SamplingInputs | None = None):
        """Next token of every row from this rank's logit shard. Greedy: vocabulary-parallel arg-max (8 bytes per row
        cross NVLink). Sampling: the shards are gathered (every rank then draws the same token from the same
        per-request random stream), as the reference gathers logits before its sampler
        (crates/skein_runtime/src/cuda/nccl.rs:251-298)."""
        tp = self.comm is not None and self.comm.size > 1
        if sampling is None:
            return self.comm.vocab_parallel_argmax(lg, self.sh["V_local"]) if tp else ops.sample_argmax(lg)
        if tp:
            rows, vl = lg.shape
            full = self.comm.all_gather(lg.contiguous()).view(self.comm.size, rows, vl).permute(1, 0, 2).reshape(rows, -1)
            lg = full[:, :self.cfg.vocab_size].contiguous()
        n = lg.shape[0]
        return ops.sample(lg, sampling.temperature[:n], sampling.top_k[:n], sampling.top_p[:n], sampling.seeds[:n],
                          sampling.step[:n])
