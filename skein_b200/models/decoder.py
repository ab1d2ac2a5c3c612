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
    bqkv: torch.Tensor | None = None   # [(Hq + 2 Hkv) / tp * D] bias of the fused q / k / v projection (Qwen2), else None


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
            wo=rnd(H, sh["Hq"] * D), ffn_norm=torch.ones(H, dtype=dtype, device=device), router=router, w13=w13, w2=w2,
            bqkv=rnd((sh["Hq"] + 2 * sh["Hkv"]) * D) if cfg.qkv_bias else None))
    first, last = lay.pp_rank == 0, lay.pp_rank == lay.pp - 1
    embed = rnd(sh["V_local"] if (shard_embed and lay.tp > 1) else cfg.vocab_size, H) if first else None
    if cfg.tie_word_embeddings and first and last:      # the output projection is (this rank's rows of) the embedding table
        v0 = 0 if embed.shape[0] == sh["V_local"] else lay.tp_rank * sh["V_local"]
        lm_head = embed[v0:v0 + sh["V_local"]]
    else:
        lm_head = rnd(sh["V_local"], H) if last else None
    return ModelWeights(embed=embed, layers=layers, final_norm=torch.ones(H, dtype=dtype, device=device) if last else None,
                        lm_head=lm_head)


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
        if self.layout.ep > 1 and comm_moe is None:
            raise ValueError("expert parallelism needs a communicator over the stage's tp x ep ranks (comm_moe)")
        self.sh = shard_shapes(cfg, self.layout)
        self.page_size = page_size
        dev = (weights.embed if weights.embed is not None else weights.layers[0].attn_norm).device
        self.device = dev
        if dev.type == "cuda" and cfg.head_dim != 128:
            # say so when the model is set up, not in the middle of the first request
            raise ValueError(f"the attention kernels are built for head size 128; this model has {cfg.head_dim}")
        self.max_pos = max_pos or cfg.max_position_embeddings
        self.cos_sin = ref.rope_cos_sin_table(self.max_pos, cfg.head_dim, cfg.rope_theta, dev, cfg.rope_scaling)
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
        # Expert parallelism with data-parallel attention (decode): every expert-parallel rank runs attention, norms and
        # the router for its own slice of the step's rows and the MoE blocks exchange tokens (dispatch) and expert outputs
        # (combine) over peer memory. The caller must keep a sequence on the same slice for its whole life, because only
        # that rank's cache receives the sequence's new tokens (runtime/engine.py does; a benchmark's rows are static).
        self.dp_attention = False
        # Set by a caller that pins sequences to ranks (the engine): a decode step that does not fit the data-parallel
        # path then raises instead of falling back to attention over all rows, which would read cache pages this rank
        # never wrote.
        self.dp_strict = False
        self.program = self._load_program()
        self._ops = {name[4:]: getattr(self, name) for name in dir(self) if name.startswith("_op_")}
        missing = sorted({it[1] for it in self.program if it[0] == "op"} - set(self._ops))
        if missing:
            raise RuntimeError(f"the lowering names operators this runtime does not implement: {missing}")
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

    # ---- the lowered program ------------------------------------------------------------------------
    def _load_program(self):
        """This rank's schedule from the lowering (csrc/core/emit.hpp: lower_device): the named operators of every
        segment and the collectives between the segments, in order. It is what forward_hidden executes, so where a
        collective sits is decided in one place, the lowering, and the artifact's segments.json describes exactly what
        runs (compile/artifact.py: check_lowering compares the two)."""
        import json

        from .. import core
        lay = self.layout
        low = json.loads(core.lower_device_for(json.dumps(self.cfg.to_hf_dict()), lay.tp, lay.pp, lay.ep, lay.rank))
        first_block = lay.stage_layers(self.cfg.num_layers)[0] if len(lay.stage_layers(self.cfg.num_layers)) else 0
        segs = {s_["idx"]: s_["ops"] for s_ in low["segments"]}
        prog = []
        for st in low["sequencing"]:
            if st["kind"] == "execute_segment":
                for name in segs[st["segment"]]:
                    if name.startswith("block_"):
                        _, b, op = name.split("_", 2)
                        prog.append(("op", op, int(b) - first_block))
                    else:
                        prog.append(("op", name, -1))
            elif st["kind"] == "collective":
                prog.append(("collective", st["collective"], st["tensor"]))
        return prog

    class _Run:
        """State of one pass over the program."""
        __slots__ = ("inp", "residual", "normed", "qkv", "attn", "pending", "pending_kind", "routed", "h", "sp", "T",
                     "crossing", "embed_deferred", "row_idx", "row_w", "owner", "dp", "wts")

        def __init__(self, inp, residual):
            self.inp, self.residual = inp, residual
            self.normed = self.qkv = self.attn = self.pending = self.routed = self.h = None
            self.pending_kind, self.crossing, self.sp, self.T = None, None, False, 0
            self.embed_deferred = False
            self.row_idx = self.row_w = self.owner = self.wts = None
            self.dp = 0          # rows per rank under data-parallel attention (0: every rank holds all rows)

    def dp_ways(self) -> int:
        """Expert-parallel ranks that share a decode step's rows among them for attention (1: every rank holds all rows)."""
        lay = self.layout
        return lay.ep if (self.dp_attention and lay.ep > 1 and lay.tp == 1 and lay.pp == 1 and self.cfg.is_moe) else 1

    def dp_rows_ok(self, B: int, device=None) -> bool:
        """True when a decode step of B rows can run with data-parallel attention on this layout."""
        ways, k = self.dp_ways(), self.cfg.top_k
        if ways == 1 or B % ways:
            return False
        per = B // ways
        # the sampled tokens of a slice are gathered 16 bytes at a time; the fused reduce + router needs one CTA per row
        fits = getattr(self.comm_moe, "dispatch_fits", None)      # CPU rank communicators carry no dispatch buffers
        return (per % 4 == 0 and ops.can_fuse_route(per, k, device) and B * k <= 2048 and (fits is None or fits(per, k)))

    def dp_rows_limit(self, device=None) -> int:
        """Largest power-of-two number of rows per rank that dp_rows_ok accepts (0: none does)."""
        best, per = 0, 4
        while per <= 1024 and self.dp_rows_ok(per * self.dp_ways(), device):
            best, per = per, per * 2
        return best

    def _dp_rows(self, inp: BatchInputs) -> int:
        """Rows per rank when this step runs with data-parallel attention, else 0."""
        if self.dp_ways() == 1 or inp.is_prefill or inp.seq_of_token is not None or not inp.token_ids.is_cuda:
            return 0
        B = inp.token_ids.shape[0]
        if not self.dp_rows_ok(B, inp.token_ids.device):
            if self.dp_strict:
                raise RuntimeError(f"a decode step of {B} rows cannot run with data-parallel attention over {self.dp_ways()} "
                                   "ranks, and its sequences' new tokens are cached on their own rank only")
            return 0
        return B // self.dp_ways()

    @property
    def _multi(self) -> bool:
        return (self.comm is not None and self.comm.size > 1) or (self.comm_moe is not None and self.comm_moe.size > 1)

    # ---- operators of the program (one method per operator name of the lowering) -----------------------
    def _op_embed_tokens(self, st, _):
        if self.embed_vocab_start is not None:
            st.embed_deferred = True       # the ranks' lookups are summed where the lowering puts the embed_out all-reduce
        else:
            st.residual = ops.embed(st.inp.token_ids, self.w.embed)

    def _op_input_layernorm(self, st, li):
        gamma = self.w.layers[li].attn_norm
        if st.pending is not None:
            self._reduce(st, gamma)
        elif st.normed is None:
            st.normed = ops.rmsnorm(st.residual, gamma, self.cfg.rms_norm_eps)
        if li == 0:
            self._maybe_shard_rows(st)

    def _maybe_shard_rows(self, st):
        """Prefill-sized chunks under tensor parallelism take the sequence-parallel dataflow: from here on the residual
        stream is this rank's slice of the token rows (see _reduce)."""
        cfg, comm = self.cfg, self.comm
        st.T = T = st.residual.shape[0]
        if (st.inp.is_prefill and comm is not None and comm.size > 1 and self.layout.ep == 1 and st.residual.is_cuda
                and hasattr(comm, "sp_ok") and comm.sp_ok(T, T * max(1, cfg.top_k if cfg.is_moe else 1))):
            r0, n, _ = comm.sp_slice(T)
            st.residual = st.residual[r0:r0 + n].contiguous()
            st.sp = True

    def _op_qkv_proj(self, st, li):
        lw = self.w.layers[li]
        st.qkv = self._col_linear(st.normed, lw, "wqkv")
        if lw.bqkv is not None:
            st.qkv += lw.bqkv       # Qwen2: one elementwise pass over [tokens, (Hq + 2 Hkv) D]; the GEMM epilogue carries no bias

    def _rope_fused(self, st, li) -> bool:
        inp = st.inp
        return (not inp.is_prefill and inp.seq_of_token is None
                and ops.can_fuse_rope(self.kv[li], self.sh["Hq"], self.sh["Hkv"]))

    def _op_rope_kv_append(self, st, li):
        if self._rope_fused(st, li):
            return          # decode: RoPE and the cache append ride in the attention kernel
        inp, sh = st.inp, self.sh
        ops.rope_kv_append(st.qkv, inp.positions, inp.seq_of_token, inp.block_table, self.cos_sin, self.kv[li],
                           sh["Hq"], sh["Hkv"], self.cfg.head_dim)

    def _op_attention(self, st, li):
        inp, sh, D = st.inp, self.sh, self.cfg.head_dim
        if self._rope_fused(st, li):
            st.attn = ops.attn_decode_rope(st.qkv, inp.positions, inp.block_table, self.cos_sin, self.kv[li], inp.seq_lens,
                                           sh["Hq"], sh["Hkv"], D, ctx_hint=inp.ctx_hint)
        elif inp.is_prefill:
            st.attn = ops.attn_prefill(st.qkv, self.kv[li], inp.block_table, inp.q_start, inp.q_len, inp.seq_lens,
                                       inp.max_q_len, sh["Hq"], sh["Hkv"], D)
        else:
            st.attn = ops.attn_decode(st.qkv, self.kv[li], inp.block_table, inp.seq_lens, sh["Hq"], sh["Hkv"], D,
                                      ctx_hint=inp.ctx_hint)

    def _op_o_proj(self, st, li):
        st.pending = self._row_parallel(st.attn, self.w.layers[li], "wo")
        st.pending_kind, st.row_idx, st.row_w, st.owner, st.crossing = "attn", None, None, None, None

    def _op_post_attention_layernorm(self, st, li):
        cfg, lw = self.cfg, self.w.layers[li]
        residual = st.residual
        if st.dp:
            # this rank's rows only: residual + RMSNorm + router in one launch, with the normalised rows and the expert
            # choices written straight into the published buffer; one pull kernel then gathers the rows of this rank's
            # experts from all ranks (parallel/tp.py: ep_dispatch, csrc/kernels/ep_dispatch.cu)
            part, flags, epoch = st.pending
            e_local = self.sh["E_local"]
            box = {}

            def fill(normed_view, ids_view):
                out = ops.reduce_norm_route(residual, part, lw.ffn_norm, cfg.rms_norm_eps, lw.router, cfg.top_k, 0, cfg.num_experts,
                                            flags=flags, epoch=epoch, normed_out=normed_view, ids_out=ids_view, scatter=False)
                box["res"], box["wts"] = out[0], out[3]
            ids_all, counts, offsets, row_of, src_token, xs = self.comm_moe.ep_dispatch(
                st.dp, cfg.top_k, cfg.num_experts, self.layout.ep_rank * e_local, e_local, fill)
            st.residual, st.wts = box["res"], box["wts"]
            st.normed = None        # lives in the published buffer; the experts read xs
            st.routed = (ids_all, None, counts, offsets, row_of, src_token, xs)
            st.pending = None
            return
        if (cfg.is_moe and not st.sp and residual.is_cuda and ops.can_fuse_route(residual.shape[0], cfg.top_k, residual.device)):
            # decode-sized batches: the router and the expert-sorted scatter ride in the reduce kernel
            self._check_crossing(st)
            ep = self.layout.ep > 1
            e_first = 0 if ep else self.layout.ep_rank * self.sh["E_local"]
            e_cnt = cfg.num_experts if ep else self.sh["E_local"]
            part, flags, epoch = st.pending
            out = ops.reduce_norm_route(residual, part, lw.ffn_norm, cfg.rms_norm_eps, lw.router, cfg.top_k,
                                        e_first, e_cnt, flags=flags, epoch=epoch)
            st.residual, st.normed, st.routed = out[0], out[1], out[2:]
            st.pending = None
        else:
            self._reduce(st, lw.ffn_norm)
            st.routed = None

    def _op_router(self, st, li):
        if st.routed is not None:
            return          # produced by the fused reduce + router kernel
        cfg, lw = self.cfg, self.w.layers[li]
        e_local = self.sh["E_local"]
        if self.layout.ep > 1:
            # every rank of the stage routes all tokens the same way (global expert-sorted layout)
            ids, wts, counts, offsets, row_of, src_token = ops.route(st.normed, lw.router, cfg.top_k)
        else:
            ids, wts, counts, offsets, row_of, src_token = ops.route(st.normed, lw.router, cfg.top_k,
                                                                     self.layout.ep_rank * e_local, e_local)
        xs = ops.gather_rows(st.normed, src_token, n_rows_dev=offsets[cfg.num_experts:])
        st.routed = (ids, wts, counts, offsets, row_of, src_token, xs)

    def _op_experts_gate_up(self, st, li):
        cfg, lw = self.cfg, self.w.layers[li]
        T = st.dp * self.layout.ep if st.dp else st.normed.shape[0]
        e_local = self.sh["E_local"]
        first = self.layout.ep_rank * e_local
        ids, wts, counts, offsets, row_of, src_token, xs = st.routed
        cnt_l, off_l = counts[first:first + e_local], offsets[first:first + e_local]
        st.h = (self._col_linear(xs, lw, "w13", swiglu=True, grouped=(cnt_l, off_l), rows_hint=T * cfg.top_k // self.layout.ep),
                cnt_l, off_l)

    def _op_experts_down(self, st, li):
        cfg, lw = self.cfg, self.w.layers[li]
        T = st.dp * self.layout.ep if st.dp else st.normed.shape[0]
        ids, wts, counts, offsets, row_of, src_token, xs = st.routed
        h, cnt_l, off_l = st.h
        if self.layout.ep > 1:
            # Expert parallel: a rank computes only the rows of the experts it owns and its down projection publishes them;
            # the combine then reads each (token, slot) pair from the ranks that own its expert. Row positions are global,
            # so no index exchange is needed.
            w8 = lw.fp8.get("w2")
            if w8 is not None and self._expand_fp8(h, w8, (cnt_l, off_l), rows_hint=T * cfg.top_k // self.layout.ep):
                st.pending = self.comm_moe.linear_push(h, w8.dequant(), (cnt_l, off_l))
            elif w8 is not None and h.is_cuda and hasattr(self.comm_moe, "linear_push_fp8"):
                st.pending = self.comm_moe.linear_push_fp8(h, None, w8, (cnt_l, off_l))
            else:
                w2 = lw.w2 if lw.w2 is not None else w8.dequant()
                st.pending = self.comm_moe.linear_push(h, w2, (cnt_l, off_l))
            # the owner-aware pull only applies to published partials; a chunk too large for the published buffers came back
            # from the library all-reduce as one complete tensor
            st.owner = (ids, self.sh["E_local"], self.layout.tp) if hasattr(st.pending[0], "ptrs") else None
        else:
            st.pending = self._row_parallel(h, lw, "w2", (cnt_l, off_l))
            st.owner = None
        st.pending_kind, st.row_idx, st.row_w, st.crossing = "ffn", row_of.view(T, cfg.top_k), wts, None
        if st.dp:
            # the combine of this rank's own rows: their pairs' global row positions, weights and expert ids
            lo, hi = self.layout.ep_rank * st.dp, (self.layout.ep_rank + 1) * st.dp
            st.row_idx, st.row_w = st.row_idx[lo:hi].contiguous(), st.wts
            st.owner = (ids[lo:hi].contiguous(), self.sh["E_local"], self.layout.tp) if st.owner is not None else None
        st.h = st.routed = None

    def _op_gate_up_proj(self, st, li):
        st.h = self._col_linear(st.normed, self.w.layers[li], "w13", swiglu=True)

    def _op_down_proj(self, st, li):
        st.pending = self._row_parallel(st.h, self.w.layers[li], "w2")
        st.pending_kind, st.row_idx, st.row_w, st.owner, st.crossing, st.h = "ffn", None, None, None, None, None

    def _op_norm(self, st, _):
        self._reduce(st, self.w.final_norm)

    def _op_lm_head(self, st, _):     # logits() and sample() run these on the rows that need them
        pass

    _op_sample = _op_lm_head

    def _collective(self, st, kind, tensor):
        if tensor == "embed_out":
            if st.embed_deferred:
                st.residual, st.normed = self.comm.embed_reduce(st.inp.token_ids, self.w.embed, self.embed_vocab_start,
                                                                self.w.layers[0].attn_norm, self.cfg.rms_norm_eps)
                st.embed_deferred = False
        elif kind in ("ring_allreduce", "alltoall"):
            # the exchange itself is carried by the kernels on both sides of this point (publish epilogue of the producing
            # GEMM, pull inside the consuming reduce): record that the lowering put one here
            st.crossing = tensor
        # send_recv between pipeline stages is issued by parallel/pp.py around this stage's program; the sampler's
        # candidate exchange belongs to sample()

    def _check_crossing(self, st):
        if self._multi and st.pending is not None and hasattr(st.pending[0], "ptrs") and st.crossing is None:
            raise RuntimeError("partial results of other ranks are about to be summed, but the lowering placed no collective here")

    def _reduce(self, st, gamma):
        """residual += sum over ranks of the pending partial (dense, or the weighted top-k combine of expert rows), then
        RMSNorm with `gamma` (None: no normalised output). Sequence-parallel form: only this rank's row slice, followed
        by the all-gather of the normalised slices (parallel/tp.py)."""
        cfg = self.cfg
        self._check_crossing(st)
        part, flags, epoch = st.pending
        kind = st.pending_kind
        if st.sp:
            st.residual, normed_loc = self.comm.reduce_scatter_norm(st.residual, part, gamma, cfg.rms_norm_eps, st.T,
                                                                    st.row_idx, st.row_w)
            st.normed = self.comm.gather_rows(normed_loc, st.T) if gamma is not None else None
        else:
            own = {} if st.owner is None else dict(owner_ids=st.owner[0], experts_per_owner=st.owner[1], owner_span=st.owner[2])
            st.residual, st.normed = ops.reduce_residual_rmsnorm(st.residual, part, gamma, cfg.rms_norm_eps, st.row_idx, st.row_w,
                                                                 flags=flags, epoch=epoch, **own)
        st.pending = st.row_idx = st.row_w = st.owner = None
        if kind == "ffn" and self.capture_hidden is not None:
            full = self._gather_residual(st.residual, st.T) if st.sp else st.residual
            self.capture_hidden.append(full.detach().float().cpu())

    def _col_linear(self, x, lw, name, swiglu=False, grouped=None, rows_hint=None):
        """Column-parallel (local) projection through the block's bf16 weight or, when the plan's dtype map
        selected fp8 for this block, its block-scaled e4m3 copy."""
        w8 = lw.fp8.get(name)
        w = getattr(lw, name)
        if w8 is not None and self._expand_fp8(x, w8, grouped, rows_hint):
            w, w8 = w8.dequant(), None
        if w8 is not None:
            # weights e4m3 with 1 x 128 block scales, activations bf16: the GEMM streams the e4m3 tiles and rescales them
            # to bf16 on their way to the tensor cores (ops/fp8.py)
            if grouped is not None:
                return fp8.grouped_linear_a16(x, w8, *grouped, swiglu=swiglu, rows_hint=rows_hint)
            return fp8.linear_a16(x, w8, swiglu=swiglu)
        if grouped is not None:
            return ops.grouped_linear(x, w, *grouped, swiglu=swiglu, rows_hint=rows_hint)
        return ops.swiglu_linear(x, w) if swiglu else ops.linear(x, w)

    def _expand_fp8(self, x, w8, grouped=None, rows_hint=None) -> bool:
        """Whether an e4m3 weight is expanded to a transient bf16 matrix for this call. The weight-fp8 GEMM rescales a
        weight tile once per token tile that uses it, which is free while a step is a few token tiles wide (decode) and
        dominates at prefill size; there one expansion pass (csrc/kernels/quant.cu) plus the bf16 GEMM is faster."""
        if not x.is_cuda or getattr(self, "fp8_expand_rows", 256) <= 0:
            return False
        groups = w8.shape[0] if (grouped is not None and len(w8.shape) == 3) else 1
        rows = rows_hint if rows_hint is not None else x.shape[0]
        return rows / groups > getattr(self, "fp8_expand_rows", 256)

    def _row_parallel(self, x, lw, name, grouped=None):
        """Row-parallel projection. Returns (partial [n_src, rows, H], flags, epoch) for the fused reduce."""
        single = self.comm is None or self.comm.size == 1
        w8 = lw.fp8.get(name)
        if w8 is not None and self._expand_fp8(x, w8, grouped):
            w = w8.dequant()
            if single:
                y = ops.grouped_linear(x, w, *grouped) if grouped is not None else ops.linear(x, w)
                return y.unsqueeze(0), None, None
            return self.comm.linear_push(x, w, grouped)
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

    # ---- the step ---------------------------------------------------------------------------------
    def forward_hidden(self, inp: BatchInputs, hidden_in: torch.Tensor | None = None):
        """Runs this stage's part of the lowered program. Returns (residual stream [T, H], normed [T, H]) where `normed`
        is the final norm on the last stage and None otherwise.

        Under tensor parallelism the two row-parallel projections of a block (o_proj, down) publish their partial
        results from the GEMM epilogue and the reduce that follows pulls the peers' partials, so a block launches no
        stand-alone collective; prefill-sized chunks run sequence-parallel between the projections (reduce-scatter fused
        with residual + RMSNorm on this rank's rows, all-gather of the normalised rows, no library collective).
        The reference keeps activations replicated and all-reduces twice per block through NCCL
        (crates/skein_emit/src/handoff.rs:104-211, crates/skein_runtime/src/cuda/nccl.rs:196-245)."""
        st = Decoder._Run(inp, hidden_in)
        if hidden_in is not None:
            st.T = hidden_in.shape[0]
        st.dp = self._dp_rows(inp)
        if st.dp:
            r, per = self.layout.ep_rank, st.dp
            st.inp = BatchInputs(token_ids=inp.token_ids[r * per:(r + 1) * per], positions=inp.positions[r * per:(r + 1) * per],
                                 block_table=inp.block_table[r * per:(r + 1) * per], seq_lens=inp.seq_lens[r * per:(r + 1) * per],
                                 ctx_hint=inp.ctx_hint)
        for item in self.program:
            if item[0] == "op":
                self._ops[item[1]](st, item[2])
            else:
                self._collective(st, item[1], item[2])
        last_stage = self.w.final_norm is not None
        if st.pending is not None:        # a stage that is not the last: its final partial goes into the residual stream
            if st.crossing is None and self._multi and self.layout.tp > 1:
                st.crossing = "carry"     # the hand-off to the next stage follows; the lowering cut the segment there
            self._reduce(st, None)
        residual = st.residual
        if st.sp:
            residual = self._gather_residual(residual, st.T) if not last_stage else None
        return residual, (st.normed if last_stage else None)

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
        out = self._forward(inp, hidden_in, sampling)
        for c in (self.comm, self.comm_moe):
            if c is not None and hasattr(c, "even_out"):
                c.even_out()
        return out

    def _forward(self, inp: BatchInputs, hidden_in=None, sampling: SamplingInputs | None = None):
        _, normed = self.forward_hidden(inp, hidden_in)
        per = self._dp_rows(inp) if hidden_in is None else 0
        if per:
            # data-parallel attention: this rank holds the final hidden state of its own rows; every rank samples its
            # slice and the tokens are gathered through the small published buffer
            r = self.layout.ep_rank
            lg = ops.linear(normed, self.w.lm_head)
            smp = None
            if sampling is not None:
                smp = SamplingInputs(sampling.temperature[r * per:(r + 1) * per], sampling.top_k[r * per:(r + 1) * per],
                                     sampling.top_p[r * per:(r + 1) * per], sampling.seeds[r * per:(r + 1) * per],
                                     sampling.step[r * per:(r + 1) * per])
            tok = ops.sample_argmax(lg) if smp is None else ops.sample(lg, smp.temperature, smp.top_k, smp.top_p, smp.seeds, smp.step)
            return self.comm_moe.all_gather_aux(tok), lg
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
