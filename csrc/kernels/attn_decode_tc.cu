// Paged-KV decode attention on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory, K / V page
// tiles staged by TMA). Same operator and cache layout as attn_decode_mma.cu, RoPE of q / k and the KV append of the new
// token included; this kernel takes the launches with one split, head size 128, 16-token pages and at most 8 query
// heads per kv head, the mma.sync kernel keeps the rest (split-KV, other page sizes).
//
// One query token per sequence leaves the usual "queries on M" tile almost empty, so the tile is turned around, the same
// swap the weight-streaming GEMM makes: the 128 TOKENS of a context tile sit on the 128-row M side and the G query heads
// that share the kv head on N = 16.
//
//   S^T = K Q^T     A = K tile [128 tokens][128] (K-major, as TMA lays the pages down), B = Q^T [16 heads][128] (shared
//                   memory, written once by the compute warps, RoPE applied), accumulator 128 lanes x 16 columns
//   softmax         over tokens = across tensor-memory lanes: the scores go through a [heads][128] staging array in shared
//                   memory, each warp then owns whole heads (row max, exp2, row sum with five shuffles) and writes P^T
//                   [16 heads][128 tokens] (bf16, 128-byte swizzle) as the next B operand
//   O^T += V^T P    A = V tile read as an MN-major operand (M = head dimension, the reduction runs over the tokens,
//                   which is how the cache stores V), accumulator 128 lanes (d) x 16 columns (heads)
//
// One CTA per (sequence, kv head): warp 0 streams the K and V tiles of the context through a ring of 32 KB slots (three
// slots and two CTAs per SM when the launch has more CTAs than SMs, six slots and one CTA per SM otherwise: 192 KB of
// cache in flight per SM either way), warp 1 issues the MMAs (the next tile's scores go into a second S^T buffer ahead of
// the softmax whenever its K tile has already landed), warps 2-5 do the rest. With RoPE fused, the new
// token's rotated K row and its V row are stored to the cache AND patched into the last tile in shared memory after TMA
// has landed it, so the kernel never reads back through TMA what it has just written with ordinary stores.
// Every wait is bounded; on expiry the CTA records a status code, waits (bounded) for its copies in flight, frees its
// tensor memory and returns.
//
// Reference: fused_decode_attn (vendor/luminal/crates/luminal_cuda_lite/src/kernel/decode_attention.rs:66-139) and the
// FlashInfer batch-decode wrapper (vendor/luminal/crates/luminal_cuda_lite/src/host/flashinfer/wrapper.cu:123-251).
#include "ptx.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes, uint32_t box_rows);

constexpr int DT_BN = 128, DT_D = 128, DT_PS = 16, DT_GP = 8;   // tokens per tile, head size, page size, heads handled
constexpr int DT_THREADS = 192;
constexpr int DT_HALF = 128 * 128;                 // bytes of one 64-element half of a 128-row tile (128-byte rows)
constexpr int DT_TILE = 2 * DT_HALF;               // 32 KB: one K or V tile
constexpr int DT_QP_HALF = 16 * 128;               // bytes of one half of a 16-row B operand tile
// Shared-memory layout for a ring of SLOTS K / V tiles. Three slots (110 KB) let two CTAs share an SM, which is what a
// launch with more CTAs than SMs wants; a launch with at most one CTA per SM takes six slots (three context tiles in
// flight), because there a CTA's own copies in flight are all that hides the memory latency.
template <int SLOTS>
struct DtLayout {
  static constexpr int OFF_Q = SLOTS * DT_TILE;                 // Q^T: two halves
  static constexpr int OFF_P = OFF_Q + 2 * DT_QP_HALF;
  static constexpr int OFF_ST = OFF_P + 2 * DT_QP_HALF;         // fp32 scores [DT_GP][128]
  static constexpr int OFF_NEW = OFF_ST + DT_GP * DT_BN * 4;    // rotated k row, v row of the new token (2 x 256 bytes)
  static constexpr int OFF_STATS = OFF_NEW + 512;               // m[8], l[8], alpha[8] fp32
  static constexpr int OFF_BARS = OFF_STATS + 128;              // mbarriers, tensor-memory slot, abort flags
  static constexpr int SMEM = OFF_BARS + 192 + 1024 /* alignment slack */;
};
constexpr int DT_TMEM_COLS = 64;     // two S^T buffers of 16 columns, O^T at 32
constexpr uint64_t DT_BUDGET_NS = 4000000000ull;

struct AttnDecodeTcParams {
  const __nv_bfloat16* q;   // [B, q_stride]: head h at h * 128 (with RoPE fused: the raw q / k / v projection rows)
  __nv_bfloat16* kv_rw;     // the paged cache, writable (append of the new token)
  const int* block_table;   // [B, max_blocks]
  const int* seq_lens;      // [B] context length including the new token; 0 = padding row
  __nv_bfloat16* out;       // [B, Hq * 128]
  int* status;
  long long q_stride;
  int Hq, Hkv, G, max_blocks, num_pages;
  float scale_log2e;
  const float* cos_sin;     // [max_pos, 64, 2] fp32, or null: q is rotated and the cache holds the token already
  const int* positions;     // [B] position of the new token, -1 = padding row
  int max_pos;
};

__device__ __forceinline__ uint64_t dt_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {   // MN-major, 128-byte swizzle
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ void dt_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void dt_bar_compute() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// byte offset of element (row, d) in a 128-row tile of two 64-element halves with the 128-byte swizzle
__device__ __forceinline__ uint32_t dt_tile_off(int row, int d) {
  return (uint32_t)((d >> 6) * DT_HALF + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4) + (d & 7) * 2);
}

template <int DT_SLOTS>
__global__ void __launch_bounds__(DT_THREADS, DT_SLOTS == 3 ? 2 : 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmKV, const AttnDecodeTcParams p) {
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G;
  const int len = p.seq_lens[b];
  if (len <= 0) {   // padding row: zeros
    for (int i = tid; i < G * DT_D / 8; i += DT_THREADS)
      reinterpret_cast<uint4*>(p.out + (size_t)b * p.Hq * DT_D + (size_t)kvh * G * DT_D)[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int n_tiles = (len + DT_BN - 1) / DT_BN;
  const bool rope = p.cos_sin != nullptr;
  int pos = rope ? p.positions[b] : -1;
  // the new token is the last one of the context (its rows are patched into the last tile)
  if (rope && pos >= 0 && (pos >= p.max_pos || pos != len - 1)) { report_status(p.status, ST_BAD_INDEX, pos); pos = -1; }

  extern __shared__ uint8_t dt_smem_raw[];
  const uint32_t base = (smem_u32(dt_smem_raw) + 1023u) & ~1023u;
  uint8_t* bp = dt_smem_raw + (base - smem_u32(dt_smem_raw));
  const uint32_t q_s = base + DtLayout<DT_SLOTS>::OFF_Q, p_s = base + DtLayout<DT_SLOTS>::OFF_P;
  float* sT = reinterpret_cast<float*>(bp + DtLayout<DT_SLOTS>::OFF_ST);
  __nv_bfloat16* new_kv = reinterpret_cast<__nv_bfloat16*>(bp + DtLayout<DT_SLOTS>::OFF_NEW);     // [0..127] k row, [128..255] v row
  float* m_s = reinterpret_cast<float*>(bp + DtLayout<DT_SLOTS>::OFF_STATS);
  float* l_s = m_s + DT_GP;
  float* alpha_s = l_s + DT_GP;
  const uint32_t bars = base + DtLayout<DT_SLOTS>::OFF_BARS;
  const uint32_t bar_sfull = bars /* S^T buffer 0 */, bar_sfull1 = bars + 8 /* S^T buffer 1 */, bar_pfull = bars + 16,
                 bar_odone = bars + 24, bar_qready = bars + 32, bar_kpatch = bars + 40;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bp + DtLayout<DT_SLOTS>::OFF_BARS + 48);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bp + DtLayout<DT_SLOTS>::OFF_BARS + 56);    // [1]: never set
  const uint32_t bar_full = bars + 64, bar_empty = bars + 64 + 8 * DT_SLOTS;       // one pair per ring slot

  if (tid == 0) {
    for (int i = 0; i < DT_SLOTS; ++i) { mbar_init(bar_full + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
    mbar_init(bar_sfull, 1); mbar_init(bar_sfull1, 1); mbar_init(bar_pfull, 128); mbar_init(bar_odone, 1);
    mbar_init(bar_qready, 128); mbar_init(bar_kpatch, 128);
    abort_flag[0] = 0; abort_flag[1] = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), DT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_s = tmem, tm_o = tmem + 32;      // S^T of tile j at tm_s + 16 * (j & 1)

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: K_0, V_0, K_1, V_1, ... through the ring
    if (lane == 0) {
      tma_prefetch_desc(&tmKV);
      const uint64_t pol = l2_policy_evict_first();
      bool ok = true;
      int armed = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int n0 = j * DT_BN;
        const int n_pages = (min(len, n0 + DT_BN) - n0 + DT_PS - 1) / DT_PS;
        const int* bt = p.block_table + (size_t)b * p.max_blocks + n0 / DT_PS;
        for (int kv01 = 0; kv01 < 2; ++kv01) {
          const int it = 2 * j + kv01, s = it % DT_SLOTS, use = it / DT_SLOTS;
          if (use > 0 && !mbar_wait(bar_empty + 8 * s, (use - 1) & 1, abort_flag, DT_BUDGET_NS)) { ok = false; break; }
          mbar_expect_tx(bar_full + 8 * s, (uint32_t)n_pages * 2 * DT_PS * 128);
          ++armed;
          const uint32_t dst = base + s * DT_TILE;
          for (int pg = 0; pg < n_pages; ++pg) {
            int page = bt[pg];
            if (page < 0 || page >= p.num_pages) { report_status(p.status, ST_BAD_INDEX, page); page = 0; }
            const int row = ((page * 2 + kv01) * p.Hkv + kvh) * DT_PS;
            tma_load_2d(dst + pg * DT_PS * 128, &tmKV, bar_full + 8 * s, 0, row, pol);
            tma_load_2d(dst + DT_HALF + pg * DT_PS * 128, &tmKV, bar_full + 8 * s, 64, row, pol);
          }
        }
      }
      if (!ok) {
        if (abort_flag[0] == 0) { abort_flag[0] = 1; report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, 20); }
        // copies already issued still write this CTA's shared memory: wait for the last armed phase of every slot
        for (int s = 0; s < DT_SLOTS; ++s) {
          const int n_s = armed > s ? (armed - s + DT_SLOTS - 1) / DT_SLOTS : 0;
          if (n_s > 0) mbar_wait(bar_full + 8 * s, (n_s - 1) & 1, abort_flag + 1, DT_BUDGET_NS);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, DT_BN, 16);
      const uint32_t idesc_o = umma_idesc(1, 1, DT_D, 16) | (1u << 15);        // A operand (V) MN-major
      bool ok = mbar_wait(bar_qready, 0, abort_flag, DT_BUDGET_NS);
      // S^T of tile j + 1 is issued before the wait for the softmax of tile j (two S^T buffers), so the scores of the next
      // tile are ready when the compute warps come for them
      auto issue_s = [&](int j, bool k_landed) -> bool {
        const int itk = 2 * j;
        const uint32_t ks = base + (itk % DT_SLOTS) * DT_TILE;
        if (!k_landed && !mbar_wait(bar_full + 8 * (itk % DT_SLOTS), (itk / DT_SLOTS) & 1, abort_flag, DT_BUDGET_NS)) return false;
        if (pos >= 0 && j == n_tiles - 1 && !mbar_wait(bar_kpatch, 0, abort_flag, DT_BUDGET_NS)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < DT_D / 16; ++k)
          mma_f16(tm_s + 16 * (j & 1), umma_desc_sw128(ks + (k >> 2) * DT_HALF + (k & 3) * 32),
                  umma_desc_sw128(q_s + (k >> 2) * DT_QP_HALF + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
        tc_commit(bar_empty + 8 * (itk % DT_SLOTS));
        tc_commit((j & 1) ? bar_sfull1 : bar_sfull);
        return true;
      };
      ok = ok && issue_s(0, false);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int itv = 2 * j + 1;
        const uint32_t vs = base + (itv % DT_SLOTS) * DT_TILE;
        // While waiting for P^T of tile j: if the K tile of j + 1 has landed, its scores are issued ahead (never the other
        // way round: O^T of tile j does not wait for a K tile still in flight). The last tile of a step with RoPE fused
        // waits for the patch of its K row, which the compute warps make after their work on tile j: not issued ahead.
        bool s_next = !(j + 1 < n_tiles);
        const bool may_ahead = j + 1 < n_tiles && !(pos >= 0 && j + 1 == n_tiles - 1);
        {
          const int itk = 2 * (j + 1);
          const uint32_t kbar = bar_full + 8 * (itk % DT_SLOTS), kpar = (itk / DT_SLOTS) & 1;
          const uint64_t t0 = global_timer_ns();
          bool p_ready = false;
          uint32_t spins = 0;
          while (!p_ready) {
            if (may_ahead && !s_next && mbar_test_wait(kbar, kpar)) {
              if (!issue_s(j + 1, true)) { ok = false; break; }
              s_next = true;
            }
            p_ready = mbar_try_wait(bar_pfull, j & 1);
            if (!p_ready && (++spins & 255) == 0 && (abort_flag[0] || global_timer_ns() - t0 > DT_BUDGET_NS)) { ok = false; break; }
          }
          if (!ok) break;
        }
        if (!mbar_wait(bar_full + 8 * (itv % DT_SLOTS), (itv / DT_SLOTS) & 1, abort_flag, DT_BUDGET_NS)) { ok = false; break; }
        tc_fence_after();
        const int n_valid = min(len, (j + 1) * DT_BN) - j * DT_BN;
        const int k_steps = (n_valid + 15) / 16;
        for (int k = 0; k < k_steps; ++k)       // 16 tokens per step: A advances 16 rows of 128 bytes, B 32 bytes
          mma_f16(tm_o, dt_desc_mn(vs + k * 16 * 128, DT_HALF), umma_desc_sw128(p_s + (k >> 2) * DT_QP_HALF + (k & 3) * 32),
                  idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar_empty + 8 * (itv % DT_SLOTS));
        tc_commit(bar_odone);
        if (!s_next && !issue_s(j + 1, false)) { ok = false; break; }
      }
      if (!ok && abort_flag[0] == 0) { abort_flag[0] = 1; report_status(p.status, ST_TIMEOUT_SMEM_FULL, 21); }
    }
  } else {
    // ------------------------------------------------------------ compute warps (128 threads)
    const int ct = tid - 64, cw = warp - 2;
    const int lane_grp = warp & 3;                       // tensor-memory lanes this warp may access: 32 * lane_grp ..
    const int row = lane_grp * 32 + lane;                // token of the tile (S^T) / head-dimension index (O^T)
    const uint32_t lane_addr = (uint32_t)(lane_grp * 32) << 16;
    // ---- prologue: Q^T tile (rows >= G zero), P^T rows zero, running statistics; new token's K / V rows ----
    {
      const int r = ct >> 3, ch = ct & 7;                // one pair of 16-byte chunks (dims ch*8.., 64 + ch*8..) of row r
      uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
      if (r < G && (!rope || pos >= 0)) {
        const __nv_bfloat16* qp = p.q + (size_t)b * p.q_stride + (size_t)(kvh * G + r) * DT_D;
        lo = *reinterpret_cast<const uint4*>(qp + ch * 8);
        hi = *reinterpret_cast<const uint4*>(qp + 64 + ch * 8);
        if (rope) {   // rotate-half: dim i pairs with dim i + 64
          const float4* cs = reinterpret_cast<const float4*>(p.cos_sin + ((size_t)pos * 64 + ch * 8) * 2);
          __nv_bfloat162* lb = reinterpret_cast<__nv_bfloat162*>(&lo);
          __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 c2 = cs[i];   // (cos, sin) of dims 2i and 2i + 1 of this chunk
            const float2 x0 = __bfloat1622float2(lb[i]), x1 = __bfloat1622float2(hb[i]);
            lb[i] = __floats2bfloat162_rn(x0.x * c2.x - x1.x * c2.y, x0.y * c2.z - x1.y * c2.w);
            hb[i] = __floats2bfloat162_rn(x1.x * c2.x + x0.x * c2.y, x1.y * c2.z + x0.y * c2.w);
          }
        }
      }
      // 16-row B operand tile: half h at h * 2 KB, row r at r * 128, 16-byte chunk c at (c ^ (r & 7)) * 16
      const uint32_t qa = q_s + r * 128 + ((ch ^ (r & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(qa), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(qa + DT_QP_HALF), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(p_s + ct * 16), "r"(0) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(p_s + DT_QP_HALF + ct * 16), "r"(0) : "memory");
      if (ct < DT_GP) { m_s[ct] = -INFINITY; l_s[ct] = 0.f; alpha_s[ct] = 1.f; }
      if (pos >= 0) {
        // the new token: rotated K row and V row go to the cache (for the steps to come) and into shared memory (for
        // the patch of this step's last tile)
        int pg = p.block_table[(size_t)b * p.max_blocks + pos / DT_PS];
        const bool pg_ok = pg >= 0 && pg < p.num_pages;
        if (!pg_ok && ct == 0) report_status(p.status, ST_BAD_INDEX, pg);
        const __nv_bfloat16* kr = p.q + (size_t)b * p.q_stride + (size_t)(p.Hq + kvh) * DT_D;
        const __nv_bfloat16* vr = kr + (size_t)p.Hkv * DT_D;
        __nv_bfloat16* kd = p.kv_rw + (((size_t)(pg_ok ? pg : 0) * 2) * p.Hkv + kvh) * (size_t)DT_PS * DT_D + (size_t)(pos % DT_PS) * DT_D;
        __nv_bfloat16* vd = kd + (size_t)p.Hkv * DT_PS * DT_D;
        if (ct < 64) {
          const float2 cs = reinterpret_cast<const float2*>(p.cos_sin)[(size_t)pos * 64 + ct];
          const float x0 = __bfloat162float(kr[ct]), x1 = __bfloat162float(kr[ct + 64]);
          const __nv_bfloat16 k0 = __float2bfloat16(x0 * cs.x - x1 * cs.y), k1 = __float2bfloat16(x1 * cs.x + x0 * cs.y);
          new_kv[ct] = k0; new_kv[ct + 64] = k1;
          if (pg_ok) { kd[ct] = k0; kd[ct + 64] = k1; }
        } else {
          const int j2 = ct - 64;
          const __nv_bfloat162 v2 = reinterpret_cast<const __nv_bfloat162*>(vr)[j2];
          reinterpret_cast<__nv_bfloat162*>(new_kv + 128)[j2] = v2;
          if (pg_ok) reinterpret_cast<__nv_bfloat162*>(vd)[j2] = v2;
        }
      }
      dt_fence_async_smem();          // Q^T and P^T rows were written with ordinary stores, the MMA reads them
      mbar_arrive(bar_qready);
      dt_bar_compute();
    }
    bool ok = true;
    // the new token's K row goes into the LAST K tile once TMA has landed it (row pos - the tile's first token, 128-byte
    // swizzle); the MMA warp issues that tile's scores only after this
    auto patch_k = [&]() -> bool {
      const int itk = 2 * (n_tiles - 1);
      if (!mbar_wait(bar_full + 8 * (itk % DT_SLOTS), (itk / DT_SLOTS) & 1, abort_flag, DT_BUDGET_NS)) return false;
      const uint32_t ks = base + (itk % DT_SLOTS) * DT_TILE;
      const uint16_t kvv = reinterpret_cast<const uint16_t*>(new_kv)[ct];
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(ks + dt_tile_off(pos - (n_tiles - 1) * DT_BN, ct)), "h"(kvv) : "memory");
      dt_fence_async_smem();
      mbar_arrive(bar_kpatch);
      return true;
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int n0 = j * DT_BN;
      const bool last = j == n_tiles - 1;
      if (pos >= 0 && n_tiles == 1 && !patch_k()) { ok = false; break; }
      if (!mbar_wait((j & 1) ? bar_sfull1 : bar_sfull, (j >> 1) & 1, abort_flag, DT_BUDGET_NS)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t sv[16];
        tmem_ld16(tm_s + 16 * (j & 1) + lane_addr, sv);
        tmem_ld_wait();
        const bool vis = n0 + row < len;
#pragma unroll
        for (int g = 0; g < DT_GP; ++g) sT[g * DT_BN + row] = vis ? __uint_as_float(sv[g]) : -INFINITY;
      }
      dt_bar_compute();
      // each warp owns heads cw and cw + 4: a lane holds four consecutive tokens of the row
      uint32_t pk[DT_GP / 4][2];
#pragma unroll
      for (int i = 0; i < DT_GP / 4; ++i) {
        const int g = cw + 4 * i;
        const float4 s4 = reinterpret_cast<const float4*>(sT + g * DT_BN)[lane];
        float mx = fmaxf(fmaxf(s4.x, s4.y), fmaxf(s4.z, s4.w));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        mx *= p.scale_log2e;                                   // the scale is positive
        const float m_old = m_s[g];
        // the reference maximum only moves when the tile's maximum exceeds it by more than 2^8 (see attn_prefill_tc.cu)
        const float m_new = (m_old == -INFINITY || mx > m_old + 8.f) ? fmaxf(m_old, mx) : m_old;
        const float alpha = (m_old == -INFINITY) ? 1.f : exp2f(m_old - m_new);
        const __nv_bfloat162 p01 = __floats2bfloat162_rn(exp2f(fmaf(s4.x, p.scale_log2e, -m_new)), exp2f(fmaf(s4.y, p.scale_log2e, -m_new)));
        const __nv_bfloat162 p23 = __floats2bfloat162_rn(exp2f(fmaf(s4.z, p.scale_log2e, -m_new)), exp2f(fmaf(s4.w, p.scale_log2e, -m_new)));
        const float2 f01 = __bfloat1622float2(p01), f23 = __bfloat1622float2(p23);
        float sum = (f01.x + f01.y) + (f23.x + f23.y);        // over the rounded values, the ones the tensor cores multiply
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        pk[i][0] = *reinterpret_cast<const uint32_t*>(&p01);
        pk[i][1] = *reinterpret_cast<const uint32_t*>(&p23);
        if (lane == 0) { m_s[g] = m_new; l_s[g] = l_s[g] * alpha + sum; alpha_s[g] = alpha; }
      }
      dt_bar_compute();
      if (j > 0) {
        // O^T of the previous tiles is complete in tensor memory; bring it to the new reference where a head moved
        if (!mbar_wait(bar_odone, (j - 1) & 1, abort_flag, DT_BUDGET_NS)) { ok = false; break; }
        tc_fence_after();
        float al[DT_GP];
        bool moved = false;
#pragma unroll
        for (int g = 0; g < DT_GP; ++g) { al[g] = alpha_s[g]; moved |= al[g] != 1.f; }
        if (moved) {     // uniform over the CTA: every thread reads the same eight values
          uint32_t ov[16];
          tmem_ld16(tm_o + lane_addr, ov);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < DT_GP; ++g) ov[g] = __float_as_uint(__uint_as_float(ov[g]) * al[g]);
          tmem_st16(tm_o + lane_addr, ov);
          tmem_st_wait();
        }
      }
      // P^T of this tile: only now, when the MMAs that read the previous tile's P^T have completed (o_done above)
#pragma unroll
      for (int i = 0; i < DT_GP / 4; ++i) {
        const int g = cw + 4 * i;
        // tokens 4 * lane .. + 3 of row g: half (lane >> 4), 16-byte chunk ((lane & 15) >> 1), upper or lower 8 bytes
        const uint32_t pa = p_s + (lane >> 4) * DT_QP_HALF + g * 128 + ((((lane & 15) >> 1) ^ (g & 7)) << 4) + (lane & 1) * 8;
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(pa), "r"(pk[i][0]), "r"(pk[i][1]) : "memory");
      }
      if (last) {
        // V tile: the new token's row (RoPE fused) and zeros in the rest of the last 16-token step, so that 0 * (never
        // written cache slots) cannot produce a NaN
        const int itv = 2 * j + 1;
        if (!mbar_wait(bar_full + 8 * (itv % DT_SLOTS), (itv / DT_SLOTS) & 1, abort_flag, DT_BUDGET_NS)) { ok = false; break; }
        const uint32_t vs = base + (itv % DT_SLOTS) * DT_TILE;
        const int first = len - n0;                              // rows first .. of the tile are past the context
        const int n_zero = ((first + 15) & ~15) - first;
        for (int i = ct; i < n_zero * 8; i += 128) {             // 16-byte chunks of those rows, per half
          const uint32_t a = vs + first * 128 + i * 16;
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a + DT_HALF), "r"(0) : "memory");
        }
        if (pos >= 0) {
          const uint16_t vv = reinterpret_cast<const uint16_t*>(new_kv)[128 + ct];
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(vs + dt_tile_off(pos - n0, ct)), "h"(vv) : "memory");
        }
      }
      dt_fence_async_smem();     // P^T (and the V patch) were written with ordinary stores
      tc_fence_before();
      mbar_arrive(bar_pfull);
      if (pos >= 0 && n_tiles >= 2 && j == n_tiles - 2 && !patch_k()) { ok = false; break; }
    }
    if (ok && mbar_wait(bar_odone, (n_tiles - 1) & 1, abort_flag, DT_BUDGET_NS)) {
      tc_fence_after();
      uint32_t ov[16];
      tmem_ld16(tm_o + lane_addr, ov);
      tmem_ld_wait();
      __nv_bfloat16* op = p.out + (size_t)b * p.Hq * DT_D + (size_t)kvh * G * DT_D + row;
#pragma unroll
      for (int g = 0; g < DT_GP; ++g) {
        if (g < G) {
          const float l = l_s[g];
          op[(size_t)g * DT_D] = __float2bfloat16(l > 0.f ? __uint_as_float(ov[g]) / l : 0.f);
        }
      }
    } else if (abort_flag[0] == 0) {
      abort_flag[0] = 1;
      report_status(p.status, ST_TIMEOUT_TMEM_FULL, 22);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, DT_TMEM_COLS);
  }
}

}  // namespace skein

// Returns 0, a cudaError_t, or -1 for shapes this kernel does not take (the caller then uses the mma.sync kernel).
// cos_sin / positions null: q is already rotated and the cache already holds the new token.
extern "C" int skein_attn_decode_tc(const void* q, long long q_stride, void* kv, const int* block_table, const int* seq_lens,
                                    const int* positions, const float* cos_sin, int max_pos, void* out, int* status, int B,
                                    int Hq, int Hkv, int D, int page_size, int max_blocks, int num_pages, float scale,
                                    void* stream) {
  using namespace skein;
  if (B == 0) return 0;
  if (D != DT_D || page_size != DT_PS || Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > DT_GP || q_stride % 8 != 0) return -1;
  // at most one CTA per SM: the deep ring; otherwise two CTAs per SM with three slots each
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  static int sm_cache[64] = {0};
  if (dev >= 0 && dev < 64) {
    if (sm_cache[dev] == 0) cudaDeviceGetAttribute(&sm_cache[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sm_cache[dev] > 0) sms = sm_cache[dev];
  }
  const bool deep = (long long)B * Hkv <= sms;
  static bool attr_set[2] = {false, false};
  if (!attr_set[deep ? 1 : 0]) {
    cudaError_t e = deep ? cudaFuncSetAttribute(attn_decode_tc_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, DtLayout<6>::SMEM)
                         : cudaFuncSetAttribute(attn_decode_tc_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, DtLayout<3>::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set[deep ? 1 : 0] = true;
  }
  CUtensorMap tmKV;
  int rc = cached_tmap_2d(&tmKV, kv, (uint64_t)num_pages * 2 * Hkv * DT_PS, DT_D, 2, DT_PS);
  if (rc != 0) return rc;
  AttnDecodeTcParams p;
  p.q = (const __nv_bfloat16*)q; p.kv_rw = (__nv_bfloat16*)kv; p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = (__nv_bfloat16*)out; p.status = status; p.q_stride = q_stride;
  p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.cos_sin = cos_sin; p.positions = positions; p.max_pos = max_pos;
  if (deep)
    attn_decode_tc_kernel<6><<<dim3(Hkv, B), DT_THREADS, DtLayout<6>::SMEM, (cudaStream_t)stream>>>(tmKV, p);
  else
    attn_decode_tc_kernel<3><<<dim3(Hkv, B), DT_THREADS, DtLayout<3>::SMEM, (cudaStream_t)stream>>>(tmKV, p);
  return (int)cudaGetLastError();
}
