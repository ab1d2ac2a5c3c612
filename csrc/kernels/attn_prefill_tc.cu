// Causal prefill attention over the paged KV cache on the 5th-generation tensor cores (tcgen05, accumulators in
// tensor memory, operands staged by TMA). Same contract as attn_prefill.cu (chunked-prefill aware: a chunk of q_len
// new tokens attends to the kv_len tokens already in the cache, its own included); this is the kernel the prefill
// path runs for head_dim 128 and 16-token pages, the mma.sync kernel stays as the fallback for other shapes.
//
// One CTA = 128 query rows of one head, walking the context in 128-token tiles:
//
//   warp 0      TMA producer: the Q tile once, then per context tile the K pages and the V pages of the tile
//               (one 16-token x 64-element box per page and head-dim half, 128-byte swizzle) into single K and V
//               buffers; the block table is read here, nothing is gathered through registers
//   warp 1      MMA issuer (one elected lane): S = Q K^T (M 128 queries, N 128 tokens, K = head dim, both operands
//               K-major in shared memory, accumulator S in tensor memory), and O += P V with P taken from TENSOR
//               MEMORY as the A operand and the V tile as an MN-major B operand (tokens are the reduction dimension
//               and the cache stores a token's 128 values contiguously), accumulator O in tensor memory
//   warps 2-5   softmax: thread t owns query row t (tensor-memory lane t). Two passes over the row of S (row max,
//               then exp2 / row sum / bf16 P written back over the first half of S's columns); O is rescaled in
//               tensor memory only when some row of the warp raised its maximum; the last tile's rows are normalised
//               and stored from registers
//
// S (128 columns), P (aliased on S) and O (128 columns) take 256 tensor-memory columns and the three operand buffers
// 96 KB of shared memory, so TWO CTAs are resident per SM: while one CTA's softmax warps work on a tile, the other
// CTA's MMAs use the tensor cores. Every wait is bounded; on expiry the CTA records a status code, waits (bounded) for
// its copies in flight, frees its tensor memory and returns.
//
// The reference never runs a prefill attention kernel: its FlashInfer prefill wrapper returns -1
// (vendor/luminal/crates/luminal_cuda_lite/src/host/flashinfer/wrapper.cu:263-281) and prefill falls back to unfused
// graph ops (crates/skein_emit/src/op_wiring.rs:2155-2305).
#include "ptx.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes, uint32_t box_rows);

constexpr int TC_BM = 128, TC_BN = 128, TC_D = 128, TC_PS = 16;
constexpr int TC_THREADS = 192;
constexpr int TC_HALF_BYTES = 128 * 128;              // one 64-element half of a 128-row tile, 128-byte rows
constexpr int TC_TILE_BYTES = 2 * TC_HALF_BYTES;
constexpr int TC_SMEM = 3 * TC_TILE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int TC_TMEM_COLS = 256;
constexpr uint64_t TC_BUDGET_NS = 4000000000ull;

struct AttnPrefillTcParams {
  const int* block_table;   // [S, max_blocks]
  const int* q_start;       // [S] first row of the sequence's chunk in q / out
  const int* q_len;         // [S]
  const int* kv_len;        // [S] tokens in the cache after this chunk was appended
  __nv_bfloat16* out;       // [T, Hq * D]
  int* status;
  int Hq, Hkv, max_blocks, num_pages;
  float scale_log2e;
};

// Shared-memory descriptor of an MN-major operand tile (the reduction dimension strides over 128-byte rows): 64
// elements of the MN dimension are contiguous in a row, 8 rows form a 1024-byte swizzle atom; `lbo` is the distance
// between consecutive 64-element chunks of the MN dimension, the atoms of consecutive 8-row groups follow at 1024 bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(TC_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                       const AttnPrefillTcParams p) {
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;     // long rows first: the causal work grows with the row
  const int head = blockIdx.y, seq = blockIdx.z;
  const int qlen = p.q_len[seq];
  const int q0 = qt * TC_BM;
  if (q0 >= qlen) return;
  const int kvlen = p.kv_len[seq];
  const int pos0 = kvlen - qlen;                            // absolute position of the chunk's first token
  const int qrow0 = p.q_start[seq];
  const int kvh = head / (p.Hq / p.Hkv);
  int kv_hi = pos0 + min(q0 + TC_BM, qlen);                 // exclusive bound of the keys any row of this tile sees
  if (kv_hi > kvlen) kv_hi = kvlen;
  const int n_tiles = (kv_hi + TC_BN - 1) / TC_BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, k_s = base + TC_TILE_BYTES, v_s = base + 2 * TC_TILE_BYTES;
  const uint32_t bars = base + 3 * TC_TILE_BYTES;
  const uint32_t bar_q = bars, bar_kfull = bars + 8, bar_kempty = bars + 16, bar_vfull = bars + 24, bar_vempty = bars + 32,
                 bar_sfull = bars + 40, bar_pfull = bars + 48, bar_odone = bars + 56;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + 3 * TC_TILE_BYTES + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + 3 * TC_TILE_BYTES + 72);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_kfull, 1); mbar_init(bar_kempty, 1); mbar_init(bar_vfull, 1);
    mbar_init(bar_vempty, 1); mbar_init(bar_sfull, 1); mbar_init(bar_pfull, 128); mbar_init(bar_odone, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;      // never set: the drain waits of a failing producer run out on their time budget only
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_s = tmem, tm_p = tmem, tm_o = tmem + 128;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmKV);
      const uint64_t pol_q = l2_policy_evict_first(), pol_kv = l2_policy_evict_last();
      mbar_expect_tx(bar_q, TC_TILE_BYTES);
      tma_load_2d(q_s, &tmQ, bar_q, head * TC_D, qrow0 + q0, pol_q);
      tma_load_2d(q_s + TC_HALF_BYTES, &tmQ, bar_q, head * TC_D + 64, qrow0 + q0, pol_q);
      bool ok = true;
      int armed_k = 0, armed_v = 0;      // phases armed so far (for the bounded drain on an early exit)
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int n0 = j * TC_BN;
        const int n_pages = (min(kv_hi, n0 + TC_BN) - n0 + TC_PS - 1) / TC_PS;
        const int* bt = p.block_table + (size_t)seq * p.max_blocks + n0 / TC_PS;
        for (int kv01 = 0; kv01 < 2 && ok; ++kv01) {
          const uint32_t full = kv01 ? bar_vfull : bar_kfull, empty = kv01 ? bar_vempty : bar_kempty;
          const uint32_t dst = kv01 ? v_s : k_s;
          if (j > 0 && !mbar_wait(empty, (j - 1) & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
          mbar_expect_tx(full, (uint32_t)n_pages * 2 * TC_PS * 128);
          if (kv01) ++armed_v; else ++armed_k;
          for (int pg = 0; pg < n_pages; ++pg) {
            int page = bt[pg];
            if (page < 0 || page >= p.num_pages) { report_status(p.status, ST_BAD_INDEX, page); page = 0; }
            const int row = ((page * 2 + kv01) * p.Hkv + kvh) * TC_PS;
            tma_load_2d(dst + pg * TC_PS * 128, &tmKV, full, 0, row, pol_kv);
            tma_load_2d(dst + TC_HALF_BYTES + pg * TC_PS * 128, &tmKV, full, 64, row, pol_kv);
          }
        }
      }
      if (!ok) {
        if (*abort_flag == 0) { *abort_flag = 1; report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, 10); }
        // copies already issued still write this CTA's shared memory: wait for them (bounded) before leaving
        if (armed_k > 0) mbar_wait(bar_kfull, (armed_k - 1) & 1, abort_flag + 1, TC_BUDGET_NS);
        if (armed_v > 0) mbar_wait(bar_vfull, (armed_v - 1) & 1, abort_flag + 1, TC_BUDGET_NS);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, TC_BM, TC_BN);
      const uint32_t idesc_o = umma_idesc(1, 1, TC_BM, TC_D) | (1u << 16);      // B operand MN-major
      bool ok = mbar_wait(bar_q, 0, abort_flag, TC_BUDGET_NS);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!mbar_wait(bar_kfull, j & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < TC_D / 16; ++k) {
          const uint32_t off = (k >> 2) * TC_HALF_BYTES + (k & 3) * 32;
          mma_f16(tm_s, umma_desc_sw128(q_s + off), umma_desc_sw128(k_s + off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_kempty);
        tc_commit(bar_sfull);
        if (!mbar_wait(bar_pfull, j & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
        if (!mbar_wait(bar_vfull, j & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
        tc_fence_after();
        const int n_valid = min(kv_hi, (j + 1) * TC_BN) - j * TC_BN;
        const int k_steps = (n_valid + 15) / 16;               // 16-token steps that hold at least one visible key
        for (int k = 0; k < k_steps; ++k)
          mma_f16_ts(tm_o, tm_p + k * 8, umma_desc_sw128_mn(v_s + k * 16 * 128, TC_HALF_BYTES), idesc_o,
                     (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar_vempty);
        tc_commit(bar_odone);
      }
      if (!ok && *abort_flag == 0) { *abort_flag = 1; report_status(p.status, ST_TIMEOUT_SMEM_FULL, 11); }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: thread <-> query row
    const int lane_grp = warp & 3;                      // the 32 tensor-memory lanes this warp may access
    const int r = lane_grp * 32 + lane;                 // row of the tile
    const uint32_t lane_addr = (uint32_t)(lane_grp * 32) << 16;
    int pos_r = pos0 + q0 + r;
    if (pos_r > kvlen - 1) pos_r = kvlen - 1;           // rows past the chunk are computed, finite, and never stored
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int n0 = j * TC_BN;
      if (!mbar_wait(bar_sfull, j & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
      tc_fence_after();
      const bool masked = n0 + TC_BN - 1 > pos0 + q0;   // some row of the tile sees only part of these keys
      const int limit = pos_r - n0;                     // this row sees columns 0 .. limit of the tile
      // pass 1: row maximum of the raw scores (64 columns per round: both loads in flight before the wait)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int h = 0; h < TC_BN / 64; ++h) {
        uint32_t sv[64];
        tmem_ld32(tm_s + lane_addr + h * 64, sv);
        tmem_ld32(tm_s + lane_addr + h * 64 + 32, sv + 32);
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], (h * 64 + i <= limit) ? __uint_as_float(sv[i]) : -INFINITY);
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;    // the scale is positive
      // The running maximum only moves when the tile's maximum exceeds it by more than 2^8: until then the
      // probabilities of this tile are at most 256 (exact in bf16 and harmless in the fp32 sums), and O needs no
      // rescaling; the final division by the row sum undoes whatever reference the row ended on.
      const float m_new = (m == -INFINITY || mx > m + 8.f) ? fmaxf(m, mx) : m;
      const float alpha = (m == -INFINITY) ? 1.f : exp2f(m - m_new);
      if (j > 0) {
        // O of the previous tiles is complete in tensor memory; bring it to the new reference if some row moved
        if (!mbar_wait(bar_odone, (j - 1) & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int h = 0; h < TC_D / 64; ++h) {
            uint32_t ov[64];
            tmem_ld32(tm_o + lane_addr + h * 64, ov);
            tmem_ld32(tm_o + lane_addr + h * 64 + 32, ov + 32);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 64; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st16(tm_o + lane_addr + h * 64 + c * 16, ov + c * 16);
          }
        }
      }
      l *= alpha;
      m = m_new;
      // pass 2: p = exp2(s * scale - m), row sum, bf16 pairs written over the columns of S already consumed
      float rs = 0.f;
#pragma unroll
      for (int h = 0; h < TC_BN / 64; ++h) {
        uint32_t sv[64];
        tmem_ld32(tm_s + lane_addr + h * 64, sv);
        tmem_ld32(tm_s + lane_addr + h * 64 + 32, sv + 32);
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float x0 = fmaf(__uint_as_float(sv[i]), p.scale_log2e, -m_new);
          float x1 = fmaf(__uint_as_float(sv[i + 1]), p.scale_log2e, -m_new);
          if (masked) {
            if (h * 64 + i > limit) x0 = -INFINITY;
            if (h * 64 + i + 1 > limit) x1 = -INFINITY;
          }
          const float p0 = exp2f(x0), p1 = exp2f(x1);
          // the row sum is taken over the rounded values, the ones the tensor cores multiply
          const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          const float2 pf = __bfloat1622float2(pb);
          rs += pf.x + pf.y;
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        // columns [32 h, 32 h + 32) of P lie inside columns [0, 64 h + 64) of S, all of which have been read
        tmem_st16(tm_p + lane_addr + h * 32, pk);
        tmem_st16(tm_p + lane_addr + h * 32 + 16, pk + 16);
      }
      l += rs;
      if (n0 + TC_BN > kv_hi) {
        // last tile: its final 16-token step may hold rows of V past the context (slots of the page that were never
        // written); zero them so that 0 * garbage cannot produce a NaN. Needs V landed; a 128-byte row is a
        // permutation of itself under the swizzle, so whole rows can be cleared without computing it.
        if (!mbar_wait(bar_vfull, j & 1, abort_flag, TC_BUDGET_NS)) { ok = false; break; }
        const int first = kv_hi - n0;
        const int n_rows = ((first + 15) & ~15) - first;        // rows of the last 16-token step past the context
        for (int i = r; i < n_rows * 8; i += 128) {              // 16-byte chunks of those rows, per half
          const uint32_t a = v_s + first * 128 + i * 16;
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a + TC_HALF_BYTES), "r"(0) : "memory");
        }
        fence_proxy_async_smem();
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_pfull);
    }
    if (ok && mbar_wait(bar_odone, (n_tiles - 1) & 1, abort_flag, TC_BUDGET_NS)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool store = q0 + r < qlen;
      __nv_bfloat16* orow = p.out + (size_t)(qrow0 + q0 + r) * ((size_t)p.Hq * TC_D) + (size_t)head * TC_D;
#pragma unroll
      for (int c = 0; c < TC_D / 16; ++c) {
        uint32_t ov[16];
        tmem_ld16(tm_o + lane_addr + c * 16, ov);
        tmem_ld_wait();
        if (store) {
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(ov[2 * i]) * inv, __uint_as_float(ov[2 * i + 1]) * inv);
            pk[i] = *reinterpret_cast<const uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(orow + c * 16 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
    } else if (*abort_flag == 0) {
      *abort_flag = 1;
      report_status(p.status, ST_TIMEOUT_TMEM_FULL, 12);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TC_TMEM_COLS);
  }
}

}  // namespace skein

// Returns 0, a cudaError_t, or a negative code for shapes this kernel does not take (the caller then uses the
// mma.sync kernel): head_dim 128, 16-token pages, 16-byte aligned rows.
extern "C" int skein_attn_prefill_tc(const void* q, long long q_stride, long long q_rows, const void* kv, const int* block_table,
                                     const int* q_start, const int* q_len, const int* kv_len, void* out, int* status, int S,
                                     int max_q_len, int Hq, int Hkv, int D, int page_size, int max_blocks, int num_pages,
                                     float scale, void* stream) {
  using namespace skein;
  if (S == 0 || max_q_len == 0) return 0;
  if (D != TC_D || page_size != TC_PS || Hq % Hkv != 0 || q_stride % 8 != 0) return -1;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  CUtensorMap tmQ, tmKV;
  int rc = cached_tmap_2d(&tmQ, q, (uint64_t)q_rows, (uint64_t)q_stride, 2, TC_BM);
  if (rc != 0) return rc;
  rc = cached_tmap_2d(&tmKV, kv, (uint64_t)num_pages * 2 * Hkv * TC_PS, TC_D, 2, TC_PS);
  if (rc != 0) return rc;
  AttnPrefillTcParams p;
  p.block_table = block_table; p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.out = (__nv_bfloat16*)out; p.status = status;
  p.Hq = Hq; p.Hkv = Hkv; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.scale_log2e = scale * 1.4426950408889634f;
  dim3 grid((max_q_len + TC_BM - 1) / TC_BM, Hq, S);
  attn_prefill_tc_kernel<<<grid, TC_THREADS, TC_SMEM, (cudaStream_t)stream>>>(tmQ, tmKV, p);
  return (int)cudaGetLastError();
}
