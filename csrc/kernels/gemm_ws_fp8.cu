// Block-scaled fp8 (e4m3) variant of the weight-streaming GEMM: both operands carry one fp32 scale per
// 1 x 128 block along K (weights quantised offline, activations online by quant.cu).
//
//   Y[t, f] = sum over K-blocks kb of  sx[t, kb] * sw[kb, f] * ( sum_{k in kb} Xq[t, k] * Wq[f, k] )
//
// The inner sum of one K-block (128 e4m3 values = one 128-byte swizzled row per operand, four
// tcgen05.mma kind::f8f6f4 with K = 32) is accumulated exactly in fp32 in TMEM; the epilogue warps pull each
// K-block's partial tile out of TMEM, apply the two scales and accumulate in registers, while the MMA warp
// is already filling the next TMEM buffer (a ring of up to 8 buffers). Everything else (swap-AB, persistent
// stream-K schedule, device-side ragged groups, SwiGLU pair epilogue, deterministic fix-up) is the bf16
// kernel's design (gemm_ws.cu). Weight bytes per decode step halve, which is the point: decode is
// bandwidth-bound.
//
// Scale layouts: w_scale is K-block major, [K / 128][G * rows_per_group], so that the 128 lanes of a tile
// read consecutive floats; x_scale is token major, [x_rows][K / 128].
//
// Replaces the reference's fp8 MoE kernels (vendor/luminal/crates/luminal_cuda_lite/src/host/moe/mod.rs:
// 383-602: per-row activation scales, per-tensor weight scales, CUDA-core GEMV) and its cuBLASLt fp8 path
// with per-tensor scales (host/cublaslt/mod.rs:1050-1071).
#include "gemm_sched.cuh"
#include "ptx.cuh"
#include "launch.cuh"
#include <cuda_runtime.h>

namespace skein {

constexpr int F8_TILE_F = 128;
constexpr int F8_W_TILE_BYTES = 128 * 128;   // 128 rows x 128 e4m3
constexpr int F8_THREADS = 192;
constexpr int F8_MAX_STAGES = 12;
constexpr int F8_MAX_BUFS = 8;

struct F8Args {
  SkeinGemmParams p;
  int stages, stage_bytes, x_tile_bytes, n_bufs, buf_cols;
  uint64_t budget_ns;
};

template <bool DUAL, int NT>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_ws_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const F8Args a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ Sched sched;
  __shared__ __align__(8) uint64_t bar_full[F8_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[F8_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[F8_MAX_BUFS];
  __shared__ __align__(8) uint64_t bar_tempty[F8_MAX_BUFS];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ int epi_last;

  const SkeinGemmParams& p = a.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int ACC = DUAL ? 2 * NT : NT;   // fp32 columns of one K-block partial

  if (threadIdx.x == 0) {
    abort_flag = 0;
    build_sched(sched, p, 128, (int)gridDim.x);
    for (int s = 0; s < a.stages; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int b = 0; b < a.n_bufs; ++b) { mbar_init(smem_u32(&bar_tfull[b]), 1); mbar_init(smem_u32(&bar_tempty[b]), 128); }
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_smem), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  const int KB = sched.KB;
  const long long kb_begin = (long long)blockIdx.x * sched.per;
  long long kb_end = kb_begin + sched.per;
  if (kb_end > sched.TK) kb_end = sched.TK;
  const bool has_work = kb_begin < sched.TK;

  if (has_work) {
    if (warp == 0) {
      // ================= TMA producer =================
      if (elect_one()) {
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
        const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
        const uint32_t tx_bytes = (DUAL ? 2 : 1) * F8_W_TILE_BYTES + a.x_tile_bytes;
        uint32_t it = 0;
        long long pos = kb_begin;
        bool ok = true;
        while (pos < kb_end && ok) {
          const int u = (int)(pos / KB);
          const int kb0 = (int)(pos - (long long)u * KB);
          int kb1 = KB;
          if ((long long)u * KB + KB > kb_end) kb1 = (int)(kb_end - (long long)u * KB);
          const Unit un = decode_unit(sched, p.G, u);
          const int w_row = un.g * p.w_rows_per_group + un.m * F8_TILE_F;
          const int x_row = sched.off[un.g] + un.n * NT;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s = it % a.stages, ph = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, blockIdx.x);
              abort_flag = 1; ok = false; break;
            }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t st = smem_base + s * a.stage_bytes;
            mbar_expect_tx(full, tx_bytes);
            tma_load_2d(st, &tmW, full, kb * 128, w_row, pol_w);
            if (DUAL) tma_load_2d(st + F8_W_TILE_BYTES, &tmW, full, kb * 128, w_row + p.up_row_off, pol_w);
            tma_load_2d(st + (DUAL ? 2 : 1) * F8_W_TILE_BYTES, &tmX, full, kb * 128, x_row, pol_x);
          }
          pos = (long long)u * KB + kb1;
        }
      }
    } else if (warp == 1) {
      // ================= MMA issuer: one fresh accumulator per K-block =================
      if (elect_one()) {
        const uint32_t idesc = umma_idesc(0, 0, F8_TILE_F, NT);   // e4m3 x e4m3 -> fp32
        bool ok = true;
        for (long long g_it = 0; g_it < kb_end - kb_begin && ok; ++g_it) {
          const uint32_t it = (uint32_t)g_it;
          const uint32_t s = it % a.stages, ph = (it / a.stages) & 1;
          const uint32_t b = it % a.n_bufs, bph = (it / a.n_bufs) & 1;
          if (!mbar_wait(smem_u32(&bar_tempty[b]), bph ^ 1, &abort_flag, a.budget_ns)) {
            report_status(p.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x);
            abort_flag = 1; break;
          }
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, a.budget_ns)) {
            report_status(p.status, ST_TIMEOUT_SMEM_FULL, blockIdx.x);
            abort_flag = 1; break;
          }
          tc_fence_after();
          const uint32_t st = smem_base + s * a.stage_bytes;
          const uint32_t d_tmem = tmem_base + b * a.buf_cols;
          const uint64_t dw = umma_desc_sw128(st);
          const uint64_t dx = umma_desc_sw128(st + (DUAL ? 2 : 1) * F8_W_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_f8(d_tmem, dw + 2 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
            if (DUAL) {
              const uint64_t du = umma_desc_sw128(st + F8_W_TILE_BYTES);
              mma_f8(d_tmem + NT, du + 2 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
            }
          }
          tc_commit(smem_u32(&bar_empty[s]));
          tc_commit(smem_u32(&bar_tfull[b]));
        }
      }
    } else {
      // ================= epilogue warps: scale-accumulate every K-block, then finish the tile =================
      const int q = warp & 3;
      const int r = q * 32 + lane;
      const int et = threadIdx.x - 64;
      const size_t slot_elems = (size_t)F8_TILE_F * ACC;
      const int kb_tot = p.K / 128;
      const size_t w_rows_total = (size_t)p.G * p.w_rows_per_group;
      uint32_t it = 0;
      long long pos = kb_begin;
      bool ok = true;
      while (pos < kb_end && ok) {
        const int u = (int)(pos / KB);
        const int kb0 = (int)(pos - (long long)u * KB);
        int kb1 = KB;
        if ((long long)u * KB + KB > kb_end) kb1 = (int)(kb_end - (long long)u * KB);
        const bool full_seg = (kb0 == 0 && kb1 == KB);
        const Unit un = decode_unit(sched, p.G, u);
        int valid = sched.cnt[un.g] - un.n * NT;
        if (valid > NT) valid = NT;
        const int f = un.m * F8_TILE_F + r;
        const bool f_ok = f < p.F;
        const long long row0 = (long long)sched.off[un.g] + (long long)un.n * NT;
        const size_t wrow_g = (size_t)un.g * p.w_rows_per_group + (f_ok ? f : 0);
        const size_t wrow_u = wrow_g + p.up_row_off;

        float accg[NT], accu[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) { accg[j] = 0.f; if (DUAL) accu[j] = 0.f; }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t b = it % a.n_bufs, bph = (it / a.n_bufs) & 1;
          // scales first: their latency hides behind the barrier wait
          const float swg = p.w_scale[(size_t)kb * w_rows_total + wrow_g];
          const float swu = DUAL ? p.w_scale[(size_t)kb * w_rows_total + wrow_u] : 0.f;
          if (!mbar_wait(smem_u32(&bar_tfull[b]), bph, &abort_flag, a.budget_ns)) {
            report_status(p.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x);
            abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t t_acc = tmem_base + b * a.buf_cols + ((uint32_t)(q * 32) << 16);
          uint32_t vg[NT], vu[NT];
#pragma unroll
          for (int c0 = 0; c0 < NT; c0 += 16) {
            tmem_ld16(t_acc + c0, vg + c0);
            if (DUAL) tmem_ld16(t_acc + NT + c0, vu + c0);
          }
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[b]));
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            if (j < valid) {
              const float sx = __ldg(&p.x_scale[(size_t)(row0 + j) * kb_tot + kb]);
              accg[j] += __uint_as_float(vg[j]) * (sx * swg);
              if (DUAL) accu[j] += __uint_as_float(vu[j]) * (sx * swu);
            }
          }
        }
        if (!ok) break;

        bool do_final = full_seg;
        int c_first = 0, c_last = 0;
        if (!full_seg) {
          const long long ub = (long long)u * KB;
          c_first = (int)(ub / sched.per);
          c_last = (int)((ub + KB - 1) / sched.per);
          const int my_slot = ((long long)blockIdx.x * sched.per) / KB == u ? 0 : 1;
          float* ws = p.workspace + ((size_t)blockIdx.x * 2 + my_slot) * slot_elems;
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            if (j < valid) {
              ws[(size_t)j * F8_TILE_F + r] = accg[j];
              if (DUAL) ws[(size_t)(NT + j) * F8_TILE_F + r] = accu[j];
            }
          }
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            const int nc = c_last - c_first + 1;
            const int old = atomicAdd(&p.counters[c_first], 1);
            const int last = (old == nc - 1);
            if (last) p.counters[c_first] = 0;
            epi_last = last;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          do_final = epi_last != 0;
          if (do_final) __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (do_final) {
#pragma unroll
            for (int j = 0; j < NT; ++j) { accg[j] = 0.f; if (DUAL) accu[j] = 0.f; }
            for (int c = c_first; c <= c_last; ++c) {
              const int slot = ((long long)c * sched.per) / KB == u ? 0 : 1;
              const float* wsr = p.workspace + ((size_t)c * 2 + slot) * slot_elems;
#pragma unroll
              for (int j = 0; j < NT; ++j) {
                if (j < valid) {
                  accg[j] += __ldcg(&wsr[(size_t)j * F8_TILE_F + r]);
                  if (DUAL) accu[j] += __ldcg(&wsr[(size_t)(NT + j) * F8_TILE_F + r]);
                }
              }
            }
          }
        }
        if (do_final && f_ok) {
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            if (j < valid) {
              float y = accg[j];
              if (DUAL) y = silu(y) * accu[j];
              const size_t idx = (size_t)(row0 + j) * p.ldo + p.out_col0 + f;
              if (p.residual) y += __bfloat162float(((const __nv_bfloat16*)p.residual)[idx]);
              const __nv_bfloat16 yb = __float2bfloat16(y);
              ((__nv_bfloat16*)p.out)[idx] = yb;
            }
          }
        }
        pos = (long long)u * KB + kb1;
      }
    }
  }

  // publish: local stores ordered device-wide, then one system-scope fence by the last CTA (see gemm_ws.cu)
  if (p.mode == 2 && warp >= 2) {
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 64) {
      const int old = atomicAdd(p.done_counter, 1);
      if (old == (int)gridDim.x - 1) {
        *p.done_counter = 0;
        __threadfence_system();
        const int e = *p.epoch + 1;
        if (p.status == nullptr || p.status[0] == 0)
          for (int pe = 0; pe < p.n_peers; ++pe) st_relaxed_sys(p.peer_flag[pe], e);
        *p.epoch = e;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <bool DUAL, int NT>
static int launch_f8(const CUtensorMap& tmW, const CUtensorMap& tmX, const F8Args& ka, int grid, size_t smem, cudaStream_t s) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_ws_fp8_kernel<DUAL, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_ws_fp8_kernel<DUAL, NT><<<grid, F8_THREADS, smem, s>>>(tmW, tmX, ka);
  return (int)cudaGetLastError();
}

}  // namespace skein

// mode 0 store, 1 SwiGLU pair (dual), 2 store + publish flags to peers. n_tile in {16, 32, 64} (dual: {16, 32}).
extern "C" int skein_gemm_ws_fp8(const SkeinGemmParams* p, void* stream) {
  using namespace skein;
  if (!p || p->G < 1 || p->G > SKEIN_MAX_GROUPS) return -1;
  if (p->K <= 0 || p->K % 128 != 0) return -2;
  const bool dual = p->mode == 1;
  if (!(p->n_tile == 16 || p->n_tile == 32 || (p->n_tile == 64 && !dual))) return -3;
  if (p->mode < 0 || p->mode > 2) return -4;
  if (p->mode == 2 && (p->n_peers < 1 || p->n_peers > SKEIN_MAX_PEERS)) return -5;
  if (!p->w_scale || !p->x_scale || !p->workspace || !p->counters) return -8;
  F8Args ka;
  ka.p = *p;
  ka.p.fp8 = 1;
  ka.x_tile_bytes = p->n_tile * 128;
  ka.stage_bytes = (dual ? 2 : 1) * F8_W_TILE_BYTES + ka.x_tile_bytes;
  int st = (200 * 1024) / ka.stage_bytes;
  if (st > F8_MAX_STAGES) st = F8_MAX_STAGES;
  if (p->stages > 0 && p->stages < st) st = p->stages;
  if (st < 2) return -7;
  ka.stages = st;
  const int acc = (dual ? 2 : 1) * p->n_tile;
  ka.buf_cols = acc < 32 ? 32 : acc;
  ka.n_bufs = 512 / ka.buf_cols;
  if (ka.n_bufs > F8_MAX_BUFS) ka.n_bufs = F8_MAX_BUFS;
  ka.budget_ns = (uint64_t)(p->wait_budget_ms > 0 ? p->wait_budget_ms : gemm_wait_budget_ms()) * 1000000ull;
  const int grid = p->grid > 0 ? p->grid : skein_sm_count();
  const size_t smem = (size_t)st * ka.stage_bytes + 1024;
  CUtensorMap tmW, tmX;
  int rc = cached_tmap_2d(&tmW, p->W, (uint64_t)p->G * p->w_rows_per_group, p->K, 1, F8_TILE_F);
  if (rc) return rc;
  rc = cached_tmap_2d(&tmX, p->X, p->x_rows, p->K, 1, p->n_tile);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (dual) {
    if (p->n_tile == 16) return launch_f8<true, 16>(tmW, tmX, ka, grid, smem, s);
    return launch_f8<true, 32>(tmW, tmX, ka, grid, smem, s);
  }
  if (p->n_tile == 16) return launch_f8<false, 16>(tmW, tmX, ka, grid, smem, s);
  if (p->n_tile == 32) return launch_f8<false, 32>(tmW, tmX, ka, grid, smem, s);
  return launch_f8<false, 64>(tmW, tmX, ka, grid, smem, s);
}
