// Weight-streaming GEMM for sm_100a: Y[t, f] = sum_k X[t, k] * W[f, k], optionally grouped
// (one weight matrix per expert, ragged token lists whose sizes live in device memory).
//
// Shape of the kernel
//   * "swap-AB": the weight tile (128 output features x 64 K) is the M-side operand of
//     tcgen05.mma, the token tile (n_tile tokens x 64 K) is the N side, so a decode batch of a few
//     dozen tokens still fills the 128-row tensor-core tile and every weight byte is read once.
//   * persistent, one CTA per SM, stream-K: the K-blocks of all tiles form one line that is cut
//     into equal contiguous pieces, one per CTA. A tile covered by several CTAs is summed by the
//     last of them to arrive (fp32 partials in a workspace, fixed summation order, so the result
//     does not depend on timing).
//   * warp roles: warp 0 issues TMA loads into a multi-stage shared-memory ring, warp 1 issues
//     tcgen05.mma into one of two TMEM accumulators, warps 2-5 drain the other accumulator
//     (tcgen05.ld), apply the epilogue and store.
//   * epilogues: plain store (+ residual), SwiGLU of a gate/up pair of weight tiles that share the
//     token tile, or a store of the partial result into every tensor-parallel peer's buffer
//     followed by a release of that peer's flag (the all-reduce is finished by the consumer,
//     see norm.cu: reduce_residual_rmsnorm).
//
// Replaces the reference's cuBLASLt matmul host op (vendor/luminal/crates/luminal_cuda_lite/src/
// host/cublaslt/mod.rs:888-1130), its fp8 GEMV (same file :797-886) and the GLUMoE GEMV kernels
// (host/moe/mod.rs:229-381) with one tensor-core kernel.
#include "gemm_ws.cuh"
#include "gemm_sched.cuh"
#include "ptx.cuh"
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>
#include <stdio.h>

namespace skein {

constexpr int TILE_F = 128;       // output features per tile (UMMA M)
constexpr int BLOCK_KB = 128;     // bytes of K per stage row (64 bf16 or 128 e4m3)
constexpr int W_TILE_BYTES = TILE_F * BLOCK_KB;  // 16 KB
constexpr int ACC_STRIDE = 256;   // TMEM columns per accumulator buffer
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int MAX_STAGES = 12;

struct KernelArgs {
  SkeinGemmParams p;
  int stages;
  int stage_bytes;
  int x_tile_bytes;
  uint64_t budget_ns;
};

template <bool DUAL>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
               const KernelArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ Sched sched;
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ int epi_last;

  const SkeinGemmParams& p = a.p;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // dynamic shared memory is only guaranteed 16-byte aligned by the runtime: align by hand
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  // ---- set-up ---------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    abort_flag = 0;
    build_sched(sched, p, p.fp8 ? 128 : 64, (int)gridDim.x);
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), EPI_THREADS);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  const int KB = sched.KB;
  const long long kb_begin = (long long)blockIdx.x * sched.per;
  long long kb_end = kb_begin + sched.per;
  if (kb_end > sched.TK) kb_end = sched.TK;
  const bool has_work = kb_begin < sched.TK;
  const int n_tile = p.n_tile;
  const int k_elems = p.fp8 ? 128 : 64;

  if (has_work) {
    if (warp == 0) {
      // ================= TMA producer =================
      if (elect_one()) {
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        const uint32_t tx_bytes = (DUAL ? 2 : 1) * W_TILE_BYTES + a.x_tile_bytes;
        uint32_t it = 0;
        long long pos = kb_begin;
        bool ok = true;
        while (pos < kb_end && ok) {
          const int u = (int)(pos / KB);
          const int kb0 = (int)(pos - (long long)u * KB);
          int kb1 = KB;
          if ((long long)u * KB + KB > kb_end) kb1 = (int)(kb_end - (long long)u * KB);
          const Unit un = decode_unit(sched, p.G, u);
          const int w_row = un.g * p.w_rows_per_group + un.m * TILE_F;
          const int x_row = sched.off[un.g] + un.n * n_tile;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s = it % a.stages;
            const uint32_t ph = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, blockIdx.x);
              abort_flag = 1;
              ok = false;
              break;
            }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t st = smem_base + s * a.stage_bytes;
            mbar_expect_tx(full, tx_bytes);
            if (p.w_packed) {
              // tile-packed weights: tile (row tile, kb) is one contiguous 16 KB block
              tma_load_2d(st, &tmW, full, 0, ((w_row / TILE_F) * KB + kb) * TILE_F, pol_w);
              if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, full, 0, (((w_row + p.up_row_off) / TILE_F) * KB + kb) * TILE_F, pol_w);
            } else {
              tma_load_2d(st, &tmW, full, kb * k_elems, w_row, pol_w);
              if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, full, kb * k_elems, w_row + p.up_row_off, pol_w);
            }
            tma_load_2d(st + (DUAL ? 2 : 1) * W_TILE_BYTES, &tmX, full, kb * k_elems, x_row, pol_x);
          }
          pos = (long long)u * KB + kb1;
        }
      }
    } else if (warp == 1) {
      // ================= MMA issuer =================
      if (elect_one()) {
        const uint32_t idesc = p.fp8 ? umma_idesc(0, 0, TILE_F, n_tile) : umma_idesc(1, 1, TILE_F, n_tile);
        uint32_t it = 0;
        uint32_t seg = 0;
        long long pos = kb_begin;
        bool ok = true;
        while (pos < kb_end && ok) {
          const int u = (int)(pos / KB);
          const int kb0 = (int)(pos - (long long)u * KB);
          int kb1 = KB;
          if ((long long)u * KB + KB > kb_end) kb1 = (int)(kb_end - (long long)u * KB);
          const uint32_t b = seg & 1;
          const uint32_t bph = (seg >> 1) & 1;
          if (!mbar_wait(smem_u32(&bar_tempty[b]), bph ^ 1, &abort_flag, a.budget_ns)) {
            report_status(p.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x);
            abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * ACC_STRIDE;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s = it % a.stages;
            const uint32_t ph = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_FULL, blockIdx.x);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t st = smem_base + s * a.stage_bytes;
            const uint64_t dw = umma_desc_sw128(st);
            const uint64_t dx = umma_desc_sw128(st + (DUAL ? 2 : 1) * W_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte row
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              if (p.fp8) mma_f8(d_tmem, dw + 2 * k, dx + 2 * k, idesc, accum);
              else mma_f16(d_tmem, dw + 2 * k, dx + 2 * k, idesc, accum);
              if (DUAL) {
                const uint64_t du = umma_desc_sw128(st + W_TILE_BYTES);
                if (p.fp8) mma_f8(d_tmem + n_tile, du + 2 * k, dx + 2 * k, idesc, accum);
                else mma_f16(d_tmem + n_tile, du + 2 * k, dx + 2 * k, idesc, accum);
              }
            }
            tc_commit(smem_u32(&bar_empty[s]));  // frees the stage when these MMAs are done
          }
          if (!ok) break;
          tc_commit(smem_u32(&bar_tfull[b]));
          ++seg;
          pos = (long long)u * KB + kb1;
        }
      }
    } else {
      // ================= epilogue (warps 2..5) =================
      const int q = warp & 3;                 // TMEM lane quarter this warp may read
      const int r = q * 32 + lane;            // feature row inside the tile
      const int et = threadIdx.x - 64;        // 0..127
      const int acc_cols = (DUAL ? 2 : 1) * n_tile;
      const size_t slot_elems = (size_t)TILE_F * acc_cols;
      uint32_t seg = 0;
      long long pos = kb_begin;
      bool ok = true;
      while (pos < kb_end && ok) {
        const int u = (int)(pos / KB);
        const int kb0 = (int)(pos - (long long)u * KB);
        int kb1 = KB;
        if ((long long)u * KB + KB > kb_end) kb1 = (int)(kb_end - (long long)u * KB);
        const bool full_seg = (kb0 == 0 && kb1 == KB);
        const Unit un = decode_unit(sched, p.G, u);
        const uint32_t b = seg & 1;
        const uint32_t bph = (seg >> 1) & 1;
        if (!mbar_wait(smem_u32(&bar_tfull[b]), bph, &abort_flag, a.budget_ns)) {
          report_status(p.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t t_acc = tmem_base + b * ACC_STRIDE + ((uint32_t)(q * 32) << 16);
        int valid = sched.cnt[un.g] - un.n * n_tile;
        if (valid > n_tile) valid = n_tile;
        const int f = un.m * TILE_F + r;
        const bool f_ok = f < p.F;
        const long long row0 = (long long)sched.off[un.g] + (long long)un.n * n_tile;

        bool do_final = full_seg;
        int c_first = 0, c_last = 0;
        if (!full_seg) {
          // ---- stream-K partial: park the fp32 tile, count arrivals, last one finishes ----
          const long long ub = (long long)u * KB;
          c_first = (int)(ub / sched.per);
          c_last = (int)((ub + KB - 1) / sched.per);
          const int my_slot = ((long long)blockIdx.x * sched.per) / KB == u ? 0 : 1;
          float* ws = p.workspace + ((size_t)blockIdx.x * 2 + my_slot) * slot_elems;
          for (int c0 = 0; c0 < acc_cols; c0 += 16) {
            // skip column chunks that hold only padding tokens
            const int cc = DUAL ? (c0 >= n_tile ? c0 - n_tile : c0) : c0;
            if (cc >= valid) continue;
            uint32_t v[16];
            tmem_ld16(t_acc + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j += 4)   // row-major partials: 16-byte accesses, few instructions on the fix-up path
              *reinterpret_cast<uint4*>(&ws[(size_t)r * acc_cols + c0 + j]) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[b]));
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
          // all 128 threads must have read epi_last before a later segment overwrites it
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }

        if (do_final) {
          for (int c0 = 0; c0 < n_tile; c0 += 16) {
            if (c0 >= valid) break;
            float g16[16], u16[16];
            if (full_seg) {
              uint32_t v[16];
              tmem_ld16(t_acc + c0, v);
              if (DUAL) {
                uint32_t w[16];
                tmem_ld16(t_acc + n_tile + c0, w);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) u16[j] = __uint_as_float(w[j]);
              } else {
                tmem_ld_wait();
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) g16[j] = __uint_as_float(v[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) { g16[j] = 0.f; u16[j] = 0.f; }
              // contributors are read four at a time so that 64+ loads are in flight per thread
              for (int cb = c_first; cb <= c_last; cb += 4) {
                float tg[4][16], tu[4][16];
#pragma unroll
                for (int ci = 0; ci < 4; ++ci) {
                  const int c = cb + ci;
                  if (c <= c_last) {
                    const int slot = ((long long)c * sched.per) / KB == u ? 0 : 1;
                    const float* ws = p.workspace + ((size_t)c * 2 + slot) * slot_elems;
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                      const float4 a4 = __ldcg(reinterpret_cast<const float4*>(&ws[(size_t)r * acc_cols + c0 + j]));
                      tg[ci][j] = a4.x; tg[ci][j + 1] = a4.y; tg[ci][j + 2] = a4.z; tg[ci][j + 3] = a4.w;
                      if (DUAL) {
                        const float4 b4 = __ldcg(reinterpret_cast<const float4*>(&ws[(size_t)r * acc_cols + n_tile + c0 + j]));
                        tu[ci][j] = b4.x; tu[ci][j + 1] = b4.y; tu[ci][j + 2] = b4.z; tu[ci][j + 3] = b4.w;
                      }
                    }
                  } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) { tg[ci][j] = 0.f; if (DUAL) tu[ci][j] = 0.f; }
                  }
                }
#pragma unroll
                for (int ci = 0; ci < 4; ++ci)
#pragma unroll
                  for (int j = 0; j < 16; ++j) { g16[j] += tg[ci][j]; if (DUAL) u16[j] += tu[ci][j]; }
              }
            }
            if (f_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + j >= valid) break;
                float y = g16[j];
                if (DUAL) y = silu(y) * u16[j];
                const size_t idx = (size_t)(row0 + c0 + j) * p.ldo + p.out_col0 + f;
                if (p.residual) y += __bfloat162float(((const __nv_bfloat16*)p.residual)[idx]);
                const __nv_bfloat16 yb = __float2bfloat16(y);
                if (p.mode == 2) {
                  for (int pe = 0; pe < p.n_peers; ++pe) ((__nv_bfloat16*)p.peer_out[pe])[idx] = yb;
                } else {
                  ((__nv_bfloat16*)p.out)[idx] = yb;
                }
              }
            }
          }
        }
        if (full_seg) {
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[b]));
        }
        ++seg;
        pos = (long long)u * KB + kb1;
      }
    }
  }

  // ---- tensor-parallel push: the last CTA to finish publishes this rank's flag on every peer ---
  if (p.mode == 2) {
    if (warp >= 2) {
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int old = atomicAdd(p.done_counter, 1);
        if (old == (int)gridDim.x - 1) {
          *p.done_counter = 0;
          __threadfence_system();
          const int e = *p.epoch + 1;
          // a failed launch publishes nothing: the consumers' bounded waits then report it
          if (p.status == nullptr || p.status[0] == 0) {
            for (int pe = 0; pe < p.n_peers; ++pe) st_release_sys(p.peer_flag[pe], e);
          }
          *p.epoch = e;
        }
      }
    }
  }

  // ---- tear-down --------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // let TMA copies that are still in flight land before the shared memory is given back
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D row-major tensor [rows, k_elems] of 1- or 2-byte elements; box = [box_rows, 128 bytes].
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes,
                 uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return -11;
  if ((k_elems * elem_bytes) % 16 != 0) return -12;
  cuuint64_t dims[2] = {k_elems, rows};
  cuuint64_t strides[1] = {k_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -13;
}

struct TmapKey {
  const void* base; uint64_t rows, k; int eb; uint32_t box;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && k == o.k && eb == o.eb && box == o.box;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.k * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (size_t)k.box * 0x165667B19E3779F9ull + k.eb;
    return h;
  }
};

int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes,
                   uint32_t box_rows) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{base, rows, k_elems, elem_bytes, box_rows};
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  int rc = make_tmap_2d(out, base, rows, k_elems, elem_bytes, box_rows);
  if (rc == 0) {
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
  }
  return rc;
}

static int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static int plan(const SkeinGemmParams* p, KernelArgs* ka, int* grid, size_t* smem) {
  if (!p || p->G < 1 || p->G > SKEIN_MAX_GROUPS) return -1;
  const int kelem = p->fp8 ? 128 : 64;
  if (p->K <= 0 || p->K % kelem != 0) return -2;
  const bool dual = p->mode == 1;
  if (p->n_tile < 16 || p->n_tile % 16 != 0 || p->n_tile > (dual ? 128 : 256)) return -3;
  if (p->mode < 0 || p->mode > 2) return -4;
  if (p->mode == 2 && (p->n_peers < 1 || p->n_peers > SKEIN_MAX_PEERS)) return -5;
  if (p->fp8) return -6;  // block-scaled e4m3 goes through skein_gemm_ws_fp8
  ka->p = *p;
  ka->x_tile_bytes = p->n_tile * BLOCK_KB;
  ka->stage_bytes = (dual ? 2 : 1) * W_TILE_BYTES + ka->x_tile_bytes;
  const int budget = 200 * 1024;
  int st = budget / ka->stage_bytes;
  if (st > MAX_STAGES) st = MAX_STAGES;
  if (p->stages > 0 && p->stages < st) st = p->stages;
  if (st < 2) return -7;
  ka->stages = st;
  ka->budget_ns = (uint64_t)(p->wait_budget_ms > 0 ? p->wait_budget_ms : 2000) * 1000000ull;
  *grid = p->grid > 0 ? p->grid : sm_count_cached();
  *smem = (size_t)st * ka->stage_bytes + 1024;
  return 0;
}

}  // namespace skein

extern "C" int skein_sm_count(void) { return skein::sm_count_cached(); }

extern "C" int64_t skein_gemm_ws_workspace_bytes(const SkeinGemmParams* p) {
  const int grid = p->grid > 0 ? p->grid : skein::sm_count_cached();
  const int acc_cols = (p->mode == 1 ? 2 : 1) * p->n_tile;
  return (int64_t)grid * 2 * skein::TILE_F * acc_cols * (int64_t)sizeof(float);
}

extern "C" int skein_gemm_ws(const SkeinGemmParams* p, void* stream) {
  using namespace skein;
  KernelArgs ka;
  int grid = 0;
  size_t smem = 0;
  int rc = plan(p, &ka, &grid, &smem);
  if (rc) return rc;
  if (!p->workspace || !p->counters) return -8;
  CUtensorMap tmW, tmX;
  const int eb = p->fp8 ? 1 : 2;
  if (p->w_packed) {
    if (p->w_rows_per_group % TILE_F != 0 || (p->mode == 1 && p->up_row_off % TILE_F != 0)) return -9;
    const uint64_t tiles = (uint64_t)p->G * (p->w_rows_per_group / TILE_F) * (p->K / (p->fp8 ? 128 : 64));
    rc = cached_tmap_2d(&tmW, p->W, tiles * TILE_F, p->fp8 ? 128 : 64, eb, TILE_F);
  } else {
    rc = cached_tmap_2d(&tmW, p->W, (uint64_t)p->G * p->w_rows_per_group, p->K, eb, TILE_F);
  }
  if (rc) return rc;
  rc = cached_tmap_2d(&tmX, p->X, p->x_rows, p->K, eb, p->n_tile);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static bool attr_done[2] = {false, false};
  const bool dual = p->mode == 1;
  if (!attr_done[dual]) {
    cudaError_t e = dual ? cudaFuncSetAttribute(gemm_ws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048)
                         : cudaFuncSetAttribute(gemm_ws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048);
    if (e != cudaSuccess) return (int)e;
    attr_done[dual] = true;
  }
  if (dual) gemm_ws_kernel<true><<<grid, NUM_THREADS, smem, s>>>(tmW, tmX, ka);
  else gemm_ws_kernel<false><<<grid, NUM_THREADS, smem, s>>>(tmW, tmX, ka);
  return (int)cudaGetLastError();
}
