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
//     token tile, or a store of the partial result into a peer-mapped local buffer followed by a
//     release of this rank's flag on every tensor-parallel peer (the all-reduce is finished by the
//     consumer, which pulls the partials over NVLink: see norm.cu, reduce_residual_rmsnorm).
//   * block-scaled fp8 weights with bf16 activations (the plan's weight fp8_e4m3 / activation bf16 combination):
//     the weight tile travels as e4m3 (half the bytes of the decode step's dominant traffic), eight more warps
//     turn each landed tile into bf16, multiplying every row by its 1 x 128 block scale on the way, and write it
//     into TENSOR MEMORY, from where the tensor cores take it as the A operand of the same bf16 MMAs (the token
//     tile stays in shared memory), accumulating into ONE accumulator for the whole K range. Nothing is drained
//     per K block, the activations are not quantised, and shared memory carries only the e4m3 bytes: with a bf16
//     copy of the tile in shared memory the kernel was bound by shared-memory bandwidth (tile written by TMA, read
//     and written again by the conversion, read by the MMA), not by HBM.
//
// Replaces the reference's cuBLASLt matmul host op (vendor/luminal/crates/luminal_cuda_lite/src/
// host/cublaslt/mod.rs:888-1130), its fp8 GEMV (same file :797-886) and the GLUMoE GEMV kernels
// (host/moe/mod.rs:229-381) with one tensor-core kernel.
#include "gemm_ws.cuh"
#include "gemm_sched.cuh"
#include "ptx.cuh"
#include "launch.cuh"
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <stdio.h>

namespace skein {

constexpr int TILE_F = 128;       // output features per tile (UMMA M)
constexpr int BLOCK_KB = 128;     // bytes of K per stage row (64 bf16 or 128 e4m3)
constexpr int W_TILE_BYTES = TILE_F * BLOCK_KB;  // 16 KB
constexpr int ACC_STRIDE_MAX = 256;   // TMEM columns per accumulator buffer, at most
constexpr int NUM_THREADS = 192;
constexpr int W8_CONV_THREADS = 256;
constexpr int W8_THREADS = NUM_THREADS + W8_CONV_THREADS;   // + 8 converter warps (e4m3 -> scaled bf16 in shared memory)
constexpr int EPI_THREADS = 128;
constexpr int MAX_STAGES = 12;
constexpr int W8_CONV_SLOTS = 3;  // ring of converted half K-blocks in tensor memory (64 K elements = 32 columns per weight tile)
constexpr int W8_SLOT_COLS = 32;  // 32-bit columns of one converted weight tile half: 64 bf16 K elements, two per column

// Optional phase timer (compile with -DSKEIN_GEMM_TIMING): every CTA records %globaltimer at the points marked
// TS(i) below into g_gemm_times[cta][i]; skein_gemm_times() copies the table out. Points: 0 entry, 1 set-up done,
// 2 first stage landed (MMA warp), 3 first accumulator ready (epilogue), 4 partial parked and counted in,
// 5 all contributors seen, 6 slice reduced and stored, 7 before TMEM release.
#ifdef SKEIN_GEMM_TIMING
__device__ unsigned long long g_gemm_times[160][8];
#define TS(i) do { g_gemm_times[blockIdx.x][i] = global_timer_ns(); } while (0)
// Cycle accounting of the e4m3-weight pipeline, per CTA: [0] converter waits for a landed stage, [1] converter waits
// for a free converted slot, [2] converter converts, [3] MMA thread waits for a converted half, [4] MMA thread issues,
// [5] producer waits for a free stage, [6] half K-blocks processed.
__device__ unsigned long long g_w8_prof[160][8];
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(i) do { g_w8_prof[blockIdx.x][i] += (unsigned long long)(clock64() - prof_t0_); } while (0)
#else
#define TS(i) do { } while (0)
#define PROF_T0() do { } while (0)
#define PROF_ADD(i) do { } while (0)
#endif

struct KernelArgs {
  SkeinGemmParams p;
  int acc_stride;   // TMEM columns per accumulator buffer: power of two >= (dual ? 2 : 1) * n_tile, at least 32
  int stages;
  int stage_bytes;
  int x_tile_bytes;
  int conv_base;    // W8: first tensor-memory column of the converted-tile ring (behind the two accumulators)
  int conv_slots;   // W8: slots of that ring
  int scale_off;    // W8: byte offset, inside a stage, of the tile's block scales (128 floats per weight tile)
  uint64_t budget_ns;
};

// Four e4m3 bytes of `w` -> four bf16 values times the block scale, without a conversion instruction. An e4m3 byte
// s eeee mmm, moved to s 0000eeee mmm0000, is a bf16 number whose value is the e4m3 value times 2^-120, subnormals
// and zero included (both formats count their subnormals from the same exponent field value 0). One bf16x2
// multiplication by (block scale * 2^120) therefore yields the scaled weight; it is exact when the scale is a
// power of two, which is how this framework quantises weights (ops/fp8.py: quantize_weight).
// Per pair of values: one byte permute that also spreads each byte's sign over the byte above it (S:b per 16-bit
// half), one shift left by 4 (sign at bit 15, the seven exponent / mantissa bits at 10..4), one mask that drops the
// spare sign copies and what the shift carried over from the lower half, one multiplication.
// (The hardware conversion e4m3x2 -> f16x2 would be cheaper still, but the MMA then needs f16 for BOTH operands: an f16
// A operand with bf16 activations is not a legal operand pair of kind::f16.)
__device__ __forceinline__ void e4m3x4_to_scaled_bf16x4(uint32_t w, uint32_t sc2, uint32_t& lo, uint32_t& hi) {
  uint32_t t0, t1;
  asm("prmt.b32 %0, %1, 0, 0x9180;" : "=r"(t0) : "r"(w));   // [sign(b1), b1, sign(b0), b0]
  asm("prmt.b32 %0, %1, 0, 0xB3A2;" : "=r"(t1) : "r"(w));   // [sign(b3), b3, sign(b2), b2]
  const uint32_t r0 = (t0 << 4) & 0x87F087F0u;
  const uint32_t r1 = (t1 << 4) & 0x87F087F0u;
  // spelled out so that no fast-math flag turns it into a form that flushes the subnormal inputs
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(r0), "r"(sc2));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(r1), "r"(sc2));
}

template <bool DUAL, bool W8>
__global__ void __launch_bounds__(W8 ? W8_THREADS : NUM_THREADS, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
               const KernelArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ Sched sched;
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_cfull[W8_CONV_SLOTS];    // W8: a converted half K-block is ready for the MMA warp
  __shared__ __align__(8) uint64_t bar_cempty[W8_CONV_SLOTS];   // W8: the MMAs that read it are done
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
  // Nothing before pdl_wait() touches global memory: barriers, TMEM and the descriptor prefetch overlap the
  // tail of the previous kernel in the stream (launch.cuh).
  pdl_trigger();
  if (threadIdx.x == 0) {
    TS(0);
    abort_flag = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), EPI_THREADS);
    }
    if (W8) {
      for (int c = 0; c < a.conv_slots; ++c) {
        mbar_init(smem_u32(&bar_cfull[c]), W8_CONV_THREADS);
        mbar_init(smem_u32(&bar_cempty[c]), 1);
      }
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), W8 ? 512 : 2 * a.acc_stride);
    tmem_relinquish();
  }
  if (warp == 0 && elect_one()) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  pdl_wait();
  if (threadIdx.x == 0) build_sched(sched, p, W8 ? 128 : 64, (int)gridDim.x, p.line_cut_only == 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  if (threadIdx.x == 0) TS(1);

  const int KB = sched.KB;
  const int kb_begin = cta_begin(sched, blockIdx.x);
  const int kb_end = cta_end(sched, blockIdx.x);
  const bool has_work = kb_begin < kb_end;
  const int n_tile = p.n_tile;
  const int k_elems = W8 ? 128 : 64;
  constexpr int W_STAGE_BYTES = (DUAL ? 2 : 1) * W_TILE_BYTES;   // weight bytes of one stage (bf16: 64 K, e4m3: 128 K)
  // W8: one converter -> MMA hand-over per stage. A slot of the tensor-memory ring holds the whole converted K block of the
  // stage as pairs of 32-column sub-tiles: with a gate/up pair, (gate, up) of K half 0 then of K half 1; else the two K
  // halves of the one tile.
  constexpr int W8_PAIRS = DUAL ? 2 : 1;
  constexpr int W8_SLOT = W8_PAIRS * 2 * W8_SLOT_COLS;

  if (has_work) {
    if (warp == 0) {
      // ================= TMA producer =================
      if (elect_one()) {
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        uint32_t tx_bytes = (DUAL ? 2 : 1) * W_TILE_BYTES + a.x_tile_bytes;
        const uint32_t tx_base = tx_bytes;
        const long long w_rows_total = (long long)p.G * p.w_rows_per_group;
        uint32_t it = 0;
        int pos = kb_begin;
        bool ok = true;
        while (pos < kb_end && ok) {
          const int u = pos / KB;
          const int kb0 = pos - u * KB;
          int kb1 = KB;
          if (u * KB + KB > kb_end) kb1 = kb_end - u * KB;
          const Unit un = decode_unit(sched, p.G, u);
          const int w_row = un.g * p.w_rows_per_group + un.m * TILE_F;
          const int x_row = sched.off[un.g] + un.n * n_tile;
          // W8: the 128 block scales of each weight tile travel with the stage (512 bytes per tile), unless the tile
          // sticks out of the matrix; the converters then read the few scales they need themselves
          const bool scales_by_copy = W8 && (w_row + (DUAL ? p.up_row_off : 0) + TILE_F <= w_rows_total) &&
                                      (un.m * TILE_F + TILE_F <= p.F) && (w_rows_total % 4 == 0) && (p.up_row_off % 4 == 0);
          if (W8) tx_bytes = tx_base + (scales_by_copy ? (DUAL ? 2 : 1) * 512u : 0u);
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s = it % a.stages;
            const uint32_t ph = (it / a.stages) & 1;
            {
              PROF_T0();
              if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, a.budget_ns)) {
                report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, blockIdx.x);
                abort_flag = 1;
                ok = false;
                break;
              }
              if (W8) PROF_ADD(5);
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
            tma_load_2d(st + W_STAGE_BYTES, &tmX, full, kb * k_elems, x_row, pol_x);
            // e4m3 weights: a stage covers 128 K elements, i.e. two 64-wide bf16 activation tiles
            if (W8) {
              tma_load_2d(st + W_STAGE_BYTES + a.x_tile_bytes / 2, &tmX, full, kb * k_elems + 64, x_row, pol_x);
              if (scales_by_copy) {
                const float* sp = p.w_scale + (size_t)kb * w_rows_total + w_row;
                bulk_load_1d(st + a.scale_off, sp, 512, full);
                if (DUAL) bulk_load_1d(st + a.scale_off + 512, sp + p.up_row_off, 512, full);
              }
            }
          }
          pos = u * KB + kb1;
        }
      }
    } else if (warp == 1) {
      // ================= MMA issuer =================
      if (elect_one()) {
        const uint32_t idesc = umma_idesc(1, 1, TILE_F, n_tile);
        uint32_t it = 0;
        uint32_t seg = 0;
        int pos = kb_begin;
        bool ok = true;
        while (pos < kb_end && ok) {
          const int u = pos / KB;
          const int kb0 = pos - u * KB;
          int kb1 = KB;
          if (u * KB + KB > kb_end) kb1 = kb_end - u * KB;
          const uint32_t b = seg & 1;
          const uint32_t bph = (seg >> 1) & 1;
          if (!mbar_wait(smem_u32(&bar_tempty[b]), bph ^ 1, &abort_flag, a.budget_ns)) {
            report_status(p.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x);
            abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + b * a.acc_stride;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s = it % a.stages;
            const uint32_t ph = (it / a.stages) & 1;
            const uint32_t st = smem_base + s * a.stage_bytes;
            if (W8) {
              // the converted weights of this stage arrive from the converter warps in one slot of the tensor-memory ring
              const uint32_t c = it % a.conv_slots, cph = (it / a.conv_slots) & 1;
              {
                PROF_T0();
                if (!mbar_wait(smem_u32(&bar_cfull[c]), cph, &abort_flag, a.budget_ns)) {
                  report_status(p.status, ST_TIMEOUT_SMEM_FULL, blockIdx.x);
                  abort_flag = 1;
                  ok = false;
                  break;
                }
                PROF_ADD(3);
              }
              PROF_T0();
              tc_fence_after();
              if (it == 0) TS(2);
              const uint32_t aw = tmem_base + a.conv_base + c * W8_SLOT;
#pragma unroll
              for (int h = 0; h < 2; ++h) {          // K halves of the stage: 64 K elements = 4 MMAs of 16 (8 columns of A each)
                const uint64_t dx = umma_desc_sw128(st + W_STAGE_BYTES + h * (a.x_tile_bytes / 2));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint32_t accum = (kb > kb0 || h > 0 || k > 0) ? 1u : 0u;
                  if (DUAL) {
                    mma_f16_ts(d_tmem, aw + h * 2 * W8_SLOT_COLS + 8 * k, dx + 2 * k, idesc, accum);
                    mma_f16_ts(d_tmem + n_tile, aw + (h * 2 + 1) * W8_SLOT_COLS + 8 * k, dx + 2 * k, idesc, accum);
                  } else {
                    mma_f16_ts(d_tmem, aw + h * W8_SLOT_COLS + 8 * k, dx + 2 * k, idesc, accum);
                  }
                }
              }
              tc_commit(smem_u32(&bar_cempty[c]));
              PROF_ADD(4);
              if (!ok) break;
              tc_commit(smem_u32(&bar_empty[s]));  // the activation tiles of the stage have been read as well
              continue;
            }
            if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_FULL, blockIdx.x);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
            if (it == 0) TS(2);
            const uint64_t dw = umma_desc_sw128(st);
            const uint64_t dx = umma_desc_sw128(st + W_STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte row
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              mma_f16(d_tmem, dw + 2 * k, dx + 2 * k, idesc, accum);
              if (DUAL) {
                const uint64_t du = umma_desc_sw128(st + W_TILE_BYTES);
                mma_f16(d_tmem + n_tile, du + 2 * k, dx + 2 * k, idesc, accum);
              }
            }
            tc_commit(smem_u32(&bar_empty[s]));  // frees the stage when these MMAs are done
          }
          if (!ok) break;
          tc_commit(smem_u32(&bar_tfull[b]));
          ++seg;
          pos = u * KB + kb1;
        }
      }
    } else if (W8 && warp >= 6) {
      // ================= converters (warps 6..13): e4m3 tile -> bf16 rows, scaled by the row's 1 x 128 block scale, in TMEM ==
      // Two threads share weight row r of the tile, each taking two of the four 16-byte chunks of a 64-K half (eight
      // warps: two per scheduler, so that one warp's dependent instructions are covered by the other's). The raw tile
      // was written by TMA with the 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)). A warp can
      // reach the tensor-memory lanes 32 * (warp % 4) .. + 31 only, and lane = row of the A operand, so a warp converts
      // the rows of its own lane quarter; 16 K elements become 8 columns.
      const int r = (warp & 3) * 32 + lane;
      const int part = (warp - 6) >> 2;                      // which two chunks of every half this thread converts
      const long long w_rows_total = (long long)p.G * p.w_rows_per_group;
      uint32_t it = 0;
      int pos = kb_begin;
      bool ok = true;
      // The hand-over of a converted half to the MMA warp is deferred by one step: its tensor-memory stores complete
      // while the next half is loaded and converted, so the wait for them costs nothing when it finally comes.
      int pending_slot = -1;
      while (pos < kb_end && ok) {
        const int u = pos / KB;
        const int kb0 = pos - u * KB;
        int kb1 = KB;
        if (u * KB + KB > kb_end) kb1 = kb_end - u * KB;
        const Unit un = decode_unit(sched, p.G, u);
        const long long w_row = (long long)un.g * p.w_rows_per_group + un.m * TILE_F + r;
        const bool scales_by_copy = ((long long)un.g * p.w_rows_per_group + un.m * TILE_F + (DUAL ? p.up_row_off : 0) + TILE_F <= w_rows_total) &&
                                    (un.m * TILE_F + TILE_F <= p.F) && (w_rows_total % 4 == 0) && (p.up_row_off % 4 == 0);
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
          const uint32_t s = it % a.stages, ph = (it / a.stages) & 1;
          {
            PROF_T0();
            if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_FULL, blockIdx.x);
              abort_flag = 1;
              ok = false;
              break;
            }
            if (r == 0 && part == 0) PROF_ADD(0);
          }
          // shared-memory addresses (32-bit, shared state space): loads and stores below are ld.shared / st.shared, not
          // generic accesses, which the hardware tracks like global ones (they showed up as the kernel's dominant stall)
          const uint32_t raw = smem_base + s * a.stage_bytes;
          uint32_t sc[DUAL ? 2 : 1];     // the row's block scale times 2^120 as a packed bf16 pair
#pragma unroll
          for (int t = 0; t < (DUAL ? 2 : 1); ++t) {
            const long long row = w_row + (t ? p.up_row_off : 0);
            float f;
            if (scales_by_copy)     // arrived with the stage
              asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(raw + a.scale_off + (t * 128 + r) * 4));
            else  // a tile that sticks out of the matrix: rows beyond it were zero-filled by TMA, any finite scale will do
              f = (row < w_rows_total && (un.m * TILE_F + r) < p.F) ? __ldg(p.w_scale + (size_t)kb * w_rows_total + row) : 0.f;
            const __nv_bfloat162 hs = __float2bfloat162_rn(f * 0x1p120f);
            sc[t] = *reinterpret_cast<const uint32_t*>(&hs);
          }
          const uint32_t c = it % a.conv_slots, cph = (it / a.conv_slots) & 1;
          {
            PROF_T0();
            if (!mbar_wait(smem_u32(&bar_cempty[c]), cph ^ 1, &abort_flag, a.budget_ns)) {
              report_status(p.status, ST_TIMEOUT_SMEM_EMPTY, blockIdx.x);
              abort_flag = 1;
              ok = false;
              break;
            }
            if (r == 0 && part == 0) PROF_ADD(1);
          }
          PROF_T0();
          tc_fence_after();
#pragma unroll
          for (int h = 0; h < W8_PAIRS; ++h) {
            // this thread's 16 columns of its lane in each of the pair's two sub-tiles: slot c, pair h, sub-tile t, columns
            // part * 16 .. + 15. Sub-tile t is tile t (gate / up) at K half h with a pair of tiles, else K half t of the one tile.
            const uint32_t conv = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + a.conv_base + c * W8_SLOT +
                                  h * 2 * W8_SLOT_COLS + part * 16;
            uint32_t o[2][16];
            uint4 v[2][2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const uint32_t src_row = raw + (DUAL ? t : 0) * W_TILE_BYTES + r * 128;
              const int half = DUAL ? h : t;
#pragma unroll
              for (int ci = 0; ci < 2; ++ci)             // this thread's 16-byte chunks of e4m3, all loads first
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v[t][ci].x), "=r"(v[t][ci].y), "=r"(v[t][ci].z), "=r"(v[t][ci].w)
                             : "r"(src_row + (((half * 4 + part * 2 + ci) ^ (r & 7)) << 4)));
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const uint32_t sct = sc[DUAL ? t : 0];
#pragma unroll
              for (int ci = 0; ci < 2; ++ci) {
                e4m3x4_to_scaled_bf16x4(v[t][ci].x, sct, o[t][8 * ci + 0], o[t][8 * ci + 1]);
                e4m3x4_to_scaled_bf16x4(v[t][ci].y, sct, o[t][8 * ci + 2], o[t][8 * ci + 3]);
                e4m3x4_to_scaled_bf16x4(v[t][ci].z, sct, o[t][8 * ci + 4], o[t][8 * ci + 5]);
                e4m3x4_to_scaled_bf16x4(v[t][ci].w, sct, o[t][8 * ci + 6], o[t][8 * ci + 7]);
              }
            }
            if (h == 0 && pending_slot >= 0) {
              // the previous stage's stores to tensor memory have had this conversion to complete
              tmem_st_wait();
              tc_fence_before();
              mbar_arrive(smem_u32(&bar_cfull[pending_slot]));
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) tmem_st16(conv + t * W8_SLOT_COLS, o[t]);
          }
          pending_slot = (int)c;
#ifdef SKEIN_GEMM_TIMING
          if (r == 0 && part == 0) { PROF_ADD(2); g_w8_prof[blockIdx.x][6] += 1; }
#endif
        }
        pos = u * KB + kb1;
      }
      if (pending_slot >= 0) {
        // (also on the way out after a failed wait: the MMA warp gives up on the abort flag, an extra arrival is harmless)
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_cfull[pending_slot]));
      }
    } else if (warp < 6) {
      // ================= epilogue (warps 2..5) =================
      const int q = warp & 3;                 // TMEM lane quarter this warp may read
      const int r = q * 32 + lane;            // feature row inside the tile
      const int et = threadIdx.x - 64;        // 0..127
      const int acc_cols = (DUAL ? 2 : 1) * n_tile;
      const size_t slot_elems = (size_t)TILE_F * acc_cols;
      // final value of one output element: activation pair, residual, store (locally or into every peer)
      auto emit = [&](float g, float u, long long row, int f) {
        float y = g;
        if (DUAL) y = silu(g) * u;
        const size_t idx = (size_t)row * p.ldo + p.out_col0 + f;
        if (p.residual) y += __bfloat162float(((const __nv_bfloat16*)p.residual)[idx]);
        const __nv_bfloat16 yb = __float2bfloat16(y);
        ((__nv_bfloat16*)p.out)[idx] = yb;
      };
      // Stream-K tiles that several CTAs share: every contributor parks its fp32 partial and counts itself
      // in (phase 1, inside the loop); once its own work is done it waits for the tile's other
      // contributors and reduces ITS slice of the tile's rows from all partials, in contributor order
      // (phase 2). The reduction is spread over the contributors instead of falling on the last to arrive,
      // and the result does not depend on timing. All CTAs of the grid are resident (one per SM), so
      // the wait cannot starve; it is bounded all the same.
      int ps_u[2] = {0, 0};
      int n_pseg = 0;
      uint32_t seg = 0;
      int pos = kb_begin;
      bool ok = true;
      while (pos < kb_end && ok) {
        const int u = pos / KB;
        const int kb0 = pos - u * KB;
        int kb1 = KB;
        if (u * KB + KB > kb_end) kb1 = kb_end - u * KB;
        const bool full_seg = (kb0 == 0 && kb1 == KB);
        const Unit un = decode_unit(sched, p.G, u);
        const uint32_t b = seg & 1;
        const uint32_t bph = (seg >> 1) & 1;
        if (!mbar_wait(smem_u32(&bar_tfull[b]), bph, &abort_flag, a.budget_ns)) {
          report_status(p.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x);
          abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        if (et == 0 && seg == 0) TS(3);
        const uint32_t t_acc = tmem_base + b * a.acc_stride + ((uint32_t)(q * 32) << 16);
        int valid = sched.cnt[un.g] - un.n * n_tile;
        if (valid > n_tile) valid = n_tile;
        const int f = un.m * TILE_F + r;
        const bool f_ok = f < p.F;
        const long long row0 = (long long)sched.off[un.g] + (long long)un.n * n_tile;

        if (!full_seg) {
          // ---- phase 1: park the fp32 partial, count this CTA in ----
          int c_first, c_last_unused;
          tile_ctas(sched, u, c_first, c_last_unused);
          const int my_slot = cta_slot(sched, blockIdx.x, u);
          float* ws = p.workspace + ((size_t)blockIdx.x * 2 + my_slot) * slot_elems;
          // two 16-column chunks per round: both TMEM loads are issued before the one wait
          for (int c0 = 0; c0 < acc_cols; c0 += 32) {
            // skip column chunks that hold only padding tokens
            const int cc0 = DUAL ? (c0 >= n_tile ? c0 - n_tile : c0) : c0;
            const int c1 = c0 + 16;
            const int cc1 = DUAL ? (c1 >= n_tile ? c1 - n_tile : c1) : c1;
            const bool do0 = cc0 < valid, do1 = c1 < acc_cols && cc1 < valid;
            uint32_t v0[16], v1[16];
            if (do0) tmem_ld16(t_acc + c0, v0);
            if (do1) tmem_ld16(t_acc + c1, v1);
            tmem_ld_wait();
            if (do0) {
#pragma unroll
              for (int j = 0; j < 16; ++j)   // column-major partials [col][feature]: a warp writes 128 contiguous bytes
                ws[(size_t)(c0 + j) * TILE_F + r] = __uint_as_float(v0[j]);
            }
            if (do1) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                ws[(size_t)(c1 + j) * TILE_F + r] = __uint_as_float(v1[j]);
            }
          }
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[b]));
          // the barrier orders the 128 threads' partial stores before thread 0's device-scope release, which
          // publishes them (cumulatively) to the CTA that later acquires the counter
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(&p.counters[c_first]) : "memory");
          if (et == 0) TS(4);
          if (n_pseg < 2) ps_u[n_pseg] = u;
          ++n_pseg;
        } else {
          for (int c0 = 0; c0 < n_tile; c0 += 16) {
            if (c0 >= valid) break;
            uint32_t v[16], w[16];
            tmem_ld16(t_acc + c0, v);
            if (DUAL) tmem_ld16(t_acc + n_tile + c0, w);
            tmem_ld_wait();
            if (f_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + j >= valid) break;
                emit(__uint_as_float(v[j]), DUAL ? __uint_as_float(w[j]) : 0.f, row0 + c0 + j, f);
              }
            }
          }
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[b]));
        }
        ++seg;
        pos = u * KB + kb1;
      }

      // ---- phase 2: reduce this CTA's slice of every tile it shares ----
      for (int si = 0; si < n_pseg && si < 2 && ok; ++si) {
        const int u = ps_u[si];
        const Unit un = decode_unit(sched, p.G, u);
        int c_first, c_last;
        tile_ctas(sched, u, c_first, c_last);
        const int nc = c_last - c_first + 1;
        const int first_slot = cta_slot(sched, c_first, u);   // (64-bit divisions: once per tile, not per load)
        int valid = sched.cnt[un.g] - un.n * n_tile;
        if (valid > n_tile) valid = n_tile;
        const long long row0 = (long long)sched.off[un.g] + (long long)un.n * n_tile;
        if (et == 0) {
          // the low half of the counter holds arrivals, the high half departures
          int arrived = 0;
          const uint64_t t0 = global_timer_ns();
          for (;;) {
            arrived = ld_acquire_sys(&p.counters[c_first]) & 0xffff;
            if (arrived >= nc || abort_flag) break;
            if (global_timer_ns() - t0 > a.budget_ns) break;
          }
          if (arrived < nc) {
            report_status(p.status, ST_TIMEOUT_SPLITK, blockIdx.x);
            abort_flag = 1;
          }
          epi_last = arrived >= nc;
          TS(5);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool go = epi_last != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // epi_last is rewritten for the next tile
        if (!go) { ok = false; break; }
        // slices are whole groups of 8 features, so that a thread sums 8 consecutive features of one token
        // (two 16-byte loads per contributor) and stores them with one 16-byte access
        const int rows_per = ((TILE_F + nc - 1) / nc + 7) & ~7;
        const int r_lo = ((int)blockIdx.x - c_first) * rows_per;
        int r_hi = r_lo + rows_per;
        if (r_hi > TILE_F) r_hi = TILE_F;
        const int n_grp = r_hi > r_lo ? (r_hi - r_lo) / 8 : 0;
        const int n_items = n_grp * valid;
        const bool wide_ok = (p.ldo % 8 == 0) && (p.out_col0 % 8 == 0);
        // one item = 8 consecutive features of one token column
        auto store_item = [&](int rr, int col, const float* g8, const float* u8) {
          const int f0 = un.m * TILE_F + rr;
          const long long row = row0 + col;
          if (wide_ok && f0 + 8 <= p.F) {
            const size_t idx = (size_t)row * p.ldo + p.out_col0 + f0;
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = DUAL ? silu(g8[j]) * u8[j] : g8[j];
            if (p.residual) {
              const uint4 rv = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.residual + idx);
              const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
              for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(rb[j]); y[2 * j] += t.x; y[2 * j + 1] += t.y; }
            }
            uint4 o;
            __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
            *reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + idx) = o;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (f0 + j < p.F) emit(g8[j], u8[j], row, f0 + j);
          }
        };
        // IPB items of a thread are reduced together, CB = 8 / IPB contributors per batch: 16 (32 with the up half)
        // 16-byte loads are in flight per thread whatever the number of contributors, and a tile cut in two
        // costs one L2 round trip per 4 items instead of one per item. Contributors are added in rank order.
        auto reduce_items = [&](auto ipb_c) {
          constexpr int IPB = decltype(ipb_c)::value;
          constexpr int CB = 8 / IPB;
          for (int i0 = et; i0 < n_items; i0 += EPI_THREADS * IPB) {
            int rr[IPB], col[IPB];
            bool live[IPB];
            float g8[IPB][8], u8[IPB][8];
#pragma unroll
            for (int k = 0; k < IPB; ++k) {
              const int i = i0 + k * EPI_THREADS;
              live[k] = i < n_items;
              rr[k] = r_lo + (i % n_grp) * 8;     // consecutive threads -> consecutive feature groups
              col[k] = i / n_grp;                 // token column (< valid)
#pragma unroll
              for (int j = 0; j < 8; ++j) { g8[k][j] = 0.f; u8[k][j] = 0.f; }
            }
            for (int cb = c_first; cb <= c_last; cb += CB) {
              float4 tg[IPB][CB][2], tu[IPB][CB][2];
#pragma unroll
              for (int k = 0; k < IPB; ++k) {
#pragma unroll
                for (int ci = 0; ci < CB; ++ci) {
                  const int c = cb + ci;
                  tg[k][ci][0] = tg[k][ci][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                  if (DUAL) tu[k][ci][0] = tu[k][ci][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                  if (live[k] && c <= c_last) {
                    // every contributor but possibly the first begins inside this tile and used its slot 0
                    const int slot = (c == c_first) ? first_slot : 0;
                    const float* ws = p.workspace + ((size_t)c * 2 + slot) * slot_elems + (size_t)col[k] * TILE_F + rr[k];
                    tg[k][ci][0] = __ldcg(reinterpret_cast<const float4*>(ws));
                    tg[k][ci][1] = __ldcg(reinterpret_cast<const float4*>(ws + 4));
                    if (DUAL) {
                      tu[k][ci][0] = __ldcg(reinterpret_cast<const float4*>(ws + (size_t)n_tile * TILE_F));
                      tu[k][ci][1] = __ldcg(reinterpret_cast<const float4*>(ws + (size_t)n_tile * TILE_F + 4));
                    }
                  }
                }
              }
#pragma unroll
              for (int k = 0; k < IPB; ++k) {
#pragma unroll
                for (int ci = 0; ci < CB; ++ci) {   // fixed summation order
                  g8[k][0] += tg[k][ci][0].x; g8[k][1] += tg[k][ci][0].y; g8[k][2] += tg[k][ci][0].z; g8[k][3] += tg[k][ci][0].w;
                  g8[k][4] += tg[k][ci][1].x; g8[k][5] += tg[k][ci][1].y; g8[k][6] += tg[k][ci][1].z; g8[k][7] += tg[k][ci][1].w;
                  if (DUAL) {
                    u8[k][0] += tu[k][ci][0].x; u8[k][1] += tu[k][ci][0].y; u8[k][2] += tu[k][ci][0].z; u8[k][3] += tu[k][ci][0].w;
                    u8[k][4] += tu[k][ci][1].x; u8[k][5] += tu[k][ci][1].y; u8[k][6] += tu[k][ci][1].z; u8[k][7] += tu[k][ci][1].w;
                  }
                }
              }
            }
#pragma unroll
            for (int k = 0; k < IPB; ++k)
              if (live[k]) store_item(rr[k], col[k], g8[k], u8[k]);
          }
        };
        if (!DUAL && nc <= 2) reduce_items(std::integral_constant<int, 4>{});
        else if (!DUAL && nc <= 4) reduce_items(std::integral_constant<int, 2>{});
        else reduce_items(std::integral_constant<int, 1>{});
        // count this CTA out; the last one out re-arms the counter for the next launch
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) TS(6);
        if (et == 0) {
          const int old = atomicAdd(&p.counters[c_first], 0x10000);
          if ((old >> 16) == nc - 1) p.counters[c_first] = 0;
        }
      }
    }
  }

  // ---- tensor-parallel publish: the last CTA to finish sets this rank's flag on every peer -------
  // The result sits in local memory that the peers have mapped; they pull it once they see the flag. Every
  // epilogue thread orders its stores device-wide, the CTAs count themselves in, and the last one issues the
  // single system-scope fence that orders all of those stores before the flag words it then writes.
  if (p.mode == 2) {
    if (warp >= 2 && warp < 6) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int old = atomicAdd(p.done_counter, 1);
        if (old == (int)gridDim.x - 1) {
          *p.done_counter = 0;
          __threadfence_system();   // orders every CTA's stores (observed through the counter) before the flags
          const int e = *p.epoch + 1;
          // a failed launch publishes nothing: the consumers' bounded waits then report it
          if (p.status == nullptr || p.status[0] == 0) {
            for (int pe = 0; pe < p.n_peers; ++pe) st_relaxed_sys(p.peer_flag[pe], e);
          }
          *p.epoch = e;
        }
      }
    }
  }

  // ---- tear-down --------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TS(7);
  if (abort_flag) {
    // let TMA copies that are still in flight land before the shared memory is given back
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, W8 ? 512 : 2 * a.acc_stride);
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
  const bool w8 = p->fp8 == 2;   // e4m3 weights with 1 x 128 block scales, bf16 activations
  const int kelem = w8 ? 128 : 64;
  if (p->K <= 0 || p->K % kelem != 0) return -2;
  const bool dual = p->mode == 1;
  if (p->n_tile < 16 || p->n_tile % 16 != 0 || p->n_tile > (dual ? 128 : 256)) return -3;
  if (p->mode < 0 || p->mode > 2) return -4;
  if (p->mode == 2 && (p->n_peers < 1 || p->n_peers > SKEIN_MAX_PEERS)) return -5;
  if (p->fp8 == 1) return -6;  // e4m3 x e4m3 with both operands block-scaled goes through skein_gemm_ws_fp8
  if (w8 && (p->w_scale == nullptr || p->w_packed)) return -6;
  ka->p = *p;
  {
    const int acc_cols = (dual ? 2 : 1) * p->n_tile;
    int st = 32;
    while (st < acc_cols) st <<= 1;
    if (st > ACC_STRIDE_MAX) return -3;
    ka->acc_stride = st;   // two buffers: 64..512 columns, a power of two as the allocator requires
  }
  ka->x_tile_bytes = p->n_tile * BLOCK_KB * (w8 ? 2 : 1);    // e4m3 stage: 128 K elements = two bf16 activation tiles
  ka->stage_bytes = (dual ? 2 : 1) * W_TILE_BYTES + ka->x_tile_bytes;
  ka->scale_off = ka->stage_bytes;
  if (w8) ka->stage_bytes += 1024;                            // the weight tiles' block scales (keeps the 1 KB alignment)
  const int budget = 200 * 1024;
  ka->conv_base = 0;
  ka->conv_slots = 0;
  if (w8) {
    // the converted weights live in tensor memory behind the two accumulators: 512 columns in all
    // a slot holds one stage's converted K block: 64 columns per weight tile of the stage
    const int slot_cols = (dual ? 2 : 1) * 2 * W8_SLOT_COLS;
    ka->conv_base = 2 * ka->acc_stride;
    ka->conv_slots = (512 - ka->conv_base) / slot_cols;
    if (ka->conv_slots > W8_CONV_SLOTS) ka->conv_slots = W8_CONV_SLOTS;
    if (ka->conv_slots < 2) return -3;   // token tile too wide for this form
  }
  int st = budget / ka->stage_bytes;
  if (st > MAX_STAGES) st = MAX_STAGES;
  if (p->stages > 0 && p->stages < st) st = p->stages;
  if (st < 2) return -7;
  ka->stages = st;
  ka->budget_ns = (uint64_t)(p->wait_budget_ms > 0 ? p->wait_budget_ms : gemm_wait_budget_ms()) * 1000000ull;
  *grid = p->grid > 0 ? p->grid : sm_count_cached();
  if (*grid > sm_count_cached()) *grid = sm_count_cached();   // the split-K reduction needs every CTA resident
  *smem = (size_t)st * ka->stage_bytes + 1024;
  return 0;
}

}  // namespace skein

extern "C" int skein_sm_count(void) { return skein::sm_count_cached(); }

#ifdef SKEIN_GEMM_TIMING
// out: [160][8] nanosecond stamps of the last launch (synchronises the device).
extern "C" int skein_gemm_times(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, skein::g_gemm_times, sizeof(unsigned long long) * 160 * 8);
}
// out: [160][8] cycle totals of the e4m3-weight pipeline since the last call, which also clears them.
extern "C" int skein_w8_profile(unsigned long long* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, skein::g_w8_prof, sizeof(unsigned long long) * 160 * 8);
  if (e != cudaSuccess) return (int)e;
  static unsigned long long zeros[160 * 8];
  return (int)cudaMemcpyToSymbol(skein::g_w8_prof, zeros, sizeof(zeros));
}
#endif

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
  const bool w8 = p->fp8 == 2;
  if (p->w_packed) {
    if (p->w_rows_per_group % TILE_F != 0 || (p->mode == 1 && p->up_row_off % TILE_F != 0)) return -9;
    const uint64_t tiles = (uint64_t)p->G * (p->w_rows_per_group / TILE_F) * (p->K / 64);
    rc = cached_tmap_2d(&tmW, p->W, tiles * TILE_F, 64, 2, TILE_F);
  } else {
    rc = cached_tmap_2d(&tmW, p->W, (uint64_t)p->G * p->w_rows_per_group, p->K, w8 ? 1 : 2, TILE_F);
  }
  if (rc) return rc;
  rc = cached_tmap_2d(&tmX, p->X, p->x_rows, p->K, 2, p->n_tile);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static bool attr_done[4] = {false, false, false, false};
  const bool dual = p->mode == 1;
  const int variant = (w8 ? 2 : 0) + (dual ? 1 : 0);
  auto with_kernel = [&](auto fn) -> cudaError_t {
    if (!attr_done[variant]) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048);
      if (e != cudaSuccess) return e;
      attr_done[variant] = true;
    }
    return launch_pdl(fn, dim3(grid), dim3(w8 ? W8_THREADS : NUM_THREADS), smem, s, tmW, tmX, ka);
  };
  switch (variant) {
    case 0: return (int)with_kernel(gemm_ws_kernel<false, false>);
    case 1: return (int)with_kernel(gemm_ws_kernel<true, false>);
    case 2: return (int)with_kernel(gemm_ws_kernel<false, true>);
    default: return (int)with_kernel(gemm_ws_kernel<true, true>);
  }
}
