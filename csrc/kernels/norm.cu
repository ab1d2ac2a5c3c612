// Residual add + RMSNorm, with the reduction half of the tensor-parallel all-reduce and the MoE
// top-k combine folded in.
//
// One kernel covers every "sum things into the residual stream, then normalise" point of a
// decoder block:
//   acc[h] = residual[b, h]
//          + sum over sources s (the tensor-parallel ranks' partial results: slots of a local tensor, or
//            every rank's own peer-mapped buffer, pulled over NVLink; 1 on a single GPU)
//              of   partial[s][b, h]                                   (dense: attention o_proj)
//              or   sum_j weight[b, j] * partial[s][row[b, j], h]      (MoE: rows are in
//                                                                       expert-sorted order)
//   residual_out[b, h] = bf16(acc[h])
//   normed_out[b, h]   = bf16(residual_out[b, h] * rsqrt(mean(residual_out^2) + eps) * gamma[h])
// When sources are other GPUs the kernel first waits (bounded) until every source's flag has
// reached this buffer's current epoch, then reads the peers' buffers with plain loads, or, when the
// buffers are bound to an NVLink multicast object, with one in-switch reducing load per 16 bytes.
//
// Replaces the reference's unfused rms_norm graph (crates/skein_emit/src/op_wiring.rs:1787), its
// elementwise residual adds and the NCCL all-reduce + copy-back
// (crates/skein_runtime/src/cuda/nccl.rs:196-245).
#include "ptx.cuh"
#include "launch.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

struct NormParams {
  const __nv_bfloat16* residual;   // [B, H] or null (treated as zero)
  const __nv_bfloat16* partial;    // [n_src][rows][H] or null
  const __nv_bfloat16* src_base[8];  // with use_ptrs: source s is the [rows][H] buffer at src_base[s] (a peer's memory,
                                   // read over NVLink) instead of partial + s * src_stride
  int use_ptrs;
  const __nv_bfloat16* mc_base;    // non-null: the multicast mapping of the same [rows][H] buffer on all n_src ranks; the
                                   // sum over ranks then is ONE multimem.ld_reduce per 16 bytes (added inside the
                                   // NVSwitch, fp32 accumulation) instead of n_src peer loads
  const int* row_idx;              // [B, topk] rows into partial, or null (row = b)
  const float* row_w;              // [B, topk] weights, or null
  const int* owner_ids;            // [B, topk] expert id of each pair, or null: with it only the sources that own the
                                   // expert are read: ranks (id / experts_per_owner) * owner_span .. + owner_span - 1
  const __nv_bfloat16* gamma;      // [H] or null (no normalisation, normed_out unused)
  __nv_bfloat16* residual_out;     // [B, H] or null
  __nv_bfloat16* normed_out;       // [B, H] or null
  const int* flags;                // [n_src] flags written by the sources, or null
  const int* epoch;                // device int: epoch the flags must reach
  int* status;
  long long src_stride;            // elements between sources in `partial`
  int B, H, n_src, topk;
  int experts_per_owner, owner_span;
  float eps;
  unsigned long long budget_ns;
};

__device__ __forceinline__ float block_sum(float v, float* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < nw) ? sh[l] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// One CTA per token row; each thread owns 8 consecutive elements per pass (16-byte accesses).
// Returns false when the row produced no normalised output (a peer wait ran out, or no gamma);
// otherwise nb[ps] holds the thread's 8 normalised bf16 values of pass ps. Uniform over the CTA.
template <int MAX_PASSES>
__device__ __forceinline__ bool reduce_norm_row(const NormParams& p, const int b, float* sh, int& wait_failed,
                                                uint4 (&nb)[MAX_PASSES]) {
  if (p.flags != nullptr) {
    // row 0's CTA records how long it stood waiting for the peers (exposed communication time): a 64-bit
    // nanosecond total in status[2..3], read by the host together with the status word
    const uint64_t t_wait0 = (b == 0 && threadIdx.x == 0) ? global_timer_ns() : 0;
    if (threadIdx.x == 0) wait_failed = 0;
    __syncthreads();
    if ((int)threadIdx.x < p.n_src) {
      const int e = *p.epoch;
      // a peer wait that already ran out poisons the step: later kernels give up at once instead of
      // spending their own budget, so a lost rank costs one budget, not one per kernel
      const bool poisoned = p.status != nullptr && *(volatile int*)p.status == ST_TIMEOUT_PEER_FLAG;
      if (poisoned || !wait_flag_ge(p.flags + threadIdx.x, e, p.budget_ns)) {
        report_status(p.status, ST_TIMEOUT_PEER_FLAG, threadIdx.x);
        wait_failed = 1;
      }
    }
    __syncthreads();
    if (b == 0 && threadIdx.x == 0 && p.status != nullptr)
      atomicAdd(reinterpret_cast<unsigned long long*>(p.status + 2), (unsigned long long)(global_timer_ns() - t_wait0));
    if (wait_failed) return false;
  }
  float vals[MAX_PASSES][8];
  float ss = 0.f;
  const int per_pass = blockDim.x * 8;
#pragma unroll
  for (int ps = 0; ps < MAX_PASSES; ++ps) {
    const int h = ps * per_pass + threadIdx.x * 8;
    if (h >= p.H) break;
    float a[8];
    if (p.residual) {
      const uint4 r = *reinterpret_cast<const uint4*>(p.residual + (size_t)b * p.H + h);
      const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(rb[i]); a[2 * i] = f.x; a[2 * i + 1] = f.y; }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = 0.f;
    }
    if (p.partial || p.use_ptrs) {
      const int nk = p.topk > 0 ? p.topk : 1;
      // the (row, weight, owner) triples of up to 8 slots are fetched together, ahead of the data loads
      int rows8[8], own8[8];
      float w8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        rows8[j] = (j < nk) ? (p.row_idx ? p.row_idx[b * p.topk + j] : b) : -1;
        w8[j] = (j < nk && p.row_w) ? p.row_w[b * p.topk + j] : 1.f;
        own8[j] = (j < nk && p.owner_ids) ? p.owner_ids[b * p.topk + j] : 0;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // top-k is at most 8 (host-checked)
        if (j >= nk) break;
        const int row = rows8[j];
        if (row < 0) continue;  // pair routed to an expert that lives on another rank
        const float w = w8[j];
        int s_lo = 0, s_hi = p.n_src;
        if (p.owner_ids) {
          s_lo = (own8[j] / p.experts_per_owner) * p.owner_span;
          s_hi = s_lo + p.owner_span;
          if (s_lo < 0 || s_hi > p.n_src) continue;
        }
        if (p.mc_base != nullptr && p.owner_ids == nullptr) {
          const uint4 r = multimem_ld_reduce_add_bf16x8(p.mc_base + (size_t)row * p.H + h);
          const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(rb[i]); a[2 * i] += w * f.x; a[2 * i + 1] += w * f.y; }
          continue;
        }
        // sources in batches of 8: every load of a batch is issued before the first is consumed (the partials of
        // 8 tensor-parallel ranks would otherwise cost 8 dependent round trips); the sum order stays s_lo..s_hi
        for (int s0 = s_lo; s0 < s_hi; s0 += 8) {
          uint4 r8[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            r8[u] = make_uint4(0, 0, 0, 0);
            if (s0 + u < s_hi) {
              const __nv_bfloat16* src = (p.use_ptrs ? p.src_base[s0 + u] : p.partial + (size_t)(s0 + u) * p.src_stride) +
                                         (size_t)row * p.H + h;
              // data written by other GPUs: bypass L1
              asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(r8[u].x), "=r"(r8[u].y), "=r"(r8[u].z), "=r"(r8[u].w) : "l"(src));
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (s0 + u < s_hi) {
              const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r8[u]);
#pragma unroll
              for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(rb[i]); a[2 * i] += w * f.x; a[2 * i + 1] += w * f.y; }
            }
          }
        }
      }
    }
    // the residual stream is bf16: round first, normalise the rounded value
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ob[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
      const float2 f = __bfloat1622float2(ob[i]);
      vals[ps][2 * i] = f.x; vals[ps][2 * i + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
    if (p.residual_out) *reinterpret_cast<uint4*>(p.residual_out + (size_t)b * p.H + h) = o;
  }
  if (p.gamma == nullptr || p.normed_out == nullptr) return false;
  const float tot = block_sum(ss, sh);
  const float inv = rsqrtf(tot / (float)p.H + p.eps);
#pragma unroll
  for (int ps = 0; ps < MAX_PASSES; ++ps) {
    const int h = ps * per_pass + threadIdx.x * 8;
    if (h >= p.H) break;
    const uint4 g = *reinterpret_cast<const uint4*>(p.gamma + h);
    const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&g);
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 gf = __bfloat1622float2(gb[i]);
      // match the usual bf16 pipeline: round x*inv to bf16, then scale by gamma
      const __nv_bfloat162 xn = __floats2bfloat162_rn(vals[ps][2 * i] * inv, vals[ps][2 * i + 1] * inv);
      const float2 xf = __bfloat1622float2(xn);
      ob[i] = __floats2bfloat162_rn(xf.x * gf.x, xf.y * gf.y);
    }
    *reinterpret_cast<uint4*>(p.normed_out + (size_t)b * p.H + h) = o;
    nb[ps] = o;
  }
  return true;
}

template <int MAX_PASSES>
__global__ void __launch_bounds__(512) reduce_residual_rmsnorm_kernel(const NormParams p) {
  __shared__ float sh[32];
  __shared__ int wait_failed;
  uint4 nb[MAX_PASSES];
  pdl_trigger();
  pdl_wait();
  reduce_norm_row<MAX_PASSES>(p, blockIdx.x, sh, wait_failed, nb);
}

// ---------------------------------------------------------------------------------------------
// The same row reduction followed, in the same launch, by the MoE router and the scatter of the
// normalised row into expert-sorted order (decode steps: every token's CTA is resident at once).
//
//   1. reduce + residual + RMSNorm of row t (above), the normalised row stays in registers
//   2. logits[e] = normed . Wg[e] (bf16-rounded like a linear layer), top-k with ties to the lower
//      expert index, softmax over the selected k; expert_ids / expert_w of the token are published
//   3. a grid-wide arrival counter (bounded wait): every CTA then knows all T*k choices
//   4. every CTA derives the expert-sorted layout (counts, exclusive offsets; pair (t, j) sits at
//      offsets[e] + number of earlier pairs routed to e, which is the stable order the stand-alone
//      router kernel produces) and writes its own row to xs[row] for each of its k experts
// The host only launches this when T CTAs of 512 threads fit on the device at once.
// ---------------------------------------------------------------------------------------------
constexpr int NR_MAX_E = 64;
constexpr int NR_MAX_K = 8;
constexpr int NR_MAX_PAIRS = 2048;

struct RouteParams {
  const __nv_bfloat16* wg;   // [E, H]
  int* expert_ids;           // [T, k]
  float* expert_w;           // [T, k]
  int* counts;               // [E]
  int* offsets;              // [E + 1]
  int* row_of;               // [T * k]   (-1: expert not on this rank)
  int* src_token;            // [T * k]
  __nv_bfloat16* xs;         // [T * k, H] rows in expert-sorted order
  int* barrier;              // [2] arrive / depart, zero between launches
  int E, topk, e_first, e_count;
  unsigned long long barrier_budget_ns;
};

template <int MAX_PASSES>
__global__ void __launch_bounds__(512) reduce_norm_route_kernel(const NormParams p, const RouteParams r) {
  __shared__ float sh[32];
  __shared__ int wait_failed;
  __shared__ float part[16][NR_MAX_E];
  __shared__ float logit[NR_MAX_E];
  __shared__ int ids_s[NR_MAX_PAIRS];
  __shared__ int cnt_s[NR_MAX_E], bef_s[NR_MAX_E], off_s[NR_MAX_E + 1];
  __shared__ int my_row[NR_MAX_K];
  __shared__ int barrier_ok;
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const int T = gridDim.x, E = r.E, topk = r.topk;
  uint4 nb[MAX_PASSES];
  pdl_trigger();
  pdl_wait();
  const bool have_row = reduce_norm_row<MAX_PASSES>(p, t, sh, wait_failed, nb);
  // a row that failed still takes part in the barrier below, so that the other CTAs do not wait for it
  const int per_pass = blockDim.x * 8;
  for (int e0 = 0; e0 < E; e0 += 8) {
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
    if (have_row) {
#pragma unroll
      for (int ps = 0; ps < MAX_PASSES; ++ps) {
        const int h = ps * per_pass + tid * 8;
        if (h >= p.H) break;
        uint4 wr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          wr[i] = (e0 + i < E) ? *reinterpret_cast<const uint4*>(r.wg + (size_t)(e0 + i) * p.H + h) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&nb[ps]);
        float xf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(xb[i]); xf[2 * i] = f.x; xf[2 * i + 1] = f.y; }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wr[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(wb[j]); a[i] += xf[2 * j] * f.x + xf[2 * j + 1] * f.y; }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = a[i];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && e0 + i < E) part[warp][e0 + i] = v;
    }
  }
  __syncthreads();
  if (tid < E) {
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v += part[w][tid];
    logit[tid] = __bfloat162float(__float2bfloat16(v));
  }
  __syncthreads();
  if (tid == 0) {
    int ids[NR_MAX_K];
    float vals[NR_MAX_K];
    for (int j = 0; j < topk; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        bool taken = false;
        for (int q = 0; q < j; ++q) taken |= (ids[q] == e);
        if (!taken && (best < 0 || logit[e] > bv)) { best = e; bv = logit[e]; }
      }
      ids[j] = best; vals[j] = bv;
    }
    float den = 0.f;
    const float vmax = vals[0];
    for (int j = 0; j < topk; ++j) { vals[j] = __expf(vals[j] - vmax); den += vals[j]; }
    for (int j = 0; j < topk; ++j) {
      r.expert_ids[t * topk + j] = ids[j];
      r.expert_w[t * topk + j] = vals[j] / den;
    }
    // release at device scope: this thread's stores of the expert ids / weights above are visible to whoever acquires
    // the counter (one instruction instead of a full fence followed by a relaxed add)
    asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(r.barrier) : "memory");
    // grid-wide arrival, bounded: all T CTAs are resident, so this only runs out if one never started
    const bool poisoned = p.status != nullptr && *(volatile int*)p.status == ST_TIMEOUT_GRID_BARRIER;
    const bool ok = !poisoned && wait_counter_ge_gpu(r.barrier, T, r.barrier_budget_ns);
    if (!ok) report_status(p.status, ST_TIMEOUT_GRID_BARRIER, t);
    barrier_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!barrier_ok) return;   // the counters stay dirty: the host clears them when it handles the status
  const int n_pairs = T * topk;
  for (int i = tid; i < n_pairs; i += blockDim.x) ids_s[i] = __ldcg(r.expert_ids + i);
  __syncthreads();
  const int my_first = t * topk;
  for (int e = warp; e < E; e += nwarps) {
    int c = 0, before = 0;
    for (int i0 = 0; i0 < n_pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n_pairs && ids_s[i] == e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
      before += __popc(__ballot_sync(0xffffffffu, hit && i < my_first));
    }
    if (lane == 0) {
      cnt_s[e] = (e >= r.e_first && e < r.e_first + r.e_count) ? c : 0;
      bef_s[e] = before;
    }
  }
  __syncthreads();
  if (tid == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) { off_s[e] = a; a += cnt_s[e]; }
    off_s[E] = a;
    if (t == 0) {
      for (int e = 0; e < E; ++e) { r.counts[e] = cnt_s[e]; r.offsets[e] = off_s[e]; }
      r.offsets[E] = a;
    }
    for (int j = 0; j < topk; ++j) {
      const int e = ids_s[my_first + j];
      const bool mine = e >= r.e_first && e < r.e_first + r.e_count;
      const int row = mine ? off_s[e] + bef_s[e] : -1;   // a token's k experts are distinct
      my_row[j] = row;
      r.row_of[my_first + j] = row;
      if (row >= 0) r.src_token[row] = t;
    }
  }
  __syncthreads();
  if (have_row && r.xs != nullptr) {
#pragma unroll
    for (int ps = 0; ps < MAX_PASSES; ++ps) {
      const int h = ps * per_pass + tid * 8;
      if (h >= p.H) break;
      for (int j = 0; j < topk; ++j) {
        const int row = my_row[j];
        if (row >= 0) *reinterpret_cast<uint4*>(r.xs + (size_t)row * p.H + h) = nb[ps];
      }
    }
  }
  if (tid == 0) {
    const int old = atomicAdd(r.barrier + 1, 1);
    if (old == T - 1) { r.barrier[0] = 0; r.barrier[1] = 0; }   // every CTA is past the wait: re-arm
  }
}

}  // namespace skein

extern "C" int skein_reduce_residual_rmsnorm(
    const void* residual, const void* partial, const int* row_idx, const float* row_w, const void* gamma,
    void* residual_out, void* normed_out, const int* flags, const int* epoch, int* status,
    long long src_stride, int B, int H, int n_src, int topk, float eps, int wait_budget_ms, const int* owner_ids,
    int experts_per_owner, int owner_span, const void* const* src_ptrs, const void* mc_base, void* stream) {
  using namespace skein;
  if (H % 8 != 0 || H > 4 * 512 * 8 || B < 0 || topk > 8) return -1;
  if (src_ptrs != nullptr && (n_src < 1 || n_src > 8)) return -1;
  if (B == 0) return 0;
  NormParams p;
  p.use_ptrs = src_ptrs != nullptr;
  p.mc_base = p.use_ptrs ? (const __nv_bfloat16*)mc_base : nullptr;
  for (int i = 0; i < 8; ++i) p.src_base[i] = (p.use_ptrs && i < n_src) ? (const __nv_bfloat16*)src_ptrs[i] : nullptr;
  p.residual = (const __nv_bfloat16*)residual; p.partial = (const __nv_bfloat16*)partial;
  p.row_idx = row_idx; p.row_w = row_w; p.gamma = (const __nv_bfloat16*)gamma;
  p.owner_ids = owner_ids; p.experts_per_owner = experts_per_owner > 0 ? experts_per_owner : 1; p.owner_span = owner_span > 0 ? owner_span : 1;
  p.residual_out = (__nv_bfloat16*)residual_out; p.normed_out = (__nv_bfloat16*)normed_out;
  p.flags = flags; p.epoch = epoch; p.status = status; p.src_stride = src_stride;
  p.B = B; p.H = H; p.n_src = n_src; p.topk = topk; p.eps = eps;
  p.budget_ns = (unsigned long long)(wait_budget_ms > 0 ? wait_budget_ms : 10000) * 1000000ull;
  int threads = (H / 8 + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  const int passes = (H + threads * 8 - 1) / (threads * 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (passes <= 1) return (int)launch_pdl(reduce_residual_rmsnorm_kernel<1>, dim3(B), dim3(threads), 0, s, p);
  if (passes <= 2) return (int)launch_pdl(reduce_residual_rmsnorm_kernel<2>, dim3(B), dim3(threads), 0, s, p);
  return (int)launch_pdl(reduce_residual_rmsnorm_kernel<4>, dim3(B), dim3(threads), 0, s, p);
}

// Fused variant for decode-sized batches (see reduce_norm_route_kernel). `barrier` is two zeroed device
// ints reserved for this entry point; `max_resident_ctas` is how many CTAs of 512 threads the device
// holds at once (its SM count): larger batches are refused (-2) and take the separate kernels.
extern "C" int skein_reduce_norm_route(
    const void* residual, const void* partial, const void* gamma, void* residual_out, void* normed_out,
    const int* flags, const int* epoch, int* status, long long src_stride, int B, int H, int n_src, float eps,
    int wait_budget_ms, const void* wg, int E, int topk, int e_first, int e_count, int* expert_ids, float* expert_w,
    int* counts, int* offsets, int* row_of, int* src_token, void* xs, int* barrier, int max_resident_ctas,
    const void* const* src_ptrs, const void* mc_base, void* stream) {
  using namespace skein;
  if (H % 8 != 0 || H > 4 * 512 * 8 || B < 0) return -1;
  if (B == 0) return 0;
  if (E > NR_MAX_E || topk > NR_MAX_K || topk > E || B * topk > NR_MAX_PAIRS) return -1;
  if (B > max_resident_ctas) return -2;
  if (gamma == nullptr || normed_out == nullptr || wg == nullptr || barrier == nullptr) return -1;
  if (src_ptrs != nullptr && (n_src < 1 || n_src > 8)) return -1;
  NormParams p;
  p.use_ptrs = src_ptrs != nullptr;
  p.mc_base = p.use_ptrs ? (const __nv_bfloat16*)mc_base : nullptr;
  for (int i = 0; i < 8; ++i) p.src_base[i] = (p.use_ptrs && i < n_src) ? (const __nv_bfloat16*)src_ptrs[i] : nullptr;
  p.residual = (const __nv_bfloat16*)residual; p.partial = (const __nv_bfloat16*)partial;
  p.row_idx = nullptr; p.row_w = nullptr; p.gamma = (const __nv_bfloat16*)gamma;
  p.owner_ids = nullptr; p.experts_per_owner = 1; p.owner_span = 1;
  p.residual_out = (__nv_bfloat16*)residual_out; p.normed_out = (__nv_bfloat16*)normed_out;
  p.flags = flags; p.epoch = epoch; p.status = status; p.src_stride = src_stride;
  p.B = B; p.H = H; p.n_src = n_src; p.topk = 0; p.eps = eps;
  p.budget_ns = (unsigned long long)(wait_budget_ms > 0 ? wait_budget_ms : 10000) * 1000000ull;
  RouteParams r;
  r.wg = (const __nv_bfloat16*)wg; r.expert_ids = expert_ids; r.expert_w = expert_w; r.counts = counts;
  r.offsets = offsets; r.row_of = row_of; r.src_token = src_token; r.xs = (__nv_bfloat16*)xs; r.barrier = barrier;
  r.E = E; r.topk = topk; r.e_first = e_first; r.e_count = e_count;
  r.barrier_budget_ns = (unsigned long long)grid_barrier_budget_ms() * 1000000ull;
  int threads = (H / 8 + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  const int passes = (H + threads * 8 - 1) / (threads * 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (passes <= 1) return (int)launch_pdl(reduce_norm_route_kernel<1>, dim3(B), dim3(threads), 0, s, p, r);
  if (passes <= 2) return (int)launch_pdl(reduce_norm_route_kernel<2>, dim3(B), dim3(threads), 0, s, p, r);
  return (int)launch_pdl(reduce_norm_route_kernel<4>, dim3(B), dim3(threads), 0, s, p, r);
}
