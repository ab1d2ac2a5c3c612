// MoE top-k router, entirely on the device.
//
//   1. router_topk_kernel: logits[t, e] = x[t, :] . Wg[e, :] (fp32 accumulate), the k largest
//      logits per token (ties -> lower expert index) and their softmax over the selected k, which
//      equals "softmax over all experts, take top-k, renormalise" (what Mixtral does).
//   2. router_plan_kernel (one CTA): per-expert counts, exclusive offsets, and a stable position
//      for every (token, slot) pair in expert-sorted order:
//         row_of[t, j]    position of pair (t, j) in the sorted list
//         src_token[r]    token whose activation belongs at sorted row r
//      One warp per expert walks the pairs in order with ballot/popc, so the layout is the same on
//      every run and on every rank.
// The grouped GEMM reads counts/offsets straight from device memory; nothing returns to the host.
//
// Replaces the reference's host-side routing (crates/skein_runtime/src/distributed/
// segment_runner.rs:249,1417: D2H of the router logits, host top-k softmax, pointer rebinding) and
// the graph-level iterative-argmax top_k_route (crates/skein_emit/src/op_wiring.rs:1667-1712).
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

constexpr int RT_MAX_E = 64;
constexpr int RT_MAX_K = 8;
constexpr int RT_STAGE_IDS = 2048;

__device__ void router_plan_body(const int* __restrict__ expert_ids, int n_pairs, int E, int topk,
                                 int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_of,
                                 int* __restrict__ src_token, int e_first, int e_count, int* cnt_s, int* off_s,
                                 const int* ids_s);

// grid = T tokens, 512 threads: thread i owns 8 consecutive elements of the hidden vector per pass, so
// every load of a pass is issued before the first is consumed. The last CTA to finish also lays out
// the expert-sorted order (router_plan_body), which saves a launch on the decode path.
__global__ void __launch_bounds__(512) router_topk_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ wg, int T, int H, int E,
                                                           int topk, int* __restrict__ expert_ids,
                                                           float* __restrict__ expert_w, float* __restrict__ logits_out,
                                                           int* counts, int* offsets, int* row_of, int* src_token,
                                                           int e_first, int e_count, int* done_counter) {
  __shared__ float part[16][RT_MAX_E];
  __shared__ float logit[RT_MAX_E];
  __shared__ int cnt_s[RT_MAX_E];
  __shared__ int off_s[RT_MAX_E + 1];
  __shared__ int is_last;
  __shared__ int ids_stage[RT_STAGE_IDS];
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e0 = 0; e0 < E; e0 += 8) {
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
    for (int h = tid * 8; h < H; h += 512 * 8) {
      const uint4 xr = *reinterpret_cast<const uint4*>(x + (size_t)t * H + h);
      uint4 wr[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        wr[i] = (e0 + i < E) ? *reinterpret_cast<const uint4*>(wg + (size_t)(e0 + i) * H + h) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xr);
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
#pragma unroll
    for (int w = 0; w < 16; ++w) v += part[w][tid];
    // the router projection is a bf16 linear layer: round like one
    logit[tid] = __bfloat162float(__float2bfloat16(v));
    if (logits_out) logits_out[(size_t)t * E + tid] = logit[tid];
  }
  __syncthreads();
  if (tid == 0) {
    int ids[RT_MAX_K];
    float vals[RT_MAX_K];
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
    const float vmax = vals[0];  // selections come out in descending order
    for (int j = 0; j < topk; ++j) { vals[j] = __expf(vals[j] - vmax); den += vals[j]; }
    for (int j = 0; j < topk; ++j) {
      expert_ids[t * topk + j] = ids[j];
      expert_w[t * topk + j] = vals[j] / den;
    }
    int last = 0;
    if (done_counter != nullptr) {
      __threadfence();
      const int old = atomicAdd(done_counter, 1);
      last = (old == (int)gridDim.x - 1);
      if (last) *done_counter = 0;
    }
    is_last = last;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n_pairs = T * topk;
  const int* staged = nullptr;
  if (n_pairs <= RT_STAGE_IDS) {
    for (int i = tid; i < n_pairs; i += blockDim.x) ids_stage[i] = __ldcg(expert_ids + i);
    __syncthreads();
    staged = ids_stage;
  }
  router_plan_body(expert_ids, n_pairs, E, topk, counts, offsets, row_of, src_token, e_first, e_count, cnt_s, off_s, staged);
}

// One CTA; one warp per expert walks the (token, slot) pairs in order. n_pairs = T * topk.
// Experts outside [e_first, e_first + e_count) get count 0 (expert parallelism: not ours).
__device__ void router_plan_body(const int* __restrict__ expert_ids, int n_pairs, int E, int topk,
                                 int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_of,
                                 int* __restrict__ src_token, int e_first, int e_count, int* cnt_s, int* off_s,
                                 const int* ids_s) {
  // ids_s: optional copy of expert_ids in shared memory (the two passes below then never wait on L2)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int c = 0;
    for (int i0 = 0; i0 < n_pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n_pairs && (ids_s ? ids_s[i] : __ldcg(expert_ids + i)) == e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) cnt_s[e] = (e >= e_first && e < e_first + e_count) ? c : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) { off_s[e] = a; a += cnt_s[e]; }
    off_s[E] = a;
    for (int e = 0; e < E; ++e) { counts[e] = cnt_s[e]; offsets[e] = off_s[e]; }
    offsets[E] = a;  // total rows
  }
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    const bool mine = cnt_s[e] > 0;
    int base = off_s[e];
    for (int i0 = 0; i0 < n_pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n_pairs && (ids_s ? ids_s[i] : __ldcg(expert_ids + i)) == e;
      const unsigned bal = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        if (mine) {
          const int r = base + __popc(bal & ((1u << lane) - 1));
          row_of[i] = r;
          src_token[r] = i / topk;
        } else {
          row_of[i] = -1;
        }
      }
      base += __popc(bal);
    }
  }
}

__global__ void __launch_bounds__(1024) router_plan_kernel(const int* __restrict__ expert_ids, int n_pairs, int E,
                                                            int topk, int* __restrict__ counts, int* __restrict__ offsets,
                                                            int* __restrict__ row_of, int* __restrict__ src_token,
                                                            int e_first, int e_count) {
  __shared__ int cnt_s[RT_MAX_E];
  __shared__ int off_s[RT_MAX_E + 1];
  router_plan_body(expert_ids, n_pairs, E, topk, counts, offsets, row_of, src_token, e_first, e_count, cnt_s, off_s, nullptr);
}

}  // namespace skein

// With done_counter (a zeroed device int) the same launch also produces the expert-sorted layout
// (counts[E], offsets[E+1], row_of[T*topk], src_token[T*topk]); without it only ids and weights.
extern "C" int skein_router_topk(const void* x, const void* wg, int T, int H, int E, int topk, int* expert_ids,
                                 float* expert_w, float* logits_out, int* counts, int* offsets, int* row_of,
                                 int* src_token, int e_first, int e_count, int* done_counter, void* stream) {
  using namespace skein;
  if (T == 0) return 0;
  if (E > RT_MAX_E || topk > RT_MAX_K || topk > E || H % 8 != 0) return -1;
  router_topk_kernel<<<T, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)wg, T, H, E,
                                                          topk, expert_ids, expert_w, logits_out, counts, offsets,
                                                          row_of, src_token, e_first, e_count, done_counter);
  return (int)cudaGetLastError();
}

extern "C" int skein_router_plan(const int* expert_ids, int n_pairs, int E, int topk, int* counts, int* offsets,
                                 int* row_of, int* src_token, int e_first, int e_count, void* stream) {
  using namespace skein;
  if (E > RT_MAX_E) return -1;
  int warps = E < 32 ? E : 32;
  router_plan_kernel<<<1, warps * 32, 0, (cudaStream_t)stream>>>(expert_ids, n_pairs, E, topk, counts, offsets, row_of,
                                                                 src_token, e_first, e_count);
  return (int)cudaGetLastError();
}
