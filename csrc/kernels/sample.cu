// Token sampling from bf16 logits on the device: greedy argmax (ties -> lower index), and
// temperature / top-k / top-p sampling with a counter-based per-sequence RNG.
//
//   sample_argmax_kernel       one CTA per row; also emits (max value, index) so that
//                              vocabulary-parallel ranks can exchange 8 bytes per row instead of
//                              all-gathering logits
//   merge_candidates_kernel    picks the winner among the per-rank (value, index) candidates that
//                              peers pushed into this rank's buffer (bounded flag wait)
//   sample_topk_topp_kernel    k <= 64 passes of block-argmax build the descending candidate list,
//                              top-p truncates it, one uniform draw selects the token
//
// Replaces the reference's argmax_bf16 (crates/skein_runtime/src/cuda/argmax.rs:25-58, one block,
// smem tree) and the all-gather of logit shards before it (crates/skein_runtime/src/cuda/
// nccl.rs:251-298).
#include "ptx.cuh"
#include "argmax.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

__global__ void __launch_bounds__(1024) sample_argmax_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                                              int V, int idx_offset, int* __restrict__ out_idx,
                                                              float* __restrict__ out_val) {
  __shared__ ValIdx sh[32];
  const int b = blockIdx.x;
  const __nv_bfloat16* row = logits + (size_t)b * ld;
  const ValIdx best = block_argmax(thread_argmax_row(row, V), sh);
  if (threadIdx.x == 0) {
    if (out_idx) out_idx[b] = best.i + idx_offset;
    if (out_val) out_val[b] = best.v;
  }
}

// cand_val / cand_idx: [n_src][stride] (first B of each row used); the winner is the largest value, ties -> lowest global index.
__global__ void merge_candidates_kernel(const float* cand_val, const int* cand_idx, int n_src, int B, int stride,
                                        const int* flags, const int* epoch, int* status, unsigned long long budget_ns,
                                        int* __restrict__ out_idx) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (flags != nullptr && (int)threadIdx.x < n_src) {
    const bool poisoned = status != nullptr && *(volatile int*)status == ST_TIMEOUT_PEER_FLAG;
    if (poisoned || !wait_flag_ge(flags + threadIdx.x, *epoch, budget_ns)) {
      report_status(status, ST_TIMEOUT_PEER_FLAG, threadIdx.x);
      failed = 1;
    }
  }
  __syncthreads();
  if (failed) return;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < B; b += gridDim.x * blockDim.x) {
    ValIdx best{-INFINITY, 0x7fffffff};
    for (int s = 0; s < n_src; ++s) {
      ValIdx c;
      c.v = __ldcg(cand_val + (size_t)s * stride + b);
      c.i = __ldcg(cand_idx + (size_t)s * stride + b);
      best = better(best, c);
    }
    out_idx[b] = best.i;
  }
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// temperature[b] <= 0 means greedy. top_k[b] in [1, 64] (0 -> 64). top_p[b] in (0, 1].
// The draw of row b comes from splitmix64(seed[b] ^ splitmix64(counter + 1)) with counter = step[b * step_stride]:
// one counter for the whole batch (stride 0) or one per row (stride 1: the token's position, which makes a
// request's random stream a function of its seed and position only, whatever else is in the batch).
__global__ void __launch_bounds__(1024) sample_topk_topp_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                                                 int V, const float* temperature, const int* top_k,
                                                                 const float* top_p, const unsigned long long* seeds,
                                                                 const int* step, int step_stride, int* __restrict__ out_idx) {
  __shared__ ValIdx sh[32];
  __shared__ float cand_v[64];
  __shared__ int cand_i[64];
  const int b = blockIdx.x;
  const __nv_bfloat16* row = logits + (size_t)b * ld;
  const float T = temperature ? temperature[b] : 0.f;
  int K = (T <= 0.f) ? 1 : (top_k ? top_k[b] : 64);
  if (K <= 0 || K > 64) K = 64;
  if (K > V) K = V;
  float bound_v = INFINITY;
  int bound_i = -1;
  for (int k = 0; k < K; ++k) {
    // next candidate: the largest (value, -index) strictly after the previous one
    ValIdx best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = __bfloat162float(row[i]);
      const bool after = (v < bound_v) || (v == bound_v && i > bound_i);
      if (after && v > best.v) { best.v = v; best.i = i; }
    }
    best = block_argmax(best, sh);
    if (threadIdx.x == 0) { cand_v[k] = best.v; cand_i[k] = best.i; }
    bound_v = best.v; bound_i = best.i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (K == 1) { out_idx[b] = cand_i[0]; return; }
    const float P = top_p ? top_p[b] : 1.f;
    float pr[64];
    float den = 0.f;
    for (int k = 0; k < K; ++k) { pr[k] = expf((cand_v[k] - cand_v[0]) / T); den += pr[k]; }
    int keep = K;
    float cum = 0.f;
    for (int k = 0; k < K; ++k) {
      cum += pr[k] / den;
      if (cum >= P) { keep = k + 1; break; }
    }
    float kept = 0.f;
    for (int k = 0; k < keep; ++k) kept += pr[k];
    const unsigned long long s = splitmix64((seeds ? seeds[b] : 0x1234ull) ^ splitmix64((unsigned long long)(step ? step[(size_t)b * step_stride] : 0) + 1));
    const float u = (float)((s >> 40) & 0xFFFFFF) / 16777216.0f * kept;
    float run = 0.f;
    int pick = cand_i[keep - 1];
    for (int k = 0; k < keep; ++k) {
      run += pr[k];
      if (u < run) { pick = cand_i[k]; break; }
    }
    out_idx[b] = pick;
  }
}

// Feeds a decode step's sampled tokens back as the next step's inputs without a host round trip:
// live rows (seq_len > 0) take the new token and move one position forward.
__global__ void advance_decode_state_kernel(const int* __restrict__ sampled, int* __restrict__ tokens,
                                            int* __restrict__ positions, int* __restrict__ seq_lens, int B,
                                            int* step_counter) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0 && step_counter) *step_counter += 1;
  if (b >= B || seq_lens[b] <= 0) return;
  tokens[b] = sampled[b];
  positions[b] += 1;
  seq_lens[b] += 1;
}

}  // namespace skein

extern "C" int skein_advance_decode_state(const int* sampled, int* tokens, int* positions, int* seq_lens, int B,
                                          int* step_counter, void* stream) {
  if (B == 0) return 0;
  skein::advance_decode_state_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(sampled, tokens, positions,
                                                                                        seq_lens, B, step_counter);
  return (int)cudaGetLastError();
}

extern "C" int skein_sample_argmax(const void* logits, long long ld, int B, int V, int idx_offset, int* out_idx,
                                   float* out_val, void* stream) {
  if (B == 0) return 0;
  skein::sample_argmax_kernel<<<B, 1024, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V, idx_offset,
                                                                    out_idx, out_val);
  return (int)cudaGetLastError();
}

extern "C" int skein_merge_candidates(const float* cand_val, const int* cand_idx, int n_src, int B, int stride, const int* flags,
                                      const int* epoch, int* status, int wait_budget_ms, int* out_idx, void* stream) {
  if (B == 0) return 0;
  const unsigned long long budget = (unsigned long long)(wait_budget_ms > 0 ? wait_budget_ms : 10000) * 1000000ull;
  skein::merge_candidates_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(cand_val, cand_idx, n_src, B, stride, flags, epoch, status,
                                                                      budget, out_idx);
  return (int)cudaGetLastError();
}

extern "C" int skein_sample_topk_topp(const void* logits, long long ld, int B, int V, const float* temperature,
                                      const int* top_k, const float* top_p, const unsigned long long* seeds,
                                      const int* step, int step_stride, int* out_idx, void* stream) {
  if (B == 0) return 0;
  skein::sample_topk_topp_kernel<<<B, 1024, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V, temperature,
                                                                       top_k, top_p, seeds, step, step_stride, out_idx);
  return (int)cudaGetLastError();
}
