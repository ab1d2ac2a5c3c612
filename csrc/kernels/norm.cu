// Residual add + RMSNorm, with the reduction half of the tensor-parallel all-reduce and the MoE
// top-k combine folded in.
//
// One kernel covers every "sum things into the residual stream, then normalise" point of a
// decoder block:
//   acc[h] = residual[b, h]
//          + sum over sources s (tensor-parallel ranks that pushed a partial result into this
//            rank's buffer; 1 on a single GPU)
//              of   partial[s][b, h]                                   (dense: attention o_proj)
//              or   sum_j weight[b, j] * partial[s][row[b, j], h]      (MoE: rows are in
//                                                                       expert-sorted order)
//   residual_out[b, h] = bf16(acc[h])
//   normed_out[b, h]   = bf16(residual_out[b, h] * rsqrt(mean(residual_out^2) + eps) * gamma[h])
// When sources are other GPUs the kernel first waits (bounded) until every source's flag has
// reached this buffer's current epoch.
//
// Replaces the reference's unfused rms_norm graph (crates/skein_emit/src/op_wiring.rs:1787), its
// elementwise residual adds and the NCCL all-reduce + copy-back
// (crates/skein_runtime/src/cuda/nccl.rs:196-245).
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace skein {

struct NormParams {
  const __nv_bfloat16* residual;   // [B, H] or null (treated as zero)
  const __nv_bfloat16* partial;    // [n_src][rows][H] or null
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
template <int MAX_PASSES>
__global__ void __launch_bounds__(512) reduce_residual_rmsnorm_kernel(const NormParams p) {
  __shared__ float sh[32];
  __shared__ int wait_failed;
  const int b = blockIdx.x;
  if (p.flags != nullptr) {
    if (threadIdx.x == 0) wait_failed = 0;
    __syncthreads();
    if ((int)threadIdx.x < p.n_src) {
      const int e = *p.epoch;
      if (!wait_flag_ge(p.flags + threadIdx.x, e, p.budget_ns)) {
        report_status(p.status, ST_TIMEOUT_PEER_FLAG, threadIdx.x);
        wait_failed = 1;
      }
    }
    __syncthreads();
    if (wait_failed) return;
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
    if (p.partial) {
      const int nk = p.topk > 0 ? p.topk : 1;
      for (int j = 0; j < nk; ++j) {
        const int row = p.row_idx ? p.row_idx[b * p.topk + j] : b;
        if (row < 0) continue;  // pair routed to an expert that lives on another rank
        const float w = p.row_w ? p.row_w[b * p.topk + j] : 1.f;
        int s_lo = 0, s_hi = p.n_src;
        if (p.owner_ids) {
          s_lo = (p.owner_ids[b * p.topk + j] / p.experts_per_owner) * p.owner_span;
          s_hi = s_lo + p.owner_span;
          if (s_lo < 0 || s_hi > p.n_src) continue;
        }
        for (int s = s_lo; s < s_hi; ++s) {
          const __nv_bfloat16* src = p.partial + (size_t)s * p.src_stride + (size_t)row * p.H + h;
          uint4 r;
          // data written by other GPUs: bypass L1
          asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(src));
          const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(rb[i]); a[2 * i] += w * f.x; a[2 * i + 1] += w * f.y; }
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
  if (p.gamma == nullptr || p.normed_out == nullptr) return;
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
  }
}

}  // namespace skein

extern "C" int skein_reduce_residual_rmsnorm(
    const void* residual, const void* partial, const int* row_idx, const float* row_w, const void* gamma,
    void* residual_out, void* normed_out, const int* flags, const int* epoch, int* status,
    long long src_stride, int B, int H, int n_src, int topk, float eps, int wait_budget_ms, const int* owner_ids,
    int experts_per_owner, int owner_span, void* stream) {
  using namespace skein;
  if (H % 8 != 0 || H > 4 * 512 * 8 || B < 0) return -1;
  if (B == 0) return 0;
  NormParams p;
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
  if (passes <= 1) reduce_residual_rmsnorm_kernel<1><<<B, threads, 0, s>>>(p);
  else if (passes <= 2) reduce_residual_rmsnorm_kernel<2><<<B, threads, 0, s>>>(p);
  else reduce_residual_rmsnorm_kernel<4><<<B, threads, 0, s>>>(p);
  return (int)cudaGetLastError();
}
