// Row argmax building blocks shared by the greedy sampler (sample.cu) and the vocabulary-parallel candidate push
// (comm.cu): the (value, index) pair, its order (larger value, then lower index), a per-thread scan of a bf16 row
// with 16-byte loads, and the block-wide reduction.
#pragma once
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

namespace skein {

struct ValIdx { float v; int i; };

__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// This thread's share of row[0 .. V): the elements before the first 16-byte boundary one per thread, then whole
// 16-byte vectors (eight bf16) strided by the block, all of a thread's loads of one round issued before the first
// comparison, then the ragged tail. Every thread visits its indices in ascending order, so the strict comparison
// keeps the lowest index among equal values.
__device__ __forceinline__ ValIdx thread_argmax_row(const __nv_bfloat16* __restrict__ row, int V) {
  ValIdx best{-INFINITY, 0x7fffffff};
  const int tid = threadIdx.x, nt = blockDim.x;
  int head = (int)(((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u) >> 1);
  if (head > V) head = V;
  if (tid < head) {
    const float v = __bfloat162float(row[tid]);
    if (v > best.v) { best.v = v; best.i = tid; }
  }
  const int n_vec = (V - head) >> 3;
  const uint4* vec = reinterpret_cast<const uint4*>(row + head);
  constexpr int U = 4;
  for (int v0 = tid; v0 < n_vec; v0 += U * nt) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v0 + u * nt < n_vec) r[u] = __ldg(vec + v0 + u * nt);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * nt >= n_vec) continue;
      const uint32_t w[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
      const int base = head + ((v0 + u * nt) << 3);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
        if (lo > best.v) { best.v = lo; best.i = base + 2 * j; }
        if (hi > best.v) { best.v = hi; best.i = base + 2 * j + 1; }
      }
    }
  }
  const int tail0 = head + (n_vec << 3);
  if (tail0 + tid < V) {
    const float v = __bfloat162float(row[tail0 + tid]);
    if (v > best.v) { best.v = v; best.i = tail0 + tid; }
  }
  return best;
}

// Block-wide winner, returned to every thread. `sh` holds one entry per warp (32 at most).
__device__ __forceinline__ ValIdx block_argmax(ValIdx x, ValIdx* sh) {
  for (int o = 16; o > 0; o >>= 1) {
    ValIdx y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = x;
  __syncthreads();
  ValIdx r = (l < nw) ? sh[l] : ValIdx{-INFINITY, 0x7fffffff};
  for (int o = 16; o > 0; o >>= 1) {
    ValIdx y;
    y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, y);
  }
  __syncthreads();
  return r;
}

}  // namespace skein
