// Paged-KV decode attention (one new query token per sequence) with grouped-query heads and
// split-KV. Memory-bound: every K and V row of the context is read exactly once per kv head and
// shared by the G query heads that map to it.
//
//   grid = (splits, Hkv, B), 128 threads. Per 128-token chunk of the context:
//     phase 1  thread t scores token t against the G query heads (16-byte loads of its K row)
//     phase 2  running max / rescale factors per head (online softmax, base-2 exponentials)
//     phase 3  16 threads span the 128 dims (8 each) x 8 token phases accumulate P*V
//   With splits > 1 each CTA parks (m, l, o) in a workspace and the last CTA of a (sequence,
//   kv head) to arrive merges them, so no second launch is needed.
//
// Cache layout: kv_cache[page, 0 = K / 1 = V, kv_head, slot, D] bf16; block_table[seq, i] = page of
// tokens [i * page_size, (i + 1) * page_size).
//
// Replaces the reference's fused_decode_attn (vendor/luminal/crates/luminal_cuda_lite/src/kernel/
// decode_attention.rs:66-139, fixed-capacity contiguous cache, f32) and the FlashInfer batch-decode
// wrapper (vendor/luminal/crates/luminal_cuda_lite/src/host/flashinfer/wrapper.cu:123-251).
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

constexpr int AD_THREADS = 128;
constexpr int AD_CHUNK = 128;
constexpr int AD_D = 128;
constexpr int AD_MAX_SPLITS = 16;

struct AttnDecodeParams {
  const __nv_bfloat16* q;   // [B, q_stride] with head h at h * D
  const __nv_bfloat16* kv;  // paged cache
  const int* block_table;   // [B, max_blocks]
  const int* seq_lens;      // [B] context length including the new token; 0 = padding row
  __nv_bfloat16* out;       // [B, Hq * D]
  float* ws_o;              // [B, Hq, splits, D]
  float* ws_ml;             // [B, Hq, splits, 2]
  int* counters;            // [B * Hkv], zero at first use
  int* status;
  long long q_stride;
  int B, Hq, Hkv, page_size, max_blocks, num_pages, splits;
  float scale_log2e;
};

template <int G>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const AttnDecodeParams p) {
  __shared__ __align__(16) float q_s[G][AD_D];
  __shared__ float s_s[G][AD_CHUNK];
  __shared__ int page_s[AD_CHUNK];
  __shared__ float red_s[G][4];
  __shared__ __align__(16) float o_s[8][G][AD_D];
  __shared__ int is_last;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int len = p.seq_lens[b];
  const int ps = p.page_size;

  // this split's token range, rounded to whole pages
  int per = (len + p.splits - 1) / p.splits;
  per = (per + ps - 1) / ps * ps;
  const int t_begin = split * per;
  int t_end = t_begin + per;
  if (t_end > len) t_end = len;

  for (int i = tid; i < G * AD_D; i += AD_THREADS) {
    const int g = i / AD_D, d = i % AD_D;
    q_s[g][d] = __bfloat162float(p.q[(size_t)b * p.q_stride + (size_t)(kvh * G + g) * AD_D + d]) * p.scale_log2e;
  }
  __syncthreads();

  float m[G], l_part[G], o_acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l_part[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o_acc[g][i] = 0.f;
  }
  const int dgrp = tid & 15;   // which 8 dims
  const int tph = tid >> 4;    // token phase 0..7
  const size_t head_stride = (size_t)ps * AD_D;

  for (int c0 = t_begin; c0 < t_end; c0 += AD_CHUNK) {
    // ---- phase 1: scores ----
    const int tk = c0 + tid;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = -INFINITY;
    if (tk < t_end) {
      int page = p.block_table[(size_t)b * p.max_blocks + tk / ps];
      if (page < 0 || page >= p.num_pages) { report_status(p.status, ST_BAD_INDEX, page); page = 0; }
      page_s[tid] = page;
      const __nv_bfloat16* kp = p.kv + ((size_t)page * 2 * p.Hkv + kvh) * head_stride + (size_t)(tk % ps) * AD_D;
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
      for (int c = 0; c < AD_D / 8; ++c) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kp + c * 8);
        const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float kf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(kb[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
          s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                  qb.z * kf[6] + qb.w * kf[7];
        }
      }
    }
    // ---- phase 2: chunk max per head, rescale ----
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = s[g];
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) red_s[g][warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float cm = fmaxf(fmaxf(red_s[g][0], red_s[g][1]), fmaxf(red_s[g][2], red_s[g][3]));
      const float mn = fmaxf(m[g], cm);
      alpha[g] = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      m[g] = mn;
      const float pr = (tk < t_end) ? exp2f(s[g] - mn) : 0.f;
      s_s[g][tid] = pr;
      l_part[g] = l_part[g] * alpha[g] + pr;
    }
    __syncthreads();
    // ---- phase 3: o = o * alpha + P V ----
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < 8; ++i) o_acc[g][i] *= alpha[g];
    const int n_valid = min(AD_CHUNK, t_end - c0);
    // 8 V rows are requested before any is used, so 8 x 16 bytes are in flight per thread
#pragma unroll 1
    for (int tb = tph; tb < n_valid; tb += 64) {
      uint4 raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int t = tb + u * 8;
        raw[u] = make_uint4(0, 0, 0, 0);
        if (t < n_valid) {
          const __nv_bfloat16* vp = p.kv + (((size_t)page_s[t] * 2 + 1) * p.Hkv + kvh) * head_stride +
                                    (size_t)((c0 + t) % ps) * AD_D + dgrp * 8;
          raw[u] = *reinterpret_cast<const uint4*>(vp);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int t = tb + u * 8;
        if (t < n_valid) {
          const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          float vf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(vb[i]); vf[2 * i] = f.x; vf[2 * i + 1] = f.y; }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pr = s_s[g][t];
#pragma unroll
            for (int i = 0; i < 8; ++i) o_acc[g][i] += pr * vf[i];
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- combine the 8 token phases and the per-thread partial sums ----
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) o_s[tph][g][dgrp * 8 + i] = o_acc[g][i];
  float l_tot[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float v = l_part[g];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red_s[g][warp] = v;
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) l_tot[g] = red_s[g][0] + red_s[g][1] + red_s[g][2] + red_s[g][3];

  const int d = tid;  // one output dim per thread from here on
  if (p.splits == 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float o = 0.f;
#pragma unroll
      for (int ph = 0; ph < 8; ++ph) o += o_s[ph][g][d];
      const float r = l_tot[g] > 0.f ? o / l_tot[g] : 0.f;
      p.out[((size_t)b * p.Hq + kvh * G + g) * AD_D + d] = __float2bfloat16(r);
    }
    return;
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float o = 0.f;
#pragma unroll
    for (int ph = 0; ph < 8; ++ph) o += o_s[ph][g][d];
    const size_t base = ((size_t)b * p.Hq + kvh * G + g) * p.splits + split;
    p.ws_o[base * AD_D + d] = o;
    if (d == 0) { p.ws_ml[base * 2] = m[g]; p.ws_ml[base * 2 + 1] = l_tot[g]; }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = p.counters + b * p.Hkv + kvh;
    const int old = atomicAdd(ctr, 1);
    is_last = (old == p.splits - 1);
    if (is_last) *ctr = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Merge: (m, l) of every head and split are staged in shared memory with one parallel load, then each
  // thread fetches its output dim of all splits at once (independent loads, all in flight together).
  float* ml_s = &o_s[0][0][0];   // the P*V scratch is free by now: [G][AD_MAX_SPLITS][2] floats
  const size_t base0 = ((size_t)b * p.Hq + kvh * G) * p.splits;
  for (int i = tid; i < G * p.splits * 2; i += AD_THREADS) ml_s[i] = __ldcg(&p.ws_ml[base0 * 2 + i]);
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const size_t base = base0 + (size_t)g * p.splits;
    float ov[AD_MAX_SPLITS];
#pragma unroll
    for (int s2 = 0; s2 < AD_MAX_SPLITS; ++s2) ov[s2] = (s2 < p.splits) ? __ldcg(&p.ws_o[(base + s2) * AD_D + d]) : 0.f;
    float M = -INFINITY;
    for (int s2 = 0; s2 < p.splits; ++s2) M = fmaxf(M, ml_s[(g * p.splits + s2) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < AD_MAX_SPLITS; ++s2) {
      if (s2 < p.splits) {
        const float mi = ml_s[(g * p.splits + s2) * 2];
        const float w = (mi == -INFINITY) ? 0.f : exp2f(mi - M);
        L += w * ml_s[(g * p.splits + s2) * 2 + 1];
        O += w * ov[s2];
      }
    }
    p.out[((size_t)b * p.Hq + kvh * G + g) * AD_D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
  }
}

}  // namespace skein

extern "C" long long skein_attn_decode_workspace_floats(int B, int Hq, int splits) {
  return (long long)B * Hq * splits * (skein::AD_D + 2);
}

extern "C" int skein_attn_decode(const void* q, long long q_stride, const void* kv, const int* block_table,
                                 const int* seq_lens, void* out, float* workspace, int* counters, int* status, int B,
                                 int Hq, int Hkv, int D, int page_size, int max_blocks, int num_pages, int splits,
                                 float scale, void* stream) {
  using namespace skein;
  if (B == 0) return 0;
  if (D != AD_D || Hq % Hkv != 0 || splits < 1 || splits > AD_MAX_SPLITS) return -1;
  AttnDecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.kv = (const __nv_bfloat16*)kv; p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = (__nv_bfloat16*)out;
  p.ws_o = workspace;
  p.ws_ml = workspace ? workspace + (size_t)B * Hq * splits * AD_D : nullptr;
  p.counters = counters; p.status = status; p.q_stride = q_stride;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.splits = splits;
  p.scale_log2e = scale * 1.4426950408889634f;
  if (splits > 1 && (!workspace || !counters)) return -2;
  dim3 grid(splits, Hkv, B);
  cudaStream_t s = (cudaStream_t)stream;
  switch (Hq / Hkv) {
    case 1: attn_decode_kernel<1><<<grid, AD_THREADS, 0, s>>>(p); break;
    case 2: attn_decode_kernel<2><<<grid, AD_THREADS, 0, s>>>(p); break;
    case 4: attn_decode_kernel<4><<<grid, AD_THREADS, 0, s>>>(p); break;
    case 8: attn_decode_kernel<8><<<grid, AD_THREADS, 0, s>>>(p); break;
    default: return -3;
  }
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in attn_decode_noalloc.h).
// The split-KV scratch is part of the library image. In host code the names below are host-side
// stand-ins for the device arrays, not device addresses: the addresses a kernel can use come from
// cudaGetSymbolAddress, looked up once per device and cached.
// ---------------------------------------------------------------------------------------------
#include "attn_decode_noalloc.h"

namespace skein {
static __device__ __align__(256) float g_noalloc_scratch[(size_t)SKEIN_ATTN_NOALLOC_MAX_ROWS * (AD_D + 2)];
static __device__ __align__(256) int g_noalloc_counters[SKEIN_ATTN_NOALLOC_MAX_COUNTERS];

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoAllocDevice { float* scratch; int* counters; bool ready; };
static NoAllocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];
}  // namespace skein

extern "C" const char* skein_attn_decode_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case SKEIN_NOALLOC_ERR_BAD_ARGS: return "bad arguments (D must be 128, splits >= 1, Hq a multiple of Hkv, B >= 0)";
    case SKEIN_NOALLOC_ERR_TOO_LARGE:
      return "problem exceeds the built-in scratch: need B*Hq*splits <= 8192, B*Hkv <= 4096 and splits <= 16";
    case SKEIN_NOALLOC_ERR_UNSUPPORTED_GROUP: return "Hq / Hkv must be 1, 2, 4 or 8";
    case SKEIN_NOALLOC_ERR_DEVICE: return "could not identify the current device or its index is out of range";
    default: return "CUDA runtime error (positive values are cudaError_t)";
  }
}

extern "C" int skein_attn_decode_noalloc(const void* q, long long q_stride, const void* kv, const int* block_table,
                                         const int* seq_lens, void* out, int* status, int B, int Hq, int Hkv, int D,
                                         int page_size, int max_blocks, int num_pages, int splits, float scale,
                                         void* stream) {
  using namespace skein;
  if (B == 0) return 0;
  if (B < 0 || D != AD_D || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || splits < 1 || page_size <= 0) return SKEIN_NOALLOC_ERR_BAD_ARGS;
  const int G = Hq / Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return SKEIN_NOALLOC_ERR_UNSUPPORTED_GROUP;
  if ((long long)B * Hq * splits > SKEIN_ATTN_NOALLOC_MAX_ROWS || (long long)B * Hkv > SKEIN_ATTN_NOALLOC_MAX_COUNTERS)
    return SKEIN_NOALLOC_ERR_TOO_LARGE;
  if (splits > AD_MAX_SPLITS) return SKEIN_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SKEIN_NOALLOC_ERR_DEVICE;
  NoAllocDevice& nd = g_noalloc_dev[dev];
  if (!nd.ready) {
    // set-up, once per device, with that device current
    void* ps = nullptr;
    void* pc = nullptr;
    e = cudaGetSymbolAddress(&ps, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress(&pc, g_noalloc_counters);
    if (e != cudaSuccess) return (int)e;
    nd.scratch = static_cast<float*>(ps);
    nd.counters = static_cast<int*>(pc);
    nd.ready = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // the scratch keeps the previous call's contents: the arrival counters must start at zero
  e = cudaMemsetAsync(nd.counters, 0, sizeof(int) * (size_t)B * Hkv, s);
  if (e != cudaSuccess) return (int)e;
  AttnDecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.kv = (const __nv_bfloat16*)kv; p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = (__nv_bfloat16*)out;
  p.ws_o = nd.scratch;
  p.ws_ml = nd.scratch + (size_t)B * Hq * splits * AD_D;
  p.counters = nd.counters; p.status = status; p.q_stride = q_stride;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.splits = splits;
  p.scale_log2e = scale * 1.4426950408889634f;
  dim3 grid(splits, Hkv, B);
  switch (G) {
    case 1: attn_decode_kernel<1><<<grid, AD_THREADS, 0, s>>>(p); break;
    case 2: attn_decode_kernel<2><<<grid, AD_THREADS, 0, s>>>(p); break;
    case 4: attn_decode_kernel<4><<<grid, AD_THREADS, 0, s>>>(p); break;
    default: attn_decode_kernel<8><<<grid, AD_THREADS, 0, s>>>(p); break;
  }
  return (int)cudaGetLastError();
}
