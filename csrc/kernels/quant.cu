// Block-scaled fp8 (e4m3) quantisation: one fp32 scale per 1 x 128 block along K.
//   scale = max(|x| over the block) / 448   (448 = largest finite e4m3 value), q = rn(x / scale)
// Used offline for weights (rows = output features) and online for activations (rows = tokens).
// A zero block gets scale 1 so that dequantisation is exact and never divides by zero.
//
// Replaces the reference's quantize_fp8_rows (vendor/luminal/crates/luminal_cuda_lite/src/host/
// moe/mod.rs:383-409), which keeps a single scale per row.
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace skein {

// Half a warp per 128-element block: each lane loads 16 bytes (8 elements) and stores 8; a grid-stride loop keeps
// several loads of a thread in flight.
__global__ void __launch_bounds__(256) quant_fp8_block128_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  __nv_fp8_storage_t* __restrict__ q,
                                                                  float* __restrict__ scales, long long n_blocks) {
  const int lane16 = threadIdx.x & 15;
  const long long stride = (long long)gridDim.x * (blockDim.x >> 4);
  for (long long blk = (long long)blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4); blk < n_blocks; blk += stride) {
    // rows are contiguous and K is a multiple of 128, so block `blk` starts at element blk * 128
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + blk * 128) + lane16);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t v = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v |= (uint32_t)__nv_cvt_float_to_fp8(f[4 * h + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      packed[h] = v;
    }
    *reinterpret_cast<uint2*>(q + blk * 128 + lane16 * 8) = make_uint2(packed[0], packed[1]);
    if (lane16 == 0) scales[blk] = scale;
  }
}

// The inverse, for the layout the GEMMs keep their weights in: q e4m3 [rows, K], scale_t fp32 [K / 128, rows]
// (K-block major) -> bf16 [rows, K]. One thread per 16 consecutive elements of a row (one 16-byte load, two 16-byte
// stores). Used when a projection runs at prefill size: the weight is expanded once into a transient bf16 matrix and the
// bf16 GEMM reuses every tile across all token tiles, instead of converting the tile again for each of them.
__global__ void __launch_bounds__(256) dequant_fp8_block128_kernel(const uint4* __restrict__ q, const float* __restrict__ scale_t,
                                                                    uint4* __restrict__ out, long long rows, int K) {
  const long long vec_per_row = K / 16;
  const long long n_vec = rows * vec_per_row;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (long long)gridDim.x * blockDim.x) {
    const long long row = v / vec_per_row;
    const int kv = (int)(v - row * vec_per_row);
    const float sc = __ldg(scale_t + (long long)(kv >> 3) * rows + row);
    const uint4 raw = __ldg(q + v);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[j] >> (16 * h)) & 0xffffu), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        o[2 * j + h] = *reinterpret_cast<const uint32_t*>(&b);
      }
    }
    out[2 * v] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * v + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace skein

extern "C" int skein_dequant_fp8_block128_t(const void* q, const float* scale_t, void* out, long long rows, int K, void* stream) {
  if (rows == 0) return 0;
  if (K % 128 != 0) return -1;
  const long long n_vec = rows * (K / 16);
  long long grid = (n_vec + 255) / 256;
  if (grid > 148LL * 16) grid = 148LL * 16;
  skein::dequant_fp8_block128_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)q, scale_t, (uint4*)out, rows, K);
  return (int)cudaGetLastError();
}

extern "C" int skein_quant_fp8_block128(const void* x, void* q, float* scales, long long rows, int K, void* stream) {
  if (rows == 0) return 0;
  if (K % 128 != 0) return -1;
  const long long nblocks = rows * (K / 128);
  const long long per_cta = 256 / 16;
  long long grid = (nblocks + per_cta - 1) / per_cta;
  if (grid > 148LL * 32) grid = 148LL * 32;     // grid-stride beyond that
  skein::quant_fp8_block128_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_fp8_storage_t*)q, scales, nblocks);
  return (int)cudaGetLastError();
}
