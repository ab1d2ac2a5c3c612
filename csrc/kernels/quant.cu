// Block-scaled fp8 (e4m3) quantisation: one fp32 scale per 1 x 128 block along K.
//   scale = max(|x| over the block) / 448   (448 = largest finite e4m3 value), q = rn(x / scale)
// Used offline for weights (rows = output features) and online for activations (rows = tokens).
// A zero block gets scale 1 so that dequantisation is exact and never divides by zero.
//
// Replaces the reference's quantize_fp8_rows (vendor/luminal/crates/luminal_cuda_lite/src/host/
// moe/mod.rs:383-409), which keeps a single scale per row.
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace skein {

// One warp per 128-element block: each lane handles 4 consecutive elements.
__global__ void quant_fp8_block128_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ q,
                                          float* __restrict__ scales, long long rows, int K) {
  const long long blocks_per_row = K / 128;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= rows * blocks_per_row) return;
  const int lane = threadIdx.x & 31;
  const long long row = wid / blocks_per_row, kb = wid % blocks_per_row;
  const __nv_bfloat16* src = x + row * K + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 f0 = __bfloat1622float2(b2[0]), f1 = __bfloat1622float2(b2[1]);
  float amax = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
  const float inv = 1.0f / scale;
  uint32_t packed = 0;
  packed |= (uint32_t)__nv_cvt_float_to_fp8(f0.x * inv, __NV_SATFINITE, __NV_E4M3);
  packed |= (uint32_t)__nv_cvt_float_to_fp8(f0.y * inv, __NV_SATFINITE, __NV_E4M3) << 8;
  packed |= (uint32_t)__nv_cvt_float_to_fp8(f1.x * inv, __NV_SATFINITE, __NV_E4M3) << 16;
  packed |= (uint32_t)__nv_cvt_float_to_fp8(f1.y * inv, __NV_SATFINITE, __NV_E4M3) << 24;
  *reinterpret_cast<uint32_t*>(q + row * K + kb * 128 + lane * 4) = packed;
  if (lane == 0) scales[row * blocks_per_row + kb] = scale;
}

}  // namespace skein

extern "C" int skein_quant_fp8_block128(const void* x, void* q, float* scales, long long rows, int K, void* stream) {
  if (rows == 0) return 0;
  if (K % 128 != 0) return -1;
  const long long nblocks = rows * (K / 128);
  const int warps_per_cta = 8;
  const long long grid = (nblocks + warps_per_cta - 1) / warps_per_cta;
  if (grid > 0x7fffffffLL) return -2;
  skein::quant_fp8_block128_kernel<<<(unsigned)grid, warps_per_cta * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_fp8_storage_t*)q, scales, rows, K);
  return (int)cudaGetLastError();
}
