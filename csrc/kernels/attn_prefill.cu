// Causal prefill attention over the paged KV cache (chunked-prefill aware: a chunk of q_len new
// tokens attends to the kv_len tokens already in the cache, its own included).
//
// Flash-attention style, one CTA = 64 query rows of one head (4 warps x 16 rows), walking the
// context in 64-token tiles gathered from the block table into shared memory; scores and P*V run
// on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with the online softmax kept in registers.
// Prefill is a small part of the prefill step's FLOPs (the projections dominate), so this kernel
// stays on the register-resident mma path; the projections run on tcgen05 (gemm_ws.cu).
//
// The reference never runs a prefill attention kernel: its FlashInfer prefill wrapper returns -1
// (vendor/luminal/crates/luminal_cuda_lite/src/host/flashinfer/wrapper.cu:263-281) and prefill
// falls back to unfused graph ops (crates/skein_emit/src/op_wiring.rs:2155-2305).
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

constexpr int AP_BM = 64, AP_BN = 64, AP_D = 128, AP_THREADS = 128;

struct AttnPrefillParams {
  const __nv_bfloat16* q;   // [T, q_stride], head h at h * D
  const __nv_bfloat16* kv;
  const int* block_table;   // [S, max_blocks]
  const int* q_start;       // [S] first row of the sequence's chunk in q / out
  const int* q_len;         // [S]
  const int* kv_len;        // [S] tokens in the cache after this chunk was appended
  __nv_bfloat16* out;       // [T, Hq * D]
  int* status;
  long long q_stride;
  int Hq, Hkv, page_size, max_blocks, num_pages;
  float scale_log2e;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) {  // byte offset in a [rows][128] bf16 tile
  return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(AP_THREADS) attn_prefill_kernel(const AttnPrefillParams p) {
  __shared__ __align__(128) uint8_t q_s[AP_BM * AP_D * 2];
  __shared__ __align__(128) uint8_t k_s[AP_BN * AP_D * 2];
  __shared__ __align__(128) uint8_t v_s[AP_BN * AP_D * 2];

  const int qt = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qlen = p.q_len[seq];
  const int q0 = qt * AP_BM;
  if (q0 >= qlen) return;
  const int kvlen = p.kv_len[seq];
  const int pos0 = kvlen - qlen;          // absolute position of the chunk's first token
  const int qrow0 = p.q_start[seq];
  const int kvh = head / (p.Hq / p.Hkv);
  const int ps = p.page_size;

  // ---- Q tile -> shared (rows past the chunk are zero) ----
  for (int c = tid; c < AP_BM * 16; c += AP_THREADS) {
    const int r = c >> 4, ch = c & 15;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (q0 + r < qlen)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(qrow0 + q0 + r) * p.q_stride + (size_t)head * AP_D + ch * 8);
    *reinterpret_cast<uint4*>(q_s + swz(r, ch)) = v;
  }
  __syncthreads();
  // Q fragments for this warp's 16 rows, all 8 k-steps
  uint32_t qf[8][4];
  {
    const uint32_t base = smem_u32(q_s);
    const int r = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) ldsm_x4(base + swz(r, ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int row_a = q0 + warp * 16 + (lane >> 2);   // chunk-relative rows this lane's c0/c1 and c2/c3 belong to
  const int row_b = row_a + 8;
  const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;

  int kv_hi = pos0 + min(q0 + AP_BM, qlen);  // exclusive bound of keys any row of this tile may see
  if (kv_hi > kvlen) kv_hi = kvlen;
  const uint32_t kb = smem_u32(k_s), vb = smem_u32(v_s);

  for (int n0 = 0; n0 < kv_hi; n0 += AP_BN) {
    __syncthreads();  // previous tile fully consumed
    for (int c = tid; c < AP_BN * 16; c += AP_THREADS) {
      const int r = c >> 4, ch = c & 15;
      const int tk = n0 + r;
      uint4 kvv = make_uint4(0, 0, 0, 0), vvv = make_uint4(0, 0, 0, 0);
      if (tk < kv_hi) {
        int page = p.block_table[(size_t)seq * p.max_blocks + tk / ps];
        if (page < 0 || page >= p.num_pages) { report_status(p.status, ST_BAD_INDEX, page); page = 0; }
        const __nv_bfloat16* kp = p.kv + (((size_t)page * 2) * p.Hkv + kvh) * (size_t)ps * AP_D + (size_t)(tk % ps) * AP_D + ch * 8;
        kvv = *reinterpret_cast<const uint4*>(kp);
        vvv = *reinterpret_cast<const uint4*>(kp + (size_t)p.Hkv * ps * AP_D);
      }
      *reinterpret_cast<uint4*>(k_s + swz(r, ch)) = kvv;
      *reinterpret_cast<uint4*>(v_s + swz(r, ch)) = vvv;
    }
    __syncthreads();

    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        const int mat = lane >> 3;
        const int r = (nb + (mat >> 1)) * 8 + (lane & 7);
        ldsm_x4(kb + swz(r, ks * 2 + (mat & 1)), b0, b1, b2, b3);
        mma16816(s[nb], qf[ks], b0, b1);
        mma16816(s[nb + 1], qf[ks], b2, b3);
      }
    }
    // ---- scale, causal mask, online softmax ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      const int col = n0 + nb * 8 + (lane & 3) * 2;
      s[nb][0] = (col <= pos_a && col < kvlen) ? s[nb][0] * p.scale_log2e : -INFINITY;
      s[nb][1] = (col + 1 <= pos_a && col + 1 < kvlen) ? s[nb][1] * p.scale_log2e : -INFINITY;
      s[nb][2] = (col <= pos_b && col < kvlen) ? s[nb][2] * p.scale_log2e : -INFINITY;
      s[nb][3] = (col + 1 <= pos_b && col + 1 < kvlen) ? s[nb][3] * p.scale_log2e : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    // rows that see no key yet keep m = -inf; use 0 as the subtrahend there to avoid inf - inf
    const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - sub0);
    const float al1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - sub1);
    m0 = mn0; m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      s[nb][0] = exp2f(s[nb][0] - sub0); s[nb][1] = exp2f(s[nb][1] - sub0);
      s[nb][2] = exp2f(s[nb][2] - sub1); s[nb][3] = exp2f(s[nb][3] - sub1);
      rs0 += s[nb][0] + s[nb][1];
      rs1 += s[nb][2] + s[nb][3];
    }
    l0 = l0 * al0 + rs0;
    l1 = l1 * al1 + rs1;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int db = 0; db < 16; db += 2) {
        uint32_t b0, b1, b2, b3;
        const int mat = lane >> 3;
        const int r = kk * 16 + (mat & 1) * 8 + (lane & 7);
        ldsm_x4_t(vb + swz(r, db + (mat >> 1)), b0, b1, b2, b3);
        mma16816(o[db], a, b0, b1);
        mma16816(o[db + 1], a, b2, b3);
      }
    }
  }
  // ---- finish: quad-reduce the row sums, normalise, store ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const size_t ldo = (size_t)p.Hq * AP_D;
#pragma unroll
  for (int db = 0; db < 16; ++db) {
    const int d = db * 8 + (lane & 3) * 2;
    if (row_a < qlen)
      *reinterpret_cast<uint32_t*>(p.out + (size_t)(qrow0 + row_a) * ldo + (size_t)head * AP_D + d) = pack_bf16(o[db][0] * i0, o[db][1] * i0);
    if (row_b < qlen)
      *reinterpret_cast<uint32_t*>(p.out + (size_t)(qrow0 + row_b) * ldo + (size_t)head * AP_D + d) = pack_bf16(o[db][2] * i1, o[db][3] * i1);
  }
}

}  // namespace skein

extern "C" int skein_attn_prefill(const void* q, long long q_stride, const void* kv, const int* block_table,
                                  const int* q_start, const int* q_len, const int* kv_len, void* out, int* status,
                                  int S, int max_q_len, int Hq, int Hkv, int D, int page_size, int max_blocks,
                                  int num_pages, float scale, void* stream) {
  using namespace skein;
  if (S == 0 || max_q_len == 0) return 0;
  if (D != AP_D || Hq % Hkv != 0) return -1;
  AttnPrefillParams p;
  p.q = (const __nv_bfloat16*)q; p.kv = (const __nv_bfloat16*)kv; p.block_table = block_table;
  p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len; p.out = (__nv_bfloat16*)out; p.status = status;
  p.q_stride = q_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks;
  p.num_pages = num_pages; p.scale_log2e = scale * 1.4426950408889634f;
  dim3 grid((max_q_len + AP_BM - 1) / AP_BM, Hq, S);
  attn_prefill_kernel<<<grid, AP_THREADS, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
