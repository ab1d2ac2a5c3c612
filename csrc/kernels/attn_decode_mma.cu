// Paged-KV decode attention on tensor cores with an asynchronous copy pipeline.
//
// The scalar kernel in attn_decode.cu issues one FMA per (query head, key element); at 64 sequences
// it is bound by instruction issue, not by HBM. Here the G query heads that share a kv head are the
// rows of a 16-row MMA tile (rows >= G are zero padding), so a 16-token tile of the context costs
// 16 + 16 mma.sync m16n8k16 instead of ~4k scalar FMAs per warp, and K/V tiles stream from the
// cache into shared memory with cp.async while earlier tiles are being multiplied.
//
//   grid = (splits, Hkv, B), 128 threads. The split's range of 16-token tiles is dealt round-robin
//   to the 4 warps. Each warp runs its own 3- or 6-stage pipeline (no CTA-wide barrier in the loop):
//       cp.async tile i+2 (K 4 KB + V 4 KB, XOR-swizzled rows)      wait tile i
//       S = Q K^T  (2 n-tiles x 8 k-steps)   online softmax in registers   O += P V (16 n-tiles)
//   and keeps (m, l, O) for its share of the tokens. The warps' states are merged through shared
//   memory; with splits > 1 the CTA parks its state in a workspace and the last CTA of a
//   (sequence, kv head) to arrive merges the splits, as in the scalar kernel.
//
// Cache layout: kv_cache[page, 0 = K / 1 = V, kv_head, slot, 128] bf16 with page_size % 16 == 0.
// Same operator as the reference's fused_decode_attn (vendor/luminal/crates/luminal_cuda_lite/src/
// kernel/decode_attention.rs:66-139) and its FlashInfer batch-decode wrapper
// (vendor/luminal/crates/luminal_cuda_lite/src/host/flashinfer/wrapper.cu:123-251).
#include "ptx.cuh"
#include "launch.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace skein {

constexpr int AM_THREADS = 128;
constexpr int AM_WARPS = 4;
constexpr int AM_D = 128;
constexpr int AM_TILE = 16;                       // tokens per tile
// cp.async ring depth per warp: 3 (two CTAs per SM, for launches with more CTAs than SMs) or 6 (one CTA per SM gets
// the whole shared memory: twice the bytes in flight per CTA when there are fewer CTAs than SMs)
constexpr int AM_TILE_BYTES = AM_TILE * AM_D * 2;  // 4 KB (K or V)
constexpr int AM_STAGE_BYTES = 2 * AM_TILE_BYTES;  // K then V
constexpr int am_warp_bytes(int stages) { return stages * AM_STAGE_BYTES; }
constexpr int am_smem_bytes(int stages) { return AM_WARPS * am_warp_bytes(stages) + AM_TILE_BYTES; }  // + the Q tile
constexpr int AM_MAX_SPLITS = 16;

struct AttnMmaParams {
  const __nv_bfloat16* q;   // [B, q_stride] with head h at h * D
  const __nv_bfloat16* kv;  // paged cache
  __nv_bfloat16* kv_rw;     // the same cache, writable (RoPE + append fusion)
  const int* block_table;   // [B, max_blocks]
  const int* seq_lens;      // [B] context length including the new token; 0 = padding row
  __nv_bfloat16* out;       // [B, Hq * D]
  float* ws_o;              // [B, Hq, splits, D]
  float* ws_ml;             // [B, Hq, splits, 2]
  int* counters;            // [B * Hkv], zero at first use
  int* status;
  long long q_stride;
  int B, Hq, Hkv, G, page_size, max_blocks, num_pages, splits;
  float scale_log2e;
  // optional fusion of RoPE and the KV append of the new token (cos_sin == nullptr: q is already rotated and
  // the cache already holds the token). q then points at the raw fused q/k/v projection rows
  // [B, q_stride >= (Hq + 2 * Hkv) * D]: q heads, k heads, v heads.
  const float* cos_sin;     // [max_pos, D/2, 2] fp32
  const int* positions;     // [B] position of the new token, -1 = padding row
  int max_pos;
};

__device__ __forceinline__ uint32_t am_swz(int row, int chunk) {  // byte offset in a [16][128] bf16 tile
  return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void am_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void am_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void am_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t am_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// 16-byte asynchronous copy; src_bytes = 0 writes zeros (rows past the end of the context)
__device__ __forceinline__ void am_cp_async(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void am_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void am_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <int AM_STAGES>
__global__ void __launch_bounds__(AM_THREADS) attn_decode_mma_kernel(const AttnMmaParams p) {
  constexpr int AM_WARP_BYTES = AM_STAGES * AM_STAGE_BYTES;
  extern __shared__ __align__(128) uint8_t am_smem[];
  __shared__ int is_last;
  pdl_trigger();
  pdl_wait();   // q, the cache and the sequence lengths come from earlier kernels of the step
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, ps = p.page_size;
  const int len = p.seq_lens[b];

  // this split's token range, rounded to whole pages (pages are multiples of the tile)
  int per = (len + p.splits - 1) / p.splits;
  per = (per + ps - 1) / ps * ps;
  const int t_begin = split * per;
  int t_end = t_begin + per;
  if (t_end > len) t_end = len;
  const int tile_begin = t_begin / AM_TILE;
  const int n_tiles = t_end > t_begin ? (t_end - t_begin + AM_TILE - 1) / AM_TILE : 0;
  const int n_my = n_tiles > warp ? (n_tiles - warp + AM_WARPS - 1) / AM_WARPS : 0;   // tiles of this warp

  uint8_t* q_s = am_smem + AM_WARPS * AM_WARP_BYTES;
  const uint32_t q_base = smem_u32(q_s);
  const uint32_t st_base = smem_u32(am_smem) + warp * AM_WARP_BYTES;

  // ---- Q rows (G heads, zero padded to 16) -> shared -> A fragments for all 8 k-steps ----
  const bool rope = p.cos_sin != nullptr;
  int pos = rope ? p.positions[b] : -1;
  if (rope && pos >= p.max_pos) { report_status(p.status, ST_BAD_INDEX, pos); pos = -1; }
  if (!rope) {
    for (int c = tid; c < AM_TILE * 16; c += AM_THREADS) {
      const int r = c >> 4, ch = c & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < G) v = *reinterpret_cast<const uint4*>(p.q + (size_t)b * p.q_stride + (size_t)(kvh * G + r) * AM_D + ch * 8);
      *reinterpret_cast<uint4*>(q_s + am_swz(r, ch)) = v;
    }
  } else {
    // rotate-half RoPE: dim i pairs with dim i + 64, i.e. chunk ch with chunk ch + 8; one pair of chunks per thread
    const int r = tid >> 3, ch = tid & 7;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
    if (r < G && pos >= 0) {
      const __nv_bfloat16* qp = p.q + (size_t)b * p.q_stride + (size_t)(kvh * G + r) * AM_D;
      lo = *reinterpret_cast<const uint4*>(qp + ch * 8);
      hi = *reinterpret_cast<const uint4*>(qp + 64 + ch * 8);
      const float4* cs = reinterpret_cast<const float4*>(p.cos_sin + ((size_t)pos * 64 + ch * 8) * 2);
      __nv_bfloat162* lb = reinterpret_cast<__nv_bfloat162*>(&lo);
      __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 c2 = cs[i];   // (cos, sin) of dims 2i and 2i + 1 of this chunk
        const float2 x0 = __bfloat1622float2(lb[i]), x1 = __bfloat1622float2(hb[i]);
        lb[i] = __floats2bfloat162_rn(x0.x * c2.x - x1.x * c2.y, x0.y * c2.z - x1.y * c2.w);
        hb[i] = __floats2bfloat162_rn(x1.x * c2.x + x0.x * c2.y, x1.y * c2.z + x0.y * c2.w);
      }
    }
    *reinterpret_cast<uint4*>(q_s + am_swz(r, ch)) = lo;
    *reinterpret_cast<uint4*>(q_s + am_swz(r, ch + 8)) = hi;
    // the CTA whose token range holds the new token rotates its K row and appends K and V to the cache;
    // the barrier below orders these stores before the asynchronous copies that read them back
    if (pos >= 0) {
      int s_app = per > 0 ? pos / per : 0;
      if (s_app > p.splits - 1) s_app = p.splits - 1;
      if (s_app == split) {
        int pg = p.block_table[(size_t)b * p.max_blocks + pos / ps];
        if (pg < 0 || pg >= p.num_pages) {
          report_status(p.status, ST_BAD_INDEX, pg);
        } else {
          const __nv_bfloat16* kr = p.q + (size_t)b * p.q_stride + (size_t)(p.Hq + kvh) * AM_D;
          const __nv_bfloat16* vr = kr + (size_t)p.Hkv * AM_D;
          __nv_bfloat16* kd = p.kv_rw + (((size_t)pg * 2) * p.Hkv + kvh) * (size_t)ps * AM_D + (size_t)(pos % ps) * AM_D;
          __nv_bfloat16* vd = kd + (size_t)p.Hkv * ps * AM_D;
          if (tid < 64) {
            const float2 cs = reinterpret_cast<const float2*>(p.cos_sin)[(size_t)pos * 64 + tid];
            const float x0 = __bfloat162float(kr[tid]), x1 = __bfloat162float(kr[tid + 64]);
            kd[tid] = __float2bfloat16(x0 * cs.x - x1 * cs.y);
            kd[tid + 64] = __float2bfloat16(x1 * cs.x + x0 * cs.y);
          } else {
            const int j = tid - 64;
            reinterpret_cast<__nv_bfloat162*>(vd)[j] = reinterpret_cast<const __nv_bfloat162*>(vr)[j];
          }
        }
      }
    }
  }
  __syncthreads();
  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    am_ldsm_x4(q_base + am_swz(lane & 15, ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // ---- the warp's copy pipeline ----
  const size_t head_stride = (size_t)ps * AM_D;          // elements of one (page, k/v, head) slab
  int pg_block = 0;                                      // page ids of tiles j0 .. j0+31 of this warp, one per lane
  auto load_pages = [&](int j0) {
    const int j = j0 + lane;
    int pg = 0;
    if (j < n_my) {
      const int tile = tile_begin + warp + j * AM_WARPS;
      pg = p.block_table[(size_t)b * p.max_blocks + (tile * AM_TILE) / ps];
      if (pg < 0 || pg >= p.num_pages) { report_status(p.status, ST_BAD_INDEX, pg); pg = 0; }
    }
    pg_block = pg;
  };
  auto issue = [&](int j) {   // start the copy of this warp's j-th tile (or an empty group past the end)
    if (j < n_my) {
      if ((j & 31) == 0) load_pages(j);
      const int pg = __shfl_sync(0xffffffffu, pg_block, j & 31);
      const int tile = tile_begin + warp + j * AM_WARPS;
      const int tok0 = tile * AM_TILE;
      const __nv_bfloat16* kp = p.kv + ((size_t)pg * 2 * p.Hkv + kvh) * head_stride + (size_t)(tok0 % ps) * AM_D;
      const __nv_bfloat16* vp = kp + (size_t)p.Hkv * head_stride;
      const uint32_t dst = st_base + (j % AM_STAGES) * AM_STAGE_BYTES;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i, r = c >> 4, ch = c & 15;
        const int nbytes = (tok0 + r < t_end) ? 16 : 0;
        am_cp_async(dst + am_swz(r, ch), kp + r * AM_D + ch * 8, nbytes);
        am_cp_async(dst + AM_TILE_BYTES + am_swz(r, ch), vp + r * AM_D + ch * 8, nbytes);
      }
    }
    am_commit();
  };
#pragma unroll
  for (int s = 0; s < AM_STAGES - 1; ++s) issue(s);

  for (int j = 0; j < n_my; ++j) {
    am_wait<AM_STAGES - 2>();   // this lane's part of tile j has landed
    __syncwarp();               // ... and every lane's; all lanes are also done with tile j-1
    issue(j + AM_STAGES - 1);   // refills the stage tile j-1 used
    const uint32_t kb = st_base + (j % AM_STAGES) * AM_STAGE_BYTES, vb = kb + AM_TILE_BYTES;
    const int tok0 = (tile_begin + warp + j * AM_WARPS) * AM_TILE;

    // ---- S = Q K^T (16 rows x 16 tokens) ----
    float s[2][4];
    s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
    s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
    const int mat = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t b0, b1, b2, b3;
      am_ldsm_x4(kb + am_swz((mat >> 1) * 8 + (lane & 7), ks * 2 + (mat & 1)), b0, b1, b2, b3);
      am_mma(s[0], qf[ks], b0, b1);
      am_mma(s[1], qf[ks], b2, b3);
    }
    // ---- scale, mask the tokens past the end, online softmax (rows lane/4 and lane/4 + 8) ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int col = tok0 + nb * 8 + (lane & 3) * 2;
      s[nb][0] = (col < t_end) ? s[nb][0] * p.scale_log2e : -INFINITY;
      s[nb][1] = (col + 1 < t_end) ? s[nb][1] * p.scale_log2e : -INFINITY;
      s[nb][2] = (col < t_end) ? s[nb][2] * p.scale_log2e : -INFINITY;
      s[nb][3] = (col + 1 < t_end) ? s[nb][3] * p.scale_log2e : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // a tile holds at least one valid token: finite
    const float al0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0);
    const float al1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      s[nb][0] = exp2f(s[nb][0] - mn0); s[nb][1] = exp2f(s[nb][1] - mn0);
      s[nb][2] = exp2f(s[nb][2] - mn1); s[nb][3] = exp2f(s[nb][3] - mn1);
      rs0 += s[nb][0] + s[nb][1];
      rs1 += s[nb][2] + s[nb][3];
    }
    l0 = l0 * al0 + rs0;
    l1 = l1 * al1 + rs1;
    if (!__all_sync(0xffffffffu, al0 == 1.f && al1 == 1.f)) {   // the running maxima usually settle early
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    }
    // ---- O += P V (one k-step of 16 tokens, 16 n-tiles of 8 dims) ----
    uint32_t a[4];
    a[0] = am_pack(s[0][0], s[0][1]);
    a[1] = am_pack(s[0][2], s[0][3]);
    a[2] = am_pack(s[1][0], s[1][1]);
    a[3] = am_pack(s[1][2], s[1][3]);
#pragma unroll
    for (int db = 0; db < 16; db += 2) {
      uint32_t b0, b1, b2, b3;
      am_ldsm_x4_t(vb + am_swz((mat & 1) * 8 + (lane & 7), db + (mat >> 1)), b0, b1, b2, b3);
      am_mma(o[db], a, b0, b1);
      am_mma(o[db + 1], a, b2, b3);
    }
  }
  am_wait<0>();
  __syncthreads();   // every warp is done with its stages: they become the merge scratch

  // ---- park each warp's (m, l, O[16][128]) in shared memory ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* o_w = reinterpret_cast<float*>(am_smem + warp * AM_WARP_BYTES);   // [16][128] fp32 = 8 KB
  float* ml_w = o_w + 16 * AM_D;                                           // [16][2]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int db = 0; db < 16; ++db) {
      const int d = db * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(&o_w[r0 * AM_D + d]) = make_float2(o[db][0], o[db][1]);
      *reinterpret_cast<float2*>(&o_w[r1 * AM_D + d]) = make_float2(o[db][2], o[db][3]);
    }
    if ((lane & 3) == 0) {
      ml_w[r0 * 2] = m0; ml_w[r0 * 2 + 1] = l0;
      ml_w[r1 * 2] = m1; ml_w[r1 * 2 + 1] = l1;
    }
  }
  __syncthreads();

  // ---- merge the 4 warps: thread d owns output dim d of every head ----
  const int d = tid;
  float O_g[16], M_g[16], L_g[16];
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    O_g[g] = 0.f; M_g[g] = -INFINITY; L_g[g] = 0.f;
    if (g < G) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < AM_WARPS; ++w)
        M = fmaxf(M, reinterpret_cast<const float*>(am_smem + w * AM_WARP_BYTES)[16 * AM_D + g * 2]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < AM_WARPS; ++w) {
        const float* ow = reinterpret_cast<const float*>(am_smem + w * AM_WARP_BYTES);
        const float mw = ow[16 * AM_D + g * 2];
        const float wt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += wt * ow[16 * AM_D + g * 2 + 1];
        O += wt * ow[g * AM_D + d];
      }
      O_g[g] = O; M_g[g] = M; L_g[g] = L;
    }
  }
  if (p.splits == 1) {
#pragma unroll
    for (int g = 0; g < 16; ++g)
      if (g < G) p.out[((size_t)b * p.Hq + kvh * G + g) * AM_D + d] = __float2bfloat16(L_g[g] > 0.f ? O_g[g] / L_g[g] : 0.f);
    return;
  }
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    if (g < G) {
      const size_t base = ((size_t)b * p.Hq + kvh * G + g) * p.splits + split;
      p.ws_o[base * AM_D + d] = O_g[g];
      if (d == 0) { p.ws_ml[base * 2] = M_g[g]; p.ws_ml[base * 2 + 1] = L_g[g]; }
    }
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
  // last CTA of this (sequence, kv head): merge the splits. (m, l) of all heads and splits are staged in
  // shared memory with one parallel load; each thread then fetches its dim of all splits at once.
  float* ml_s = reinterpret_cast<float*>(am_smem);   // [G][splits][2]
  const size_t base0 = ((size_t)b * p.Hq + kvh * G) * p.splits;
  for (int i = tid; i < G * p.splits * 2; i += AM_THREADS) ml_s[i] = __ldcg(&p.ws_ml[base0 * 2 + i]);
  __syncthreads();
  for (int g = 0; g < G; ++g) {
    const size_t base = base0 + (size_t)g * p.splits;
    float ov[AM_MAX_SPLITS];
#pragma unroll
    for (int s2 = 0; s2 < AM_MAX_SPLITS; ++s2) ov[s2] = (s2 < p.splits) ? __ldcg(&p.ws_o[(base + s2) * AM_D + d]) : 0.f;
    float M = -INFINITY;
    for (int s2 = 0; s2 < p.splits; ++s2) M = fmaxf(M, ml_s[(g * p.splits + s2) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < AM_MAX_SPLITS; ++s2) {
      if (s2 < p.splits) {
        const float mi = ml_s[(g * p.splits + s2) * 2];
        const float w = (mi == -INFINITY) ? 0.f : exp2f(mi - M);
        L += w * ml_s[(g * p.splits + s2) * 2 + 1];
        O += w * ov[s2];
      }
    }
    p.out[((size_t)b * p.Hq + kvh * G + g) * AM_D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
  }
}

}  // namespace skein

// Same contract as skein_attn_decode (ws / counters from skein_attn_decode_workspace_floats; counters zero at
// first use). Requires D = 128, page_size a multiple of 16, at most 16 query heads per kv head.
static int attn_decode_mma_launch(const void* q, long long q_stride, void* kv, const int* block_table,
                                  const int* seq_lens, void* out, float* ws, int* counters, int* status, int B,
                                  int Hq, int Hkv, int D, int page_size, int max_blocks, int num_pages, int splits,
                                  float scale, const float* cos_sin, const int* positions, int max_pos, void* stream) {
  using namespace skein;
  if (B == 0) return 0;
  if (D != AM_D || Hq % Hkv != 0 || page_size % AM_TILE != 0) return -1;
  const int G = Hq / Hkv;
  if (G > 16) return -1;
  if (splits < 1 || splits > AM_MAX_SPLITS) return -2;
  if (splits > 1 && (ws == nullptr || counters == nullptr)) return -2;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -4;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         am_smem_bytes(3));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_mma_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, am_smem_bytes(6));
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  AttnMmaParams p;
  p.q = (const __nv_bfloat16*)q; p.kv = (const __nv_bfloat16*)kv; p.kv_rw = (__nv_bfloat16*)kv;
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.cos_sin = cos_sin; p.positions = positions; p.max_pos = max_pos;
  p.out = (__nv_bfloat16*)out; p.ws_o = ws; p.ws_ml = ws ? ws + (size_t)B * Hq * splits * AM_D : nullptr;
  p.counters = counters; p.status = status; p.q_stride = q_stride;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.page_size = page_size; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.splits = splits; p.scale_log2e = scale * 1.4426950408889634f;
  dim3 grid(splits, Hkv, B);
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  if ((long long)splits * Hkv * B <= sms)
    return (int)launch_pdl(attn_decode_mma_kernel<6>, grid, dim3(AM_THREADS), (size_t)am_smem_bytes(6), (cudaStream_t)stream, p);
  return (int)launch_pdl(attn_decode_mma_kernel<3>, grid, dim3(AM_THREADS), (size_t)am_smem_bytes(3), (cudaStream_t)stream, p);
}

extern "C" int skein_attn_decode_mma(const void* q, long long q_stride, const void* kv, const int* block_table,
                                     const int* seq_lens, void* out, float* ws, int* counters, int* status, int B,
                                     int Hq, int Hkv, int D, int page_size, int max_blocks, int num_pages, int splits,
                                     float scale, void* stream) {
  return attn_decode_mma_launch(q, q_stride, const_cast<void*>(kv), block_table, seq_lens, out, ws, counters, status, B,
                                Hq, Hkv, D, page_size, max_blocks, num_pages, splits, scale, nullptr, nullptr, 0, stream);
}

// Decode attention straight from the fused q/k/v projection: rotates q and k (rotate-half RoPE from the fp32
// cos/sin table), appends the new token's k and v rows to the paged cache and attends, in one launch.
// qkv rows: [q heads | k heads | v heads] x D; positions[b] = position of the new token (-1: padding row, whose
// seq_lens entry must be 0); seq_lens[b] = positions[b] + 1.
extern "C" int skein_attn_decode_rope_mma(const void* qkv, long long qkv_stride, void* kv, const int* block_table,
                                          const int* seq_lens, const int* positions, const float* cos_sin,
                                          int max_pos, void* out, float* ws, int* counters, int* status, int B, int Hq,
                                          int Hkv, int D, int page_size, int max_blocks, int num_pages, int splits,
                                          float scale, void* stream) {
  if (cos_sin == nullptr || positions == nullptr) return -1;
  return attn_decode_mma_launch(qkv, qkv_stride, kv, block_table, seq_lens, out, ws, counters, status, B, Hq, Hkv, D,
                                page_size, max_blocks, num_pages, splits, scale, cos_sin, positions, max_pos, stream);
}
