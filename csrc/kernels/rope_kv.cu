// RoPE (NeoX "rotate-half" convention, the one HuggingFace Mixtral/Llama use) fused with the
// append of the new K and V rows into the paged KV cache, and the embedding gather.
//
// qkv is the output of the fused q/k/v projection: [T, (Hq + 2*Hkv) * D] bf16, laid out per token
// as q heads, then k heads, then v heads. q is rotated in place; k is rotated and written, with v,
// through the block table into
//     kv_cache[page, 0 = K / 1 = V, kv_head, slot_in_page, D]        (bf16)
// cos/sin come from a host-built fp32 table [max_pos, D/2] so that large positions keep full
// accuracy regardless of fast-math flags.
//
// Replaces the reference's rope_kernel (vendor/luminal/crates/luminal_cuda_lite/src/kernel/
// rope.rs:55-85, interleaved-pair convention), the graph-level apply_rope
// (crates/skein_emit/src/op_wiring.rs:2431-2472) and kv_slot_write[_batched]
// (vendor/luminal/crates/luminal_cuda_lite/src/runtime.rs:900-909,1026-1041).
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace skein {

// grid = (T, Hq + 2*Hkv); block = D/2 threads (one rotation pair each).
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token,   // [T] row of block_table, or null (= token)
                                      const int* __restrict__ block_table, int max_blocks,
                                      const float* __restrict__ cos_sin,      // [max_pos, D/2, 2]
                                      __nv_bfloat16* __restrict__ kv_cache, int page_size, int Hq, int Hkv, int D,
                                      int max_pos, int num_pages, int* status) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;
  const int i = threadIdx.x;
  const int half = D / 2;
  if (i >= half) return;
  int pos = positions[t];
  if (pos < 0) return;  // padding row of a captured batch bucket
  if (pos >= max_pos) { report_status(status, ST_BAD_INDEX, pos); return; }
  __nv_bfloat16* row = qkv + (size_t)t * (Hq + 2 * Hkv) * D + (size_t)head * D;
  float x0 = __bfloat162float(row[i]);
  float x1 = __bfloat162float(row[i + half]);
  if (head < Hq + Hkv) {
    const float2 cs = reinterpret_cast<const float2*>(cos_sin)[(size_t)pos * half + i];
    const float y0 = x0 * cs.x - x1 * cs.y;
    const float y1 = x1 * cs.x + x0 * cs.y;
    x0 = y0; x1 = y1;
  }
  if (head < Hq) {
    row[i] = __float2bfloat16(x0);
    row[i + half] = __float2bfloat16(x1);
    return;
  }
  const int is_v = head >= Hq + Hkv;
  const int kvh = head - Hq - (is_v ? Hkv : 0);
  const int seq = seq_of_token ? seq_of_token[t] : t;
  const int page = block_table[(size_t)seq * max_blocks + pos / page_size];
  if (page < 0 || page >= num_pages) { report_status(status, ST_BAD_INDEX, page); return; }
  __nv_bfloat16* dst = kv_cache + ((((size_t)page * 2 + is_v) * Hkv + kvh) * page_size + pos % page_size) * D;
  dst[i] = __float2bfloat16(x0);
  dst[i + half] = __float2bfloat16(x1);
}

// out[t, :] = table[ids[t] - vocab_start, :] if the id falls in this rank's vocabulary shard, else 0.
__global__ void embed_gather_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                    __nv_bfloat16* __restrict__ out, int H, int vocab_start, int vocab_rows) {
  const int t = blockIdx.x;
  const int id = ids[t] - vocab_start;
  const bool mine = id >= 0 && id < vocab_rows;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(mine ? id : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int h = threadIdx.x; h < H / 8; h += blockDim.x) dst[h] = mine ? src[h] : zero;
}

// Gather rows: out[r, :] = in[src_row[r], :]   (expert-sorted copy of the token activations)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ in, const int* __restrict__ src_row,
                                   __nv_bfloat16* __restrict__ out, int H, int n_rows_max, const int* n_rows_dev) {
  const int r = blockIdx.x;
  const int n = n_rows_dev ? *n_rows_dev : n_rows_max;
  if (r >= n) return;
  const int s = src_row[r];
  const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)s * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * H);
  for (int h = threadIdx.x; h < H / 8; h += blockDim.x) dst[h] = src[h];
}

}  // namespace skein

extern "C" int skein_rope_kv_append(void* qkv, const int* positions, const int* seq_of_token, const int* block_table,
                                    int max_blocks, const float* cos_sin, void* kv_cache, int page_size, int T, int Hq,
                                    int Hkv, int D, int max_pos, int num_pages, int* status, void* stream) {
  if (T == 0) return 0;
  if (D % 2 != 0 || D / 2 > 1024) return -1;
  dim3 grid(T, Hq + 2 * Hkv);
  skein::rope_kv_append_kernel<<<grid, D / 2, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)qkv, positions, seq_of_token, block_table, max_blocks, cos_sin, (__nv_bfloat16*)kv_cache,
      page_size, Hq, Hkv, D, max_pos, num_pages, status);
  return (int)cudaGetLastError();
}

extern "C" int skein_embed_gather(const int* ids, const void* table, void* out, int T, int H, int vocab_start,
                                  int vocab_rows, void* stream) {
  if (T == 0) return 0;
  if (H % 8 != 0) return -1;
  skein::embed_gather_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(ids, (const __nv_bfloat16*)table,
                                                                  (__nv_bfloat16*)out, H, vocab_start, vocab_rows);
  return (int)cudaGetLastError();
}

extern "C" int skein_gather_rows(const void* in, const int* src_row, void* out, int n_rows_max, int H,
                                 const int* n_rows_dev, void* stream) {
  if (n_rows_max == 0) return 0;
  if (H % 8 != 0) return -1;
  skein::gather_rows_kernel<<<n_rows_max, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)in, src_row, (__nv_bfloat16*)out, H, n_rows_max, n_rows_dev);
  return (int)cudaGetLastError();
}
