/* Allocation-free entry point for split-KV paged decode attention.
 *
 * This entry point has no counterpart in the reference project. It exists for callers that must not
 * allocate device memory at the point where they run attention: code executing inside a memory-pool or
 * arena discipline that forbids cudaMalloc after start-up, plug-ins loaded into a host process whose
 * allocator owns the whole device, or latency-critical loops where an allocator call (which may
 * synchronise the device) is not acceptable. Such callers cannot hand skein_attn_decode the workspace
 * and counter buffers that its split-KV merge needs.
 *
 * skein_attn_decode_noalloc computes exactly what skein_attn_decode computes, but the split-KV scratch
 * (per-split partial outputs, running maxima and sums, and the per-(sequence, kv head) arrival counters)
 * lives in a fixed array inside the library image instead of caller memory. Inputs and outputs are still
 * the caller's.
 *
 * Limits and rules
 *   - Capacity is fixed at build time: B * Hq * splits <= SKEIN_ATTN_NOALLOC_MAX_ROWS (8192),
 *     B * Hkv <= SKEIN_ATTN_NOALLOC_MAX_COUNTERS (4096) and splits <= 16. The scratch occupies about 4.3 MB of device
 *     memory on every GPU that loads this library, from load until the process exits. A call that exceeds
 *     the capacity is refused with SKEIN_NOALLOC_ERR_TOO_LARGE and touches nothing.
 *   - The function calls no cudaMalloc / cudaFree and no allocating library routine. The first call on a
 *     device looks up the device address of the built-in scratch (one cudaGetSymbolAddress per array, with
 *     that device current) and remembers it; make that first call outside any CUDA stream capture. Two host
 *     threads that make their first call on the same device at the same time both perform the look-up and
 *     both store the same address (a benign double write of one pointer-sized value; no lock is taken).
 *   - All calls on a device share the one scratch array, and it keeps whatever the previous call left in
 *     it. Each call clears the arrival counters on `stream` before launching. Two calls whose kernels can
 *     overlap on the GPU (different streams, or different host threads without ordering) race on the
 *     scratch and give wrong results: serialise them on one stream or with events.
 *   - Arguments have the meaning they have in skein_attn_decode (attn_decode.cu). D must be 128.
 *
 * Returns 0 on success, a positive cudaError_t from the runtime, or one of the negative codes below;
 * skein_attn_decode_noalloc_strerror gives a text for the negative ones.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define SKEIN_ATTN_NOALLOC_MAX_ROWS 8192
#define SKEIN_ATTN_NOALLOC_MAX_COUNTERS 4096

#define SKEIN_NOALLOC_ERR_BAD_ARGS (-1)
#define SKEIN_NOALLOC_ERR_TOO_LARGE (-2)
#define SKEIN_NOALLOC_ERR_UNSUPPORTED_GROUP (-3)
#define SKEIN_NOALLOC_ERR_DEVICE (-4)

int skein_attn_decode_noalloc(const void* q, long long q_stride, const void* kv, const int* block_table,
                              const int* seq_lens, void* out, int* status, int B, int Hq, int Hkv, int D,
                              int page_size, int max_blocks, int num_pages, int splits, float scale, void* stream);

const char* skein_attn_decode_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
