// Peer-memory plumbing and the small stand-alone collectives.
//
//   * symmetric heap: every rank cudaMallocs one heap and exports a CUDA IPC handle; peers map it,
//     so kernels address a peer's buffer with plain loads/stores that travel over NVLink.
//   * publish_rows: copy a local tensor into this rank's peer-mapped buffer and set this rank's flag on
//     every peer. Followed by reduce_residual_rmsnorm (norm.cu), which pulls every rank's buffer over
//     NVLink and sums, it is a one-shot all-reduce; the fused path publishes from the GEMM epilogue.
//   * argmax_push: vocabulary-parallel greedy sampling. Each rank reduces its logit shard to one
//     (value, global index) pair per row and pushes 8 bytes per row to every peer
//     (merge_candidates in sample.cu picks the winner).
//   * pull_collective: after a publish, all-gather / reduce-scatter / all-to-all as ONE pull kernel: wait
//     (bounded) for every rank's flag, then read the chunks this rank needs straight out of the peers'
//     published buffers, eight 16-byte peer loads in flight per thread, summing in rank order where the
//     collective reduces.
//   * copy_pages: KV pages to (or from) a peer's cache, for prefill/decode disaggregation.
// Flags carry monotonically increasing epochs kept in device memory, so the same launches replay
// inside a CUDA graph. Every wait on a flag is bounded (ptx.cuh: wait_flag_ge).
//
// Replaces the reference's NCCL all-reduce + copy-back (crates/skein_runtime/src/cuda/nccl.rs:196-245),
// its 2-rank host-shared-memory all-reduce with an unbounded spin (crates/skein_runtime/src/cuda/
// shm_allreduce.rs:24-69), the logits all-gather (nccl.rs:251-298), the grouped send/recv exchanges
// (nccl.rs:422-445) and the host-staged KV block transport (nccl.rs:504-588).
#include "ptx.cuh"
#include "argmax.cuh"
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>

namespace skein {

constexpr int MAXP = 8;

struct PeerPtrs {
  int* flag[MAXP];   // this rank's flag word on every rank of the group (its own included)
  int n;
};

// Publishes epoch+1 on every peer once all CTAs of the launch have finished their stores.
__device__ __forceinline__ void publish_when_all_done(const PeerPtrs& pp, int* epoch, int* done_counter) {
  __threadfence_system();   // this launch may have written into peers' memory (argmax candidates)
  __syncthreads();
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y * gridDim.z;
    const int old = atomicAdd(done_counter, 1);
    if (old == total - 1) {
      *done_counter = 0;
      __threadfence_system();
      const int e = *epoch + 1;
      for (int i = 0; i < pp.n; ++i) st_relaxed_sys(pp.flag[i], e);   // ordered by the fence above
      *epoch = e;
    }
  }
}

__global__ void __launch_bounds__(256) publish_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst_local,
                                                            long long n_vec, PeerPtrs pp, int* epoch, int* done_counter) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x)
    dst_local[i] = src[i];
  publish_when_all_done(pp, epoch, done_counter);
}


// grid = B rows, 1024 threads. val_dst[p] / idx_dst[p] point at this rank's [B] slot on peer p.
struct CandPtrs {
  float* val[MAXP];
  int* idx[MAXP];
};
__global__ void __launch_bounds__(1024) argmax_push_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int V,
                                                            int idx_offset, CandPtrs cp, PeerPtrs pp, int* epoch,
                                                            int* done_counter) {
  __shared__ ValIdx sh[32];
  const int b = blockIdx.x;
  const __nv_bfloat16* row = logits + (size_t)b * ld;
  const ValIdx r = block_argmax(thread_argmax_row(row, V), sh);
  if (threadIdx.x == 0) {
    for (int p = 0; p < pp.n; ++p) { cp.val[p][b] = r.v; cp.idx[p][b] = r.i + idx_offset; }
  }
  publish_when_all_done(pp, epoch, done_counter);
}

// One CTA per page: dst_cache[dst_page[i]] = src_cache[src_page[i]] (either side may be peer memory).
__global__ void __launch_bounds__(256) copy_pages_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                          const int* __restrict__ src_page, const int* __restrict__ dst_page,
                                                          long long vec_per_page) {
  const uint4* s = src + (long long)src_page[blockIdx.x] * vec_per_page;
  uint4* d = dst + (long long)dst_page[blockIdx.x] * vec_per_page;
  for (long long i = threadIdx.x; i < vec_per_page; i += blockDim.x) d[i] = s[i];
}

// ---- pull collectives ---------------------------------------------------------------------------------
// Every rank has published a buffer of `n_chunks_src` chunks of `chunk_vec` 16-byte vectors (src[s] is rank s's
// buffer as this process maps it). What this rank pulls:
//   PULL_ALL_GATHER      (1 chunk per source):  out[s][i] = src[s][i]
//   PULL_ALL_TO_ALL      (N chunks per source): out[s][i] = src[s][rank][i]
//   PULL_REDUCE_SCATTER  (N chunks per source): out[i]    = sum over s (rank order, fp32) of src[s][rank][i], bf16
enum { PULL_ALL_GATHER = 0, PULL_ALL_TO_ALL = 1, PULL_REDUCE_SCATTER = 2 };

struct PullParams {
  const uint4* src[MAXP];
  uint4* out;
  const int* flags;       // [n_src] local flag words, written by the peers
  const int* epoch;       // epoch the flags must have reached (this rank's own publish count)
  int* status;
  unsigned long long budget_ns;
  long long chunk_vec;
  int n_src, rank, mode;
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
}

__global__ void __launch_bounds__(256) pull_collective_kernel(const PullParams p) {
  __shared__ int wait_failed;
  if (threadIdx.x == 0) wait_failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < p.n_src) {
    const bool poisoned = p.status != nullptr && *(volatile int*)p.status == ST_TIMEOUT_PEER_FLAG;
    if (poisoned || !wait_flag_ge(p.flags + threadIdx.x, *p.epoch, p.budget_ns)) {
      report_status(p.status, ST_TIMEOUT_PEER_FLAG, threadIdx.x);
      wait_failed = 1;
    }
  }
  __syncthreads();
  if (wait_failed) return;   // the output keeps its old contents; the host reads the status word
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long own = p.mode == PULL_ALL_GATHER ? 0 : (long long)p.rank * p.chunk_vec;
  if (p.mode == PULL_REDUCE_SCATTER) {
    for (long long i = first; i < p.chunk_vec; i += stride) {
      uint4 v[MAXP];
#pragma unroll
      for (int s = 0; s < MAXP; ++s)
        if (s < p.n_src) v[s] = p.src[s][own + i];          // all sources in flight before the first add
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < MAXP; ++s)
        if (s < p.n_src) add_bf16x8(acc, v[s]);
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) ob[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      p.out[i] = o;
    }
  } else {
    for (long long i = first; i < p.chunk_vec; i += stride) {
      uint4 v[MAXP];
#pragma unroll
      for (int s = 0; s < MAXP; ++s)
        if (s < p.n_src) v[s] = p.src[s][own + i];
#pragma unroll
      for (int s = 0; s < MAXP; ++s)
        if (s < p.n_src) p.out[(long long)s * p.chunk_vec + i] = v[s];
    }
  }
}

// A wait that nothing satisfies within its budget: used to test the timeout path without a fault.
__global__ void wait_flag_kernel(const int* flag, int epoch, unsigned long long budget_ns, int* status) {
  if (!wait_flag_ge(flag, epoch, budget_ns)) report_status(status, ST_TIMEOUT_PEER_FLAG, 0);
}

}  // namespace skein

// ---- IPC heap -----------------------------------------------------------------------------------
extern "C" int skein_ipc_alloc(void** ptr, long long bytes) {
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, (size_t)bytes);
}
extern "C" int skein_ipc_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int skein_ipc_get_handle(void* ptr, void* handle_out_64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out_64, &h, sizeof(h));
  return 0;
}
extern "C" int skein_ipc_open(const void* handle_64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int skein_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int skein_ipc_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

// ---- collectives ----------------------------------------------------------------------------------
extern "C" int skein_publish_rows(const void* src, long long bytes, void* dst_local, int* const* peer_flag, int n_peers,
                                  int* epoch, int* done_counter, void* stream) {
  using namespace skein;
  if (bytes % 16 != 0 || n_peers < 1 || n_peers > MAXP) return -1;
  PeerPtrs pp;
  pp.n = n_peers;
  for (int i = 0; i < n_peers; ++i) pp.flag[i] = peer_flag[i];
  const long long n_vec = bytes / 16;
  int grid = (int)((n_vec + 255) / 256);
  if (grid > 296) grid = 296;
  if (grid < 1) grid = 1;
  publish_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst_local, n_vec, pp, epoch,
                                                             done_counter);
  return (int)cudaGetLastError();
}

// src_ptrs[s]: rank s's published buffer as mapped here; chunk_bytes: size of one chunk (a multiple of 16).
extern "C" int skein_pull_collective(int mode, const void* const* src_ptrs, int n_src, int rank, long long chunk_bytes,
                                     void* out, const int* flags, const int* epoch, int* status, int budget_ms,
                                     void* stream) {
  using namespace skein;
  if (n_src < 1 || n_src > MAXP || rank < 0 || rank >= n_src || chunk_bytes % 16 != 0 || mode < 0 || mode > 2) return -1;
  // chunk_bytes == 0: nothing to move, but the launch still waits for every rank's flag (an empty exchange)
  PullParams p;
  for (int s = 0; s < MAXP; ++s) p.src[s] = s < n_src ? (const uint4*)src_ptrs[s] : nullptr;
  p.out = (uint4*)out;
  p.flags = flags;
  p.epoch = epoch;
  p.status = status;
  p.budget_ns = (unsigned long long)(budget_ms > 0 ? budget_ms : 10000) * 1000000ull;
  p.chunk_vec = chunk_bytes / 16;
  p.n_src = n_src;
  p.rank = rank;
  p.mode = mode;
  long long grid = (p.chunk_vec + 255) / 256;
  if (grid < 1) grid = 1;
  if (grid > 592) grid = 592;   // 4 CTAs per SM: enough loads in flight to cover the NVLink round trip
  pull_collective_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

extern "C" int skein_argmax_push(const void* logits, long long ld, int B, int V, int idx_offset, float* const* peer_val,
                                 int* const* peer_idx, int* const* peer_flag, int n_peers, int* epoch,
                                 int* done_counter, void* stream) {
  using namespace skein;
  if (B == 0) return 0;
  if (n_peers < 1 || n_peers > MAXP) return -1;
  CandPtrs cp;
  PeerPtrs pp;
  pp.n = n_peers;
  for (int i = 0; i < n_peers; ++i) { cp.val[i] = peer_val[i]; cp.idx[i] = peer_idx[i]; pp.flag[i] = peer_flag[i]; }
  argmax_push_kernel<<<B, 1024, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V, idx_offset, cp, pp,
                                                           epoch, done_counter);
  return (int)cudaGetLastError();
}

extern "C" int skein_copy_pages(const void* src_cache, void* dst_cache, const int* src_page, const int* dst_page,
                                int n_pages, long long page_bytes, void* stream) {
  if (n_pages == 0) return 0;
  if (page_bytes % 16 != 0) return -1;
  skein::copy_pages_kernel<<<n_pages, 256, 0, (cudaStream_t)stream>>>((const uint4*)src_cache, (uint4*)dst_cache,
                                                                      src_page, dst_page, page_bytes / 16);
  return (int)cudaGetLastError();
}

extern "C" int skein_wait_flag(const int* flag, int epoch, int budget_ms, int* status, void* stream) {
  skein::wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, epoch, (unsigned long long)budget_ms * 1000000ull,
                                                             status);
  return (int)cudaGetLastError();
}
