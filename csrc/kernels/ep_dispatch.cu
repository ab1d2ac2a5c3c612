// Expert-parallel token dispatch over peer memory.
//
// With data-parallel attention every expert-parallel rank owns a slice of the step's sequences: it runs attention,
// the residual/RMSNorm and the router for its own `per` tokens only, writes the normalised rows and the router's
// expert choices into its published (peer-mapped) buffer and raises its flag. This kernel is the receiving half
// of the dispatch, one launch on every rank:
//
//   1. wait (bounded) for every rank's flag,
//   2. read all ranks' expert choices (T * k integers) and derive the same global expert-sorted layout on every
//      rank: counts, exclusive offsets, and for pair (t, j) the row  offsets[e] + #earlier pairs routed to e,
//      which is the stable order of the single-GPU router (router.cu, norm.cu),
//   3. for every pair routed to one of THIS rank's experts, pull the token's normalised row out of its owner's
//      buffer over NVLink (plain peer loads, every 16-byte load of a row in flight at once) into the local
//      expert-sorted activation matrix that the grouped expert GEMM reads.
//
// Only rows that an expert here needs cross NVLink (T * k / ep of them on average), nothing is staged through the
// host, and no count exchange precedes the data: the layout is recomputed from the published choices. The combine
// half already exists: the grouped down projection publishes its rows and the combine in norm.cu pulls each
// (token, slot) row from the rank that owns the expert.
//
// The reference describes this dispatch in its cost model (two all-to-alls per MoE block,
// crates/skein_cost/src/comm.rs:65-151) and ships the dispatch/combine math as an unwired graph
// (crates/skein_emit/src/op_wiring.rs:1741, tests crates/skein_emit/tests/ep_routing.rs:14,68).
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace skein {

constexpr int EPD_MAXP = 8;
constexpr int EPD_MAX_PAIRS = 2048;
constexpr int EPD_MAX_E = 64;
constexpr int EPD_THREADS = 128;

struct EpDispatchParams {
  const __nv_bfloat16* src_rows[EPD_MAXP];   // rank s's published normalised rows [per, H]
  const int* src_ids[EPD_MAXP];              // rank s's published expert choices [per, k]
  const int* flags;                          // [n_src] local flag words written by the ranks
  const int* epoch;
  int* status;
  unsigned long long budget_ns;
  int n_src, per, k, E, e_first, e_count, H;
  int* ids_all;        // [T, k]
  int* counts;         // [E]
  int* offsets;        // [E + 1]
  int* row_of;         // [T * k] global expert-sorted row of every pair
  int* src_token;      // [T * k] token of every row that belongs to one of this rank's experts
  __nv_bfloat16* xs;   // [T * k, H] rows of this rank's experts, at their global positions
};

// One CTA per (token, slot) pair.
__global__ void __launch_bounds__(EPD_THREADS) ep_dispatch_pull_kernel(const EpDispatchParams p) {
  __shared__ int ids_s[EPD_MAX_PAIRS];
  __shared__ int cnt_s[EPD_MAX_E];
  __shared__ int red[EPD_THREADS / 32];
  __shared__ int wait_failed;
  const int tid = threadIdx.x;
  const int n_pairs = p.n_src * p.per * p.k;
  if (tid == 0) wait_failed = 0;
  for (int e = tid; e < p.E; e += EPD_THREADS) cnt_s[e] = 0;
  __syncthreads();
  if (tid < p.n_src) {
    const bool poisoned = p.status != nullptr && *(volatile int*)p.status == ST_TIMEOUT_PEER_FLAG;
    if (poisoned || !wait_flag_ge(p.flags + tid, *p.epoch, p.budget_ns)) {
      report_status(p.status, ST_TIMEOUT_PEER_FLAG, tid);
      wait_failed = 1;
    }
  }
  __syncthreads();
  if (wait_failed) return;
  const int per_pairs = p.per * p.k;
  for (int i = tid; i < n_pairs; i += EPD_THREADS) {
    const int s = i / per_pairs;
    int e;
    // written by another GPU: bypass L1
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(e) : "l"(p.src_ids[s] + (i - s * per_pairs)));
    if (e < 0 || e >= p.E) { report_status(p.status, ST_BAD_INDEX, i); e = 0; }
    ids_s[i] = e;
    atomicAdd(&cnt_s[e], 1);
  }
  __syncthreads();
  const int me = blockIdx.x;              // this CTA's pair
  const int my_e = ids_s[me];
  int before = 0;
  for (int i = tid; i < me; i += EPD_THREADS) before += (ids_s[i] == my_e);
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  if ((tid & 31) == 0) red[tid >> 5] = before;
  __syncthreads();
  int row = 0;
  for (int w = 0; w < EPD_THREADS / 32; ++w) row += red[w];
  for (int e = 0; e < my_e; ++e) row += cnt_s[e];
  const bool mine = my_e >= p.e_first && my_e < p.e_first + p.e_count;
  const int t = me / p.k;
  if (tid == 0) {
    p.row_of[me] = row;
    p.ids_all[me] = my_e;
    if (mine) p.src_token[row] = t;
    if (me == 0) {
      int a = 0;
      for (int e = 0; e < p.E; ++e) { p.counts[e] = cnt_s[e]; p.offsets[e] = a; a += cnt_s[e]; }
      p.offsets[p.E] = a;
    }
  }
  if (!mine) return;
  const int s = t / p.per;
  const uint4* src = reinterpret_cast<const uint4*>(p.src_rows[s] + (size_t)(t - s * p.per) * p.H);
  uint4* dst = reinterpret_cast<uint4*>(p.xs + (size_t)row * p.H);
  const int n_vec = p.H / 8;
  // batches of four loads per thread are issued before the first store
  for (int v0 = tid; v0 < n_vec; v0 += 4 * EPD_THREADS) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * EPD_THREADS;
      if (v < n_vec)
        asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(src + v));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * EPD_THREADS;
      if (v < n_vec) dst[v] = r[u];
    }
  }
}

}  // namespace skein

// src_rows[s] / src_ids[s]: rank s's published rows and expert choices as mapped in this process. T = n_src * per
// tokens in rank order. Returns 0, a cudaError_t, or -1 for arguments out of range.
extern "C" int skein_ep_dispatch_pull(const void* const* src_rows, const void* const* src_ids, int n_src, int per, int k, int E,
                                      int e_first, int e_count, int H, const int* flags, const int* epoch, int* status,
                                      int budget_ms, int* ids_all, int* counts, int* offsets, int* row_of, int* src_token,
                                      void* xs, void* stream) {
  using namespace skein;
  if (n_src < 1 || n_src > EPD_MAXP || per < 1 || k < 1 || E < 1 || E > EPD_MAX_E || H % 8 != 0) return -1;
  if ((long long)n_src * per * k > EPD_MAX_PAIRS) return -1;
  EpDispatchParams p;
  for (int s = 0; s < EPD_MAXP; ++s) {
    p.src_rows[s] = s < n_src ? (const __nv_bfloat16*)src_rows[s] : nullptr;
    p.src_ids[s] = s < n_src ? (const int*)src_ids[s] : nullptr;
  }
  p.flags = flags; p.epoch = epoch; p.status = status;
  p.budget_ns = (unsigned long long)(budget_ms > 0 ? budget_ms : 10000) * 1000000ull;
  p.n_src = n_src; p.per = per; p.k = k; p.E = E; p.e_first = e_first; p.e_count = e_count; p.H = H;
  p.ids_all = ids_all; p.counts = counts; p.offsets = offsets; p.row_of = row_of; p.src_token = src_token;
  p.xs = (__nv_bfloat16*)xs;
  ep_dispatch_pull_kernel<<<n_src * per * k, EPD_THREADS, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
