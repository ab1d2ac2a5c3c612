// Work decomposition shared by the weight-streaming GEMM kernels (bf16 and block-scaled fp8).
//
// A "unit" is one output tile: (group g, feature tile m of 128 rows, token tile n of n_tile rows). Units are
// ordered group-major, then m, then n, and each owns KB consecutive K-blocks of one long line of K-blocks.
// CTA c processes K-blocks [c * per, (c + 1) * per) of that line (stream-K). Group sizes are read from
// device memory, so every CTA rebuilds the same table at start-up.
#pragma once
#include "gemm_ws.cuh"
#include <cuda.h>

namespace skein {

struct Sched {
  int pre[SKEIN_MAX_GROUPS + 1];  // first unit of each group
  int cnt[SKEIN_MAX_GROUPS];
  int off[SKEIN_MAX_GROUPS];
  int ntile[SKEIN_MAX_GROUPS];
  int MT, KB, U, per;
  long long TK;
};

struct Unit { int g, m, n; };

__device__ __forceinline__ Unit decode_unit(const Sched& s, int G, int u) {
  int g = 0;
  while (g + 1 < G && u >= s.pre[g + 1]) ++g;
  int r = u - s.pre[g];
  Unit x;
  x.g = g;
  x.m = r / s.ntile[g];
  x.n = r - x.m * s.ntile[g];
  return x;
}

// Fills the table (one thread). k_elems_per_block: 64 for bf16, 128 for e4m3.
__device__ __forceinline__ void build_sched(Sched& sched, const SkeinGemmParams& p, int k_elems_per_block, int grid) {
  const int G = p.G;
  const int MT = (p.F + 127) / 128;
  int acc = 0;
  for (int g = 0; g < G; ++g) {
    const int c = p.group_cnt ? p.group_cnt[g] : p.t_static;
    const int o = p.group_off ? p.group_off[g] : 0;
    const int nt = (c + p.n_tile - 1) / p.n_tile;
    sched.cnt[g] = c;
    sched.off[g] = o;
    sched.ntile[g] = nt > 0 ? nt : 1;  // never divide by zero; such a group has no units
    sched.pre[g] = acc;
    acc += MT * nt;
  }
  sched.pre[G] = acc;
  sched.MT = MT;
  sched.KB = p.K / k_elems_per_block;
  sched.U = acc;
  sched.TK = (long long)acc * sched.KB;
  // equal share per CTA, but never so small that a tile is cut into more than 8 pieces
  long long per = (sched.TK + grid - 1) / grid;
  const long long min_per = sched.KB >= 32 ? sched.KB / 8 : 4;
  if (per < min_per) per = min_per;
  sched.per = (int)per;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// host helpers defined in gemm_ws.cu
int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes, uint32_t box_rows);

}  // namespace skein
