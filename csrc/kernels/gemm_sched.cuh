// Work decomposition shared by the weight-streaming GEMM kernels (bf16 and block-scaled fp8).
//
// A "unit" is one output tile: (group g, feature tile m of 128 rows, token tile n of n_tile rows). Units are
// ordered group-major, inside a group as decode_unit says, and each owns KB consecutive K-blocks of one long
// line of K-blocks.
// Two ways to deal the line to the CTAs:
//   * line cut (stream-K): CTA c processes K-blocks [c * per, (c + 1) * per). Balanced for any tile count, but
//     a CTA's range usually straddles a tile boundary, so it parks and reduces two partial tiles.
//   * tile-aligned (only when there are no more tiles than CTAs): each tile is cut into `split` near-equal
//     pieces owned by `split` consecutive CTAs, so every CTA has exactly one piece of one tile.
// Group sizes are read from device memory, so every CTA rebuilds the same table at start-up.
#pragma once
#include "gemm_ws.cuh"
#include "ptx.cuh"
#include <cuda.h>

namespace skein {

struct Sched {
  int pre[SKEIN_MAX_GROUPS + 1];  // first unit of each group
  int cnt[SKEIN_MAX_GROUPS];
  int off[SKEIN_MAX_GROUPS];
  int ntile[SKEIN_MAX_GROUPS];
  int MT, KB, U, per;
  int split;   // > 0: tile-aligned with this many CTAs per tile; 0: line cut with `per` K-blocks per CTA
  long long TK;
};

struct Unit { int g, m, n; };

// Units of a group are numbered in bands of RASTER_BAND feature tiles: inside a band the feature tile runs
// fastest, then the token tile. The ~148 units in flight at any time then cover about 12 x 12 tiles
// (12 weight tiles + 12 activation tiles to fetch) instead of 4 x 32, and a band re-reads its weight tiles
// from L2 while it walks the token tiles: a prefill-sized projection (8192 tokens x 6144 features) moved 2.5 GB
// through DRAM for 218 MB of operands with token-fastest numbering. With one token tile per group (decode)
// the numbering is the plain feature-tile order.
constexpr int RASTER_BAND = 12;

__device__ __forceinline__ Unit decode_unit(const Sched& s, int G, int u) {
  int g = 0;
  while (g + 1 < G && u >= s.pre[g + 1]) ++g;
  const int r = u - s.pre[g];
  const int nt = s.ntile[g];
  Unit x;
  x.g = g;
  if (nt == 1) { x.m = r; x.n = 0; return x; }
  const int band_units = RASTER_BAND * nt;
  const int band = r / band_units;
  const int rb = r - band * band_units;
  int bm = s.MT - band * RASTER_BAND;      // feature tiles in this band (the last one may be short)
  if (bm > RASTER_BAND) bm = RASTER_BAND;
  x.n = rb / bm;
  x.m = band * RASTER_BAND + (rb - x.n * bm);
  return x;
}

// K-block range of CTA c on the line, the CTAs that share tile u, and which of its two workspace slots CTA c
// uses for tile u (slot 0: the tile its range begins in).
// (32-bit arithmetic: these run on every segment of every role, and 64-bit divisions cost microseconds there;
//  build_sched refuses a line of 2^31 K-blocks or more.)
__device__ __forceinline__ int cta_begin(const Sched& s, int c) {
  const int tk = (int)s.TK;
  if (s.split > 0) {
    const int u = c / s.split, pc = c - u * s.split;
    if (u >= s.U) return tk;
    return u * s.KB + pc * s.KB / s.split;
  }
  const long long b = (long long)c * s.per;
  return b < tk ? (int)b : tk;
}
__device__ __forceinline__ int cta_end(const Sched& s, int c) {
  const int tk = (int)s.TK;
  if (s.split > 0) {
    const int u = c / s.split, pc = c - u * s.split;
    if (u >= s.U) return tk;
    return u * s.KB + (pc + 1) * s.KB / s.split;
  }
  const long long e = (long long)(c + 1) * s.per;
  return e < tk ? (int)e : tk;
}
__device__ __forceinline__ void tile_ctas(const Sched& s, int u, int& c_first, int& c_last) {
  if (s.split > 0) { c_first = u * s.split; c_last = c_first + s.split - 1; return; }
  const int ub = u * s.KB;
  c_first = ub / s.per;
  c_last = (ub + s.KB - 1) / s.per;
}
__device__ __forceinline__ int cta_slot(const Sched& s, int c, int u) { return cta_begin(s, c) / s.KB == u ? 0 : 1; }

// Fills the table (one thread). k_elems_per_block: 64 for bf16, 128 for e4m3.
__device__ __forceinline__ void build_sched(Sched& sched, const SkeinGemmParams& p, int k_elems_per_block, int grid,
                                            bool allow_aligned = false) {
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
  if (sched.TK >= (1ll << 31)) {   // no work is handed out; the host sees the status
    report_status(p.status, ST_BAD_INDEX, acc);
    sched.U = 0;
    sched.TK = 0;
  }
  // equal share per CTA, but never so small that a tile is cut into more than 8 pieces
  long long per = (sched.TK + grid - 1) / grid;
  const long long min_per = sched.KB >= 32 ? sched.KB / 8 : 4;
  if (per < min_per) per = min_per;
  sched.per = (int)per;
  sched.split = 0;
  if (allow_aligned && acc > 0 && acc <= grid) {
    int sp = grid / acc;
    if (sp > 8) sp = 8;
    const int by_k = sched.KB / 4 > 0 ? sched.KB / 4 : 1;   // at least 4 K-blocks per piece
    if (sp > by_k) sp = by_k;
    // with fewer than two CTAs per tile, whole tiles on `acc` CTAs beat the line cut while the longer
    // K loop costs less than the second partial tile that the line cut's straddling brings
    if (sp >= 2 || (long long)sched.KB * (grid - acc) < 30ll * grid) sched.split = sp;
  }
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// host helpers defined in gemm_ws.cu
int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes, uint32_t box_rows);

}  // namespace skein
