// Parameter block shared by the weight-streaming GEMM kernel, its C launchers and the ctypes
// mirror in skein_b200/ops/_lib.py (keep the field order identical there).
#pragma once
#include <stdint.h>

#define SKEIN_MAX_PEERS 8
#define SKEIN_MAX_GROUPS 64

extern "C" {

// Y_g[t, f] = sum_k X[off_g + t, k] * W[g * w_rows_per_group + f, k]      (t < cnt_g, f < F)
// W and X are row-major with K contiguous ("K-major"); both bf16, or both e4m3 when fp8 != 0.
typedef struct SkeinGemmParams {
  const void* W;            // [G * w_rows_per_group, K]
  const void* X;            // [x_rows, K]
  void* out;                // bf16 [*, ldo]: row = off_g + t, column = out_col0 + f
  const void* residual;     // optional bf16, same indexing as out (added before the store)
  const int32_t* group_off; // device [G] first X/out row of each group; null -> 0
  const int32_t* group_cnt; // device [G] rows in each group; null -> t_static for every group
  float* workspace;         // stream-K partial tiles: grid * 2 * 128 * acc_cols floats
  int32_t* counters;        // stream-K arrival counters: grid ints, zero at first use
  int32_t* status;          // 2 ints: error code (0 = ok) and detail
  // fp8 block scales (fp8 != 0): one float per 128 K-elements.
  const float* w_scale;     // [G * w_rows_per_group, K / 128]
  const float* x_scale;     // [x_rows, K / 128]
  // publish (mode 2): the result is stored locally (out, a buffer that the peers have mapped) and, once every
  // CTA is done, this rank's flag word on each peer is set; the consumers pull the partials over NVLink.
  int32_t* peer_flag[SKEIN_MAX_PEERS];  // flag word on each peer (this rank included) that this rank sets
  int32_t* epoch;           // device int: last epoch published through peer_flag
  int32_t* done_counter;    // device int, zero at first use
  int32_t n_peers;
  int32_t G, F, K;
  int32_t w_rows_per_group;
  int32_t up_row_off;       // dual: row offset of the "up" half inside a group (gate rows first)
  int32_t x_rows;           // rows of X (TMA bound)
  int32_t t_static;
  int32_t n_tile;           // tokens per tile: multiple of 16, <= 256 (<= 128 when dual)
  int32_t ldo;
  int32_t out_col0;
  int32_t mode;             // 0 store, 1 SwiGLU(gate, up) store (dual), 2 store + publish flags to peers
  int32_t fp8;
  int32_t stages;           // 0 -> as many as fit
  int32_t grid;             // 0 -> number of SMs
  int32_t wait_budget_ms;   // 0 -> 2000
  int32_t w_packed;         // W is stored tile by tile: [rows/128][K/64 (or /128 fp8)][128][128 bytes]
  int32_t line_cut_only;    // 1: never use the tile-aligned split (see gemm_sched.cuh), for comparison runs
} SkeinGemmParams;

// Returns 0 or a cudaError_t / negative argument-error code.
int skein_gemm_ws(const SkeinGemmParams* p, void* stream);
// Bytes of workspace and number of counters skein_gemm_ws needs for these parameters.
int64_t skein_gemm_ws_workspace_bytes(const SkeinGemmParams* p);
int skein_sm_count(void);

}  // extern "C"
