// Internal interface between the C-ABI entry points (api.cu) and the three
// grouped-GEMM kernel families.
#pragma once
#include "common.cuh"

namespace fmoe {

using GemmParams = fmoe_gemm_args;

// gated = true : gemm1, w has 2*n rows per expert (gate rows then up rows), output
//                silu(gate)*up of width n, written at the sorted position p.
// gated = false: gemm2, w has n rows per expert, output written at row slot(p).
int gemm_simt(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_stream(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_tcgen05(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_tcgen05_fp8(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_tcgen05_pair(const GemmParams& p, bool gated, cudaStream_t st);

// true when the variant can run these arguments (shape / alignment / dtype rules)
bool gemm_stream_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_fp8_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_pair_supports(const GemmParams& p, bool gated);

// Tile order of the persistent kernels.  Tiles are walked in groups of `group_m` consecutive row blocks:
// inside a group the row block varies fastest, then the column tile, so that CTAs running at the same
// time share a weight tile through L2 while the group's activation rows (sized to fit L2) are re-read
// from L2, not HBM, for every column tile.
__device__ __forceinline__ void tile_to_mn(int64_t tile, int used_blocks, int n_tiles, int group_m, int* m_blk,
                                           int* n_tile) {
  const int64_t per_group = (int64_t)group_m * n_tiles;
  const int g = (int)(tile / per_group);
  const int r = (int)(tile % per_group);
  const int rows = min(group_m, used_blocks - g * group_m);
  *n_tile = r / rows;
  *m_blk = g * group_m + r % rows;
}
// Row blocks per group.  The `ctas` tiles that run at the same time form a group_m x (ctas/group_m)
// rectangle; its HBM traffic is one A block per row block plus one B tile per (expert, column tile)
// present.  Pick the group_m that minimises that, with the expected row blocks per expert estimated
// from the launch bounds (no reliance on L2 keeping data between waves).
inline int pick_group_m(const GemmParams& g, int64_t block_rows, int64_t k_bytes_per_row, int n_tiles, int ctas) {
  const double a_blk = (double)block_rows * (double)k_bytes_per_row;
  const double b_tile = 256.0 * (double)k_bytes_per_row;
  const double active = (double)(g.numel < g.num_experts ? (g.numel > 0 ? g.numel : 1) : g.num_experts);
  double bpe = (double)g.numel / active / (double)block_rows;
  if (bpe < 1.0) bpe = 1.0;
  int best = 1;
  double best_cost = 1e300;
  const int limit = ctas < 1 ? 1 : ctas;
  for (int gm = 1; gm <= limit; ++gm) {
    double gn = (double)limit / gm;
    if (gn > n_tiles) gn = n_tiles;
    double experts = gm / bpe;
    if (experts < 1.0) experts = 1.0;
    // traffic per tile of the wave
    const double cost = (gm * a_blk + experts * gn * b_tile) / (gm * gn);
    if (cost < best_cost * 0.999) {
      best_cost = cost;
      best = gm;
    }
  }
  return best;
}

// device status word written by bounded waits (gemm_tcgen05.cu)
int read_and_clear_device_status(cudaStream_t st, int* status_out);

}  // namespace fmoe
