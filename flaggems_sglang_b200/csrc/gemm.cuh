// Internal interface between the C-ABI entry points (api.cu) and the three
// grouped-GEMM kernel families.
#pragma once
#include <cstdlib>

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

// Tile order of the persistent kernels: expert by expert, and inside an expert in groups of at most
// `group_m` row blocks; inside a group the row block varies fastest, then the column tile.  The tiles
// that run at the same time therefore belong to one or a few experts: each weight tile is fetched
// from HBM once and shared through L2 by the row blocks of its expert, while the group's activation
// rows (a few MB) stay hot in L2 across the column tiles.
//
// Because every expert's tiles are contiguous in this order, the expert of tile t is the expert of
// row block floor(t / n_tiles); its first and last block are found by bisection in expert_ids
// (ascending by construction) and cached while consecutive tiles stay inside the same expert.
struct TileCursor {
  int first = 0, last = 0;  // block range [first, last) of the cached expert; empty = nothing cached
  __device__ __forceinline__ void locate(int64_t tile, int used_blocks, int n_tiles, int group_m,
                                         const int32_t* __restrict__ expert_ids, int* m_blk, int* n_tile) {
    const int q = (int)(tile / n_tiles);
    if (q < first || q >= last) {
      const int e = expert_ids[q];
      // tiles only move forward, so the new expert starts at or after the cached range's end
      int lo = (q >= last) ? last : 0, hi = q;  // first index in [lo, q] with expert_ids[i] >= e
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (expert_ids[mid] < e) lo = mid + 1; else hi = mid;
      }
      first = lo;
      // first index past q whose expert differs: gallop, then bisect the last interval
      int step = 1, known = q;  // expert_ids[known] == e
      hi = used_blocks;
      while (known + step < used_blocks) {
        if (expert_ids[known + step] == e) {
          known += step;
          step <<= 1;
        } else {
          hi = known + step;
          break;
        }
      }
      lo = known + 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (expert_ids[mid] == e) lo = mid + 1; else hi = mid;
      }
      last = lo;
    }
    const int nb = last - first;
    const int64_t local = tile - (int64_t)first * n_tiles;
    const int64_t per_group = (int64_t)group_m * n_tiles;
    const int g = (int)(local / per_group);
    const int r = (int)(local % per_group);
    const int rows = min(group_m, nb - g * group_m);
    *n_tile = r / rows;
    *m_blk = first + g * group_m + r % rows;
  }
};
// Row blocks per group: the group's A rows should stay around 16 MB.
inline int pick_group_m(int64_t block_rows, int64_t k_bytes_per_row) {
  if (const char* env = getenv("FMOE_TC_GROUP_M")) {  // tuning aid
    const int g = atoi(env);
    if (g >= 1 && g <= 1024) return g;
  }
  const int64_t per_block = block_rows * k_bytes_per_row;
  int64_t g = (16ll << 20) / (per_block > 0 ? per_block : 1);
  return (int)(g < 8 ? 8 : (g > 64 ? 64 : g));
}

// device status word written by bounded waits (gemm_tcgen05.cu)
int read_and_clear_device_status(cudaStream_t st, int* status_out);

}  // namespace fmoe
