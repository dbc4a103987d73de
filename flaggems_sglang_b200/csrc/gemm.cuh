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

// true when the variant can run these arguments (shape / alignment / dtype rules)
bool gemm_stream_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_supports(const GemmParams& p, bool gated);
int64_t gemm_tcgen05_split_workspace_bytes();
int tail_plan_unit(int64_t total_tiles, int k_steps, int max_split, int grid, int cta, int64_t it, int64_t* out);
bool gemm_tcgen05_fp8_supports(const GemmParams& p, bool gated);

// Tile order of the persistent kernels: expert by expert, and inside an expert in groups of at most
// `group_m` row blocks; inside a group the row block varies fastest, then the column tile.  The tiles
// that run at the same time therefore belong to one or a few experts: each weight tile is fetched
// from HBM once and shared through L2 by the row blocks of its expert, while the group's activation
// rows (a few MB) stay hot in L2 across the column tiles.
//
// Because every expert's tiles are contiguous in this order, the expert of tile t is the expert of
// row block floor(t / n_tiles).  Every CTA first builds, in shared memory, the first row block and the
// number of row blocks of every expert (one pass over expert_ids); looking a tile up is then ONE global
// load (the block's expert) and two shared-memory reads.  (A bisection in expert_ids per tile, about ten
// dependent global loads, stalled the TMA producer for longer than its ring holds data: the MMA warp of
// the bf16 kernel waited 7.5 k of every 57 k clocks for it.)
#if defined(__CUDACC__)
constexpr int kExpertTableBytesPerExpert = 8;  // first block + block count
__host__ __device__ constexpr int expert_table_bytes(int num_experts) { return ((num_experts * 8) + 15) & ~15; }

// All threads of the CTA; `table` = expert_table_bytes(E) bytes of shared memory.  Ends with __syncthreads().
__device__ __forceinline__ void build_expert_table(int32_t* table, int num_experts, const int32_t* __restrict__ expert_ids,
                                                   int used_blocks) {
  int32_t* first = table;
  int32_t* count = table + num_experts;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    first[e] = 0x7fffffff;
    count[e] = 0;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < used_blocks; b += blockDim.x) {
    const int e = expert_ids[b];
    if (e >= 0 && e < num_experts) {
      atomicMin(&first[e], b);
      atomicAdd(&count[e], 1);
    }
  }
  __syncthreads();
}

struct TileCursor {
  int first = 0, last = 0, expert = 0;  // block range [first, last) and id of the cached expert; empty = nothing cached
  __device__ __forceinline__ void locate(int64_t tile, int n_tiles, int group_m, int num_experts,
                                         const int32_t* __restrict__ expert_ids, const int32_t* table, int* m_blk,
                                         int* n_tile, int* expert_out) {
    const int q = (int)(tile / n_tiles);
    if (q < first || q >= last) {
      expert = min(max(expert_ids[q], 0), num_experts - 1);
      first = table[expert];
      last = first + table[num_experts + expert];
      if (q < first || q >= last) {  // expert_ids not grouped by expert (misuse): treat the block as a range of its own
        first = q;
        last = q + 1;
      }
    }
    const int nb = last - first;
    const int64_t local = tile - (int64_t)first * n_tiles;
    const int64_t per_group = (int64_t)group_m * n_tiles;
    const int g = (int)(local / per_group);
    const int r = (int)(local % per_group);
    const int rows = min(group_m, nb - g * group_m);
    *n_tile = r / rows;
    *m_blk = first + g * group_m + r % rows;
    *expert_out = expert;
  }
};
#endif
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
