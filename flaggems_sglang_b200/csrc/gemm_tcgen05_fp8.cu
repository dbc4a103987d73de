// Large-M grouped GEMM on e4m3 operands with 128x128 weight scales and 1x128 activation scales.
//
// tcgen05 accumulates in fp32 inside TMEM and cannot apply a different scale to every 128-wide K block, so
// every K block (128 bytes = 128 e4m3 = one scale block) is multiplied into a FRESH 128x256 TMEM partial
// (4 MMAs of K=32, the first one overwriting), and the epilogue warps fold it into register accumulators:
//     acc[row, col] += partial[row, col] * a_scale[row, kb] * w_scale[col/128, kb]
// Two TMEM partials (2 x 256 columns) ping-pong, so the MMAs of block kb+1 run while block kb is folded.
//
//   warps 0-15: fold + epilogue.  Warp w owns TMEM lanes 32*(w%4).. (rows) and quarter c = w/4 of the columns:
//               gemm1: gate columns [32c,32c+32) and the matching up columns [128+32c, ...), 64 accumulators;
//               gemm2: columns [64c, 64c+64).  Four warps per scheduler hide the TMEM load latency.
//   warp 16   : TMA producer (A 128x128 B box, B two 128-row boxes), 4-stage ring
//   warp 17   : MMA issuer
// Same tile schedule, bounded waits and status word as the bf16 kernel; cluster size 1, every CTA loads its own tiles.
#include "gemm.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace fmoe {

// This translation unit's status word (device code is not linked across files); read by status_word_fp8().
__device__ int g_device_status_fp8 = 0;

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int KBYTES = 128;
// Three 48 KB stages (147 KB of shared memory -> 164 KB carve-out, 92 KB of L1) measured 2.5-4 % faster on the
// gate/up GEMM than four (196 KB carve-out, 60 KB of L1): the kernel is bound by its fold warps, which read block
// scales and a few spilled registers through L1, not by TMA latency.  One KB beyond the 196 KB carve-out (228 KB,
// 28 KB of L1) measured 40 % slower.
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * KBYTES;
constexpr int B_BYTES = BN * KBYTES;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int kEpiWarps = 16;
constexpr int kThreads = (kEpiWarps + 4) * 32;  // warps 18, 19 only exist to complete the fifth warpgroup
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Fp8Params {
  const int32_t* sorted_token_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_post_padded;
  const float* row_scale;
  const float* a_scale;  // [a_rows, kblocks]
  const float* w_scale;  // [E, w_rows/128, kblocks]
  void* out;
  void* const* out_rows;  // down projection: optional per-slot row addresses (may be peer memory)
  int64_t numel;
  int64_t n;
  int64_t w_rows;
  int64_t sorted_cap;
  int32_t num_experts;
  int32_t kblocks;
  int32_t n_tiles;
  int32_t max_blocks;
  int32_t activation;
  int32_t group_m;
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_device_status_fp8, 0, code); }
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
}

template <bool GATED>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tcgen05_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;            // [STAGES] MMA -> TMA
  uint64_t* part_full = bars + 2 * STAGES;        // [2] MMA -> fold
  uint64_t* part_empty = bars + 2 * STAGES + 2;   // [2] fold -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&part_full[a], 1);
      ptx::mbar_init(&part_empty[a], kEpiWarps);  // one arrival per fold warp
    }
    ptx::fence_barrier_init();
  }
  if (warp == kEpiWarps && lane == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == kEpiWarps + 1) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int used_blocks = min((int)(*p.num_tokens_post_padded / BM), p.max_blocks);
  const int64_t total_tiles = (int64_t)used_blocks * p.n_tiles;
  TileCursor cursor;
  const int kblocks = p.kblocks;

  if (warp == kEpiWarps) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    // coordinates of a tile; looked up one tile ahead so that the index loads never stall the ring
    auto tile_rows = [&](int64_t tile, int32_t* row_a, int32_t* row_b0, int32_t* row_b1) {
      int m_blk, n_tile;
      cursor.locate(tile, used_blocks, p.n_tiles, p.group_m, p.expert_ids, &m_blk, &n_tile);
      const int e = min(max(p.expert_ids[m_blk], 0), p.num_experts - 1);
      *row_a = m_blk * BM;
      *row_b0 = (int32_t)((int64_t)e * p.w_rows + (GATED ? (int64_t)n_tile * 128 : (int64_t)n_tile * 256));
      *row_b1 = GATED ? (int32_t)(*row_b0 + p.n) : *row_b0 + 128;
    };
    int32_t row_a = 0, row_b0 = 0, row_b1 = 0, nrow_a = 0, nrow_b0 = 0, nrow_b1 = 0;
    if ((int64_t)blockIdx.x < total_tiles) tile_rows(blockIdx.x, &row_a, &row_b0, &row_b1);
    for (int64_t tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
      const bool has_next = tile + gridDim.x < total_tiles;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!warp_wait(&empty_bar[stage], phase ^ 1)) {
          report(0x500 | stage);
          alive = false;
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int32_t x = kb * KBYTES;  // element coordinate (1-byte elements)
          ptx::tma_load_2d(sa, &map_a, x, row_a, &full_bar[stage]);
          ptx::tma_load_2d(sb, &map_b, x, row_b0, &full_bar[stage]);
          ptx::tma_load_2d(sb + B_BYTES / 2, &map_b, x, row_b1, &full_bar[stage]);
        }
        __syncwarp();
        if (kb == 0 && has_next) tile_rows(tile + gridDim.x, &nrow_a, &nrow_b0, &nrow_b1);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      row_a = nrow_a;
      row_b0 = nrow_b0;
      row_b1 = nrow_b1;
    }
    if (alive) {  // drain our own bulk copies before leaving
      for (int s = 0; s < STAGES; ++s) {
        if (!warp_wait(&empty_bar[stage], phase ^ 1)) {
          report(0x580 | stage);
          break;
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == kEpiWarps + 1) {
    // ---------------- MMA issuer: one fresh partial per K block ----------------
    constexpr uint32_t idesc = ptx::make_idesc(/*e4m3*/ 0, BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t step = 0;  // K blocks issued so far by this CTA (selects the partial and its phase)
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
      for (int kb = 0; kb < kblocks; ++kb, ++step) {
        const int buf = step & 1;
        const uint32_t buf_phase = (step >> 1) & 1;
        if (!warp_wait(&part_empty[buf], buf_phase ^ 1)) {
          report(0x600 | buf);
          alive = false;
          break;
        }
        if (!warp_wait(&full_bar[stage], phase)) {
          report(0x640 | stage);
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = ptx::smem_desc_sw128(sa);
          const uint64_t db = ptx::smem_desc_sw128(sa + A_BYTES);
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int kk = 0; kk < KBYTES / 32; ++kk)
            ptx::mma_f8f6f4_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, kk != 0);
          ptx::mma_commit(&empty_bar[stage]);
          ptx::mma_commit(&part_full[buf]);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp < kEpiWarps) {
    // ---------------- fold + epilogue (warps 0-15) ----------------
    const int quarter = warp & 3, cpart = warp >> 2;  // TMEM lane quarter, column quarter
    const int row = quarter * 32 + lane;
    const int64_t sblocks_per_expert = p.w_rows / 128;
    uint32_t step = 0;
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
      int m_blk, n_tile;
      cursor.locate(tile, used_blocks, p.n_tiles, p.group_m, p.expert_ids, &m_blk, &n_tile);
      const int e = min(max(p.expert_ids[m_blk], 0), p.num_experts - 1);
      const int64_t pos = (int64_t)m_blk * BM + row;
      const bool in_cap = pos < p.sorted_cap;
      const int32_t slot = in_cap ? p.sorted_token_ids[pos] : -1;
      const bool valid = slot >= 0 && slot < p.numel;
      const float rs = (valid && p.row_scale) ? p.row_scale[slot] : 1.0f;
      const float* sa_row = p.a_scale + (in_cap ? pos : 0) * kblocks;
      // weight-scale rows of this warp's two 32-column pieces (gemm1: gate / up; gemm2: both in one 128-block)
      const int64_t sw_blk0 = GATED ? n_tile : min(2 * (int64_t)n_tile + (cpart >> 1), sblocks_per_expert - 1);
      const int64_t sw_blk1 = GATED ? (p.n / 128 + n_tile) : sw_blk0;
      const float* sw0 = p.w_scale + ((int64_t)e * sblocks_per_expert + sw_blk0) * kblocks;
      const float* sw1 = p.w_scale + ((int64_t)e * sblocks_per_expert + sw_blk1) * kblocks;
      const int col0 = GATED ? 32 * cpart : 64 * cpart;
      const int col1 = GATED ? 128 + 32 * cpart : 64 * cpart + 32;

      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;

      float sa_n = in_cap ? sa_row[0] : 0.f, s0_n = sw0[0], s1_n = sw1[0];
      for (int kb = 0; kb < kblocks; ++kb, ++step) {
        const int buf = step & 1;
        const uint32_t buf_phase = (step >> 1) & 1;
        const float f0 = sa_n * s0_n, f1 = sa_n * s1_n;
        if (kb + 1 < kblocks) {  // prefetch the next block's scales while waiting for the MMAs
          sa_n = in_cap ? sa_row[kb + 1] : 0.f;
          s0_n = sw0[kb + 1];
          s1_n = sw1[kb + 1];
        }
        if (!warp_wait(&part_full[buf], buf_phase)) {
          report(0x700 | buf);
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          // 16 columns at a time keeps the staging registers small (64 accumulators stay live); two loads in
          // flight per wait were measured no faster: the fold is bound by TMEM read-out, 128 KB per K block
          uint32_t v[16];
          ptx::tmem_ld_32x32b_x16(taddr + ((c < 2) ? col0 + 16 * c : col1 + 16 * (c - 2)), v);
          ptx::tmem_ld_wait();
          const float f = (c < 2) ? f0 : f1;
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[16 * c + i] = fmaf(__uint_as_float(v[i]), f, acc[16 * c + i]);
        }
        // 512 separate arrivals on one barrier word would serialise for longer than the fold itself:
        // the warp's lanes order their TMEM reads, then one lane arrives for all of them
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&part_empty[buf]);
      }
      if (!alive) break;

      if constexpr (GATED) {
        // acc[0..31] gate, acc[32..63] up -> output columns n_tile*128 + 32*cpart + [0,32)
        if (in_cap) {
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + pos * p.n + (int64_t)n_tile * 128 + 32 * cpart;
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = v * 8 + j * 2;
              w[j] = pack_bf16x2(act_mul_fast(acc[i] * rs, acc[32 + i] * rs, p.activation),
                                 act_mul_fast(acc[i + 1] * rs, acc[32 + i + 1] * rs, p.activation));
            }
            dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        const int64_t colg = (int64_t)n_tile * 256 + 64 * cpart;
        __nv_bfloat16* obase = !valid ? nullptr
                               : p.out_rows ? reinterpret_cast<__nv_bfloat16*>(p.out_rows[slot])
                                            : reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)slot * p.n;
        if (obase && colg < p.n) {
          uint4* dst = reinterpret_cast<uint4*>(obase + colg);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = v * 8 + j * 2;
              w[j] = pack_bf16x2(acc[i] * rs, acc[i + 1] * rs);
            }
            dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  if (p.out_rows) __threadfence_system();  // rows stored to a peer are complete before the kernel ends
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == kEpiWarps + 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// defined in gemm_tcgen05.cu
int make_tensor_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes, int box_rows,
                       bool weights, int kbytes);
int device_sm_count();

namespace {

template <bool GATED>
int launch(const GemmParams& g, cudaStream_t st) {
  static PerDeviceOnce once_attr;  // the opt-in to > 48 KB of dynamic shared memory is per device
  const cudaError_t attr_err = per_device_once(once_attr, [] {
    return cudaFuncSetAttribute(grouped_gemm_tcgen05_fp8_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                SMEM_BYTES);
  });
  if (attr_err != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", SMEM_BYTES, cudaGetErrorString(attr_err));
  const int64_t w_rows = GATED ? 2 * g.n : g.n;
  CUtensorMap map_a, map_b;
  int rc = make_tensor_map_2d(&map_a, g.a, g.a_rows, g.k, 1, BM, false, 128);
  if (rc) return rc;
  rc = make_tensor_map_2d(&map_b, g.w, (int64_t)g.num_experts * w_rows, g.k, 1, 128, true, 128);
  if (rc) return rc;
  Fp8Params p;
  p.sorted_token_ids = g.sorted_token_ids;
  p.expert_ids = g.expert_ids;
  p.num_tokens_post_padded = g.num_tokens_post_padded;
  p.row_scale = g.row_scale;
  p.a_scale = g.a_scale;
  p.w_scale = g.w_scale;
  p.out = g.out;
  p.out_rows = GATED ? nullptr : g.out_rows;
  p.numel = g.numel;
  p.n = g.n;
  p.w_rows = w_rows;
  p.sorted_cap = g.sorted_cap;
  p.num_experts = g.num_experts;
  p.kblocks = (int)(g.k / 128);
  p.n_tiles = (int)ceil_div<int64_t>(g.n, GATED ? 128 : 256);
  p.max_blocks = (int)g.max_blocks;
  p.activation = g.activation;

  const int64_t max_tiles = g.max_blocks * p.n_tiles;
  const int sms = device_sm_count();
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(sms > 0 ? sms : 148, max_tiles));
  p.group_m = pick_group_m(BM, g.k);
  grouped_gemm_tcgen05_fp8_kernel<GATED><<<grid, kThreads, SMEM_BYTES, st>>>(map_a, map_b, p);
  return launch_status("grouped_gemm_tcgen05_fp8_kernel");
}

}  // namespace

bool gemm_tcgen05_fp8_supports(const GemmParams& p, bool gated) {
  if (p.dtype != FMOE_E4M3 || p.out_dtype != FMOE_BF16) return false;
  if (p.bias || p.activation == FMOE_ACT_SWIGLU_OAI) return false;  // bf16-only variant
  if (p.block_size != BM || p.a_gather) return false;
  if (p.k <= 0 || p.k % 128 != 0 || p.n <= 0 || p.n % 128 != 0) return false;
  if (!p.a_scale || !p.w_scale) return false;
  if (!aligned16(p.a) || !aligned16(p.w) || !(aligned16(p.out) && (p.out || (!gated && p.out_rows)))) return false;
  if ((int64_t)p.num_experts * (gated ? 2 * p.n : p.n) >= (1ll << 31) || p.a_rows >= (1ll << 31)) return false;
  if (p.max_blocks >= (1ll << 24)) return false;
  return true;
}

int status_word_fp8(int* out, bool clear) {
  int zero = 0;
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(out, g_device_status_fp8, sizeof(int)));
  if (clear && *out != 0) FMOE_CUDA_OK(cudaMemcpyToSymbol(g_device_status_fp8, &zero, sizeof(int)));
  return FMOE_OK;
}

int gemm_tcgen05_fp8(const GemmParams& p, bool gated, cudaStream_t st) {
  if (!gemm_tcgen05_fp8_supports(p, gated))
    return fail(FMOE_ERR_UNSUPPORTED,
                "tcgen05 fp8 gemm: needs e4m3 in, bf16 out, block_size 128, sorted input rows, n and k multiples of 128");
  if (p.max_blocks <= 0) return FMOE_OK;
  return gated ? launch<true>(p, st) : launch<false>(p, st);
}

}  // namespace fmoe
