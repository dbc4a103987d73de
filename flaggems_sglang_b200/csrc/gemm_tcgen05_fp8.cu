// Large-M grouped GEMM on e4m3 operands with 128x128 weight scales and 1x128 activation scales.
//
// tcgen05 accumulates in fp32 inside TMEM and cannot apply a different scale to every 128-wide K block, so
// every K block (128 bytes = 128 e4m3 = one scale block) is multiplied into a FRESH 128x256 TMEM partial
// (4 MMAs of K=32, the first one overwriting), and the fold warps add it into register accumulators:
//     acc[row, col] += partial[row, col] * a_scale[row, kb] * w_scale[col/128, kb]
// Two TMEM partials (2 x 256 columns) ping-pong, so the MMAs of block kb+1 run while block kb is folded.
//
//   warps 0-15: fold + epilogue.  Warp w owns TMEM lanes 32*(w%4).. (rows) and, of each 128-column half of the
//               partial, columns [32c, 32c+32) with c = w/4: 64 accumulators per thread.  gemm1: the halves are the
//               gate and the up columns; gemm2: output columns n0+32c.. and n0+128+32c...  The FMAs are issued as
//               packed fma.rn.f32x2 (two accumulators per instruction): the fold is bound by instruction issue.
//   warp 16   : TMA producer (A 128x128 B box, B two 128-row boxes), 3-stage ring
//   warp 17   : MMA issuer
//   warps 18-19: scale stagers.  One tile ahead of the fold warps they look the tile up (expert, row block, column
//               tile) and copy its block scales into shared memory: the 128 x K/128 activation scales transposed to
//               [K block][row] and the two weight-scale rows.  Read straight from global memory by the fold warps,
//               the activation scales cost 32 L1 wavefronts per warp and K block (one per row); from shared memory
//               they are one conflict-free wavefront, and the fold warps keep no pointers or tile cursor in registers
//               (the kernel runs at its 96-register limit, every spill lands in the fold loop).
// Same tile schedule, bounded waits and status word as the bf16 kernel; cluster size 1, every CTA loads its own tiles.
#include "gemm.cuh"

#include <type_traits>
#include "ptx_sm100.cuh"

#include <cstdlib>
#include <mutex>

namespace fmoe {

// This translation unit's status word (device code is not linked across files); read by status_word_fp8().
__device__ int g_device_status_fp8 = 0;
// Wait-time profile of the instrumented build of the kernel (FMOE_TC_PROFILE=1): per CTA
// {tiles, fold waits for the MMAs, fold busy, fold waits for staged scales, epilogue, kernel cycles, -, -};
// [0]: down GEMM, [1]: gate/up GEMM
__device__ long long g_wait_prof_fp8[2 * 256 * 8];

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int KBYTES = 128;
// Ring of NS 48 KB stages (template parameter of the kernel): four when both scale buffers still fit beside them
// (short reductions), else three.  The kernel is bound by its fold warps and by the shared-memory traffic of TMA
// fill + MMA operand reads, not by TMA latency: the fourth stage gains 3 %.
constexpr int kMaxStages = 4;
constexpr int A_BYTES = BM * KBYTES;
constexpr int B_BYTES = BN * KBYTES;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int kEpiWarps = 16;
constexpr int kThreads = (kEpiWarps + 4) * 32;
constexpr int kMaxSmem = 227 * 1024;
constexpr int kMaxStagedKBlocks = 64;  // two scale buffers of (128 + 2) * kblocks floats + 16 bytes must fit beside the ring
constexpr int scale_buf_bytes(int kblocks) { return (BM + 2) * kblocks * 4 + 16; }
constexpr int smem_bytes(int stages, int nbuf, int kblocks, int num_experts) {
  return stages * STAGE_BYTES + 1024 + 256 + expert_table_bytes(num_experts) + nbuf * scale_buf_bytes(kblocks);
}

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
  int32_t spin;   // 1: the partial hand-overs are polled with test_wait instead of try_wait
  int32_t nbuf;        // scale buffers in shared memory: 2 (a tile's scales are staged while the previous tile folds) or 1
  int32_t debug;  // instrumented build only, timing experiments (results are wrong): bit 0 = the fold skips the TMEM
                  // read-out and the FMAs, bit 1 = no MMAs are issued, bit 2 = read-out without FMAs
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_device_status_fp8, 0, code); }
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
}
// hand-overs of the TMEM partials (once per K block in each direction): polled without suspending
template <bool SPIN>
__device__ __forceinline__ bool warp_wait_fast(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, SPIN ? ptx::mbar_wait_spin(bar, parity) : ptx::mbar_wait(bar, parity));
}

// acc (two packed floats) += v * f, both lanes
__device__ __forceinline__ void fma2(unsigned long long& acc, uint32_t v0, uint32_t v1, unsigned long long ff) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(v0), "r"(v1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(v), "l"(ff));
}
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(a), "f"(b));
  return v;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}

// MODE 0: production.  MODE 1: instrumented build with wait-time counters (reading the clock is slow enough to distort
// the fold loop; use it for proportions only).  MODE 2: timing experiments selected by Fp8Params::debug, no counters.
template <bool GATED, int MODE, int NS>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tcgen05_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                const Fp8Params p) {
  constexpr bool PROF = MODE == 1;
  constexpr bool DBG = MODE == 2;
  constexpr int STAGES = NS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;            // [STAGES] MMA -> TMA
  uint64_t* part_full = bars + 2 * STAGES;        // [2] MMA -> fold
  uint64_t* part_empty = bars + 2 * STAGES + 2;   // [2] fold -> MMA
  uint64_t* scale_full = bars + 2 * STAGES + 4;   // [2] stagers -> fold
  uint64_t* scale_empty = bars + 2 * STAGES + 6;  // [2] fold -> stagers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8);
  int32_t* expert_table = reinterpret_cast<int32_t*>(smem + STAGES * STAGE_BYTES + 256);
  // staged scales, two buffers: [kblocks][128] activation scales, [2][kblocks] weight scales, {m_blk, n_tile, expert, -}
  uint8_t* scale_base = smem + STAGES * STAGE_BYTES + 256 + expert_table_bytes(p.num_experts);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t_kernel0 = PROF ? clock64() : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&part_full[a], 1);
      ptx::mbar_init(&part_empty[a], kEpiWarps);  // one arrival per fold warp
      ptx::mbar_init(&scale_full[a], 2);           // one arrival per stager warp
      ptx::mbar_init(&scale_empty[a], kEpiWarps);
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
  const int used_blocks = min((int)(*p.num_tokens_post_padded / BM), p.max_blocks);
  const int64_t total_tiles = (int64_t)used_blocks * p.n_tiles;
  ptx::tc_fence_before_sync();
  build_expert_table(expert_table, p.num_experts, p.expert_ids, used_blocks);  // ends with __syncthreads()
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int kblocks = p.kblocks;

  if (warp == kEpiWarps) {
    // ---------------- TMA producer ----------------
    TileCursor cursor;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    // coordinates of a tile; looked up one tile ahead so that the index load never stalls the ring
    auto tile_rows = [&](int64_t tile, int32_t* row_a, int32_t* row_b0, int32_t* row_b1) {
      int m_blk, n_tile, e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &e);
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
        if (!(p.spin ? warp_wait_fast<true>(&part_empty[buf], buf_phase ^ 1) : warp_wait_fast<false>(&part_empty[buf], buf_phase ^ 1))) {
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
          if (!DBG || !(p.debug & 2)) {
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk)
              ptx::mma_f8f6f4_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, kk != 0);
          }
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
    const int quarter = warp & 3, cpart = warp >> 2;  // TMEM lane quarter, 32-column piece of each half
    const int row = quarter * 32 + lane;
    uint32_t step = 0;
    uint32_t ltile = 0;  // tiles started by this CTA (selects the scale buffer and its phase)
    bool alive = true;
    long long prof_fw = 0, prof_fb = 0, prof_sw = 0, prof_epi = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++ltile) {
      const int tb = (int)(ltile % p.nbuf);
      const float* s_a = reinterpret_cast<const float*>(scale_base + tb * scale_buf_bytes(kblocks)) + row;
      const float* s_w = reinterpret_cast<const float*>(scale_base + tb * scale_buf_bytes(kblocks)) + BM * kblocks;
      const long long tq0 = PROF ? clock64() : 0;
      if (!warp_wait(&scale_full[tb], (ltile / p.nbuf) & 1)) {
        report(0x740 | tb);
        alive = false;
        break;
      }
      if (PROF) prof_sw += clock64() - tq0;
      const int32_t* meta = reinterpret_cast<const int32_t*>(s_w + 2 * kblocks);
      const int m_blk = meta[0], n_tile = meta[1];
      const int64_t pos = (int64_t)m_blk * BM + row;
      const int32_t slot = (pos < p.sorted_cap) ? p.sorted_token_ids[pos] : -1;  // consumed by the epilogue

      unsigned long long acc[32];  // 64 packed accumulators: [0,16) first half's 32 columns, [16,32) second half's
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0ull;

      float sa_n = s_a[0], s0_n = s_w[0], s1_n = s_w[kblocks];
      for (int kb = 0; kb < kblocks; ++kb, ++step) {
        const int buf = step & 1;
        const float f0 = sa_n * s0_n, f1 = sa_n * s1_n;
        if (kb + 1 < kblocks) {  // the next block's scales, fetched while waiting for the MMAs
          sa_n = s_a[(kb + 1) * BM];
          s0_n = s_w[kb + 1];
          s1_n = s_w[kblocks + kb + 1];
        }
        const long long tf0 = PROF ? clock64() : 0;
        if (!(p.spin ? warp_wait_fast<true>(&part_full[buf], (step >> 1) & 1) : warp_wait_fast<false>(&part_full[buf], (step >> 1) & 1))) {
          report(0x700 | buf);
          alive = false;
          break;
        }
        const long long tf1 = PROF ? clock64() : 0;
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16) + 32 * cpart;
        if (!DBG || !(p.debug & 1)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            // 16 columns at a time keeps the staging registers small (the 64 accumulators stay live)
            uint32_t v[16];
            ptx::tmem_ld_32x32b_x16(taddr + (c >> 1) * 128 + (c & 1) * 16, v);
            ptx::tmem_ld_wait();
            if (!DBG || !(p.debug & 4)) {
              const unsigned long long ff = (c < 2) ? pack2(f0, f0) : pack2(f1, f1);
#pragma unroll
              for (int i = 0; i < 8; ++i) fma2(acc[8 * c + i], v[2 * i], v[2 * i + 1], ff);
            }
          }
        }
        // 512 separate arrivals on one barrier word would serialise for longer than the fold itself:
        // the warp's lanes order their TMEM reads, then one lane arrives for all of them
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&part_empty[buf]);
        if (PROF) {
          prof_fw += tf1 - tf0;
          prof_fb += clock64() - tf1;
        }
      }
      if (!alive) break;
      // this warp has read the tile's last staged scale
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&scale_empty[tb]);

      const long long te0 = PROF ? clock64() : 0;
      const bool valid = slot >= 0 && slot < p.numel;
      const float rs = (valid && p.row_scale) ? p.row_scale[slot] : 1.0f;
      if constexpr (GATED) {
        // acc[0..15] gate, acc[16..31] up -> output columns n_tile*128 + 32*cpart + [0,32)
        if (pos < p.sorted_cap) {
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + pos * p.n + (int64_t)n_tile * 128 + 32 * cpart;
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float g0, g1, u0, u1;
              unpack2(acc[v * 4 + j], g0, g1);
              unpack2(acc[16 + v * 4 + j], u0, u1);
              w[j] = pack_bf16x2(act_mul_fast(g0 * rs, u0 * rs, p.activation), act_mul_fast(g1 * rs, u1 * rs, p.activation));
            }
            dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        // acc[0..15]: columns n0 + 32*cpart + [0,32); acc[16..31]: columns n0 + 128 + 32*cpart + [0,32)
        __nv_bfloat16* obase = !valid ? nullptr
                               : p.out_rows ? reinterpret_cast<__nv_bfloat16*>(p.out_rows[slot])
                                            : reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)slot * p.n;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int64_t colg = (int64_t)n_tile * 256 + 128 * h + 32 * cpart;
          if (obase && colg < p.n) {
            uint4* dst = reinterpret_cast<uint4*>(obase + colg);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float a0, a1;
                unpack2(acc[16 * h + v * 4 + j], a0, a1);
                w[j] = pack_bf16x2(a0 * rs, a1 * rs);
              }
              dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      if (PROF) prof_epi += clock64() - te0;
    }
    if (PROF && threadIdx.x == 0 && blockIdx.x < 256) {
      long long* out = g_wait_prof_fp8 + (GATED ? 2048 : 0) + blockIdx.x * 8;
      out[0] = ltile;
      out[1] = prof_fw;
      out[2] = prof_fb;
      out[3] = prof_sw;
      out[4] = prof_epi;
    }
  } else {
    // ---------------- scale stagers (warps 18-19): 64 rows each, one tile ahead of the fold ----------------
    TileCursor cursor;
    const int half = warp - (kEpiWarps + 2);
    const int64_t sblocks_per_expert = p.w_rows / 128;
    uint32_t ltile = 0;
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++ltile) {
      const int tb = (int)(ltile % p.nbuf);
      int m_blk, n_tile, e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &e);
      if (!warp_wait(&scale_empty[tb], ((ltile / p.nbuf) & 1) ^ 1)) {
        report(0x780 | tb);
        alive = false;
        break;
      }
      float* s_a = reinterpret_cast<float*>(scale_base + tb * scale_buf_bytes(kblocks));
      float* s_w = s_a + BM * kblocks;
      // activation scales: lane = row (conflict-free transposed stores), 16 bytes of K blocks per load,
      // four loads in flight per lane
      for (int rr = 0; rr < 64; rr += 32) {
        const int r = half * 64 + rr + lane;
        const int64_t pos = (int64_t)m_blk * BM + r;
        const bool in_cap = pos < p.sorted_cap;
        const float* srow = p.a_scale + (in_cap ? pos : 0) * kblocks;
        if ((kblocks & 3) != 0 || !aligned16(p.a_scale)) {  // rows that are not whole 16-byte pieces: scalar loads
          for (int j = 0; j < kblocks; ++j) s_a[j * BM + r] = in_cap ? __ldg(srow + j) : 0.f;
          continue;
        }
        const float4* src = reinterpret_cast<const float4*>(srow);
        const int nvec = kblocks / 4;
        for (int j0 = 0; j0 < nvec; j0 += 4) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            v[u] = (in_cap && j0 + u < nvec) ? __ldg(src + j0 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (j0 + u < nvec) {
              float* d = s_a + (4 * (j0 + u)) * BM + r;
              d[0] = v[u].x;
              d[BM] = v[u].y;
              d[2 * BM] = v[u].z;
              d[3 * BM] = v[u].w;
            }
          }
        }
      }
      // weight scales: stager `half` copies row `half` (gate / up, or the tile's first / second 128 columns)
      const int64_t blk = GATED ? (half == 0 ? (int64_t)n_tile : p.n / 128 + n_tile)
                                : min(2 * (int64_t)n_tile + half, sblocks_per_expert - 1);
      const float* wsrc = p.w_scale + ((int64_t)e * sblocks_per_expert + blk) * kblocks;
      for (int j = lane; j < kblocks; j += 32) s_w[half * kblocks + j] = __ldg(wsrc + j);
      if (half == 0 && lane == 0) {
        int32_t* meta = reinterpret_cast<int32_t*>(s_w + 2 * kblocks);
        meta[0] = m_blk;
        meta[1] = n_tile;
        meta[2] = e;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&scale_full[tb]);
    }
  }

  if (p.out_rows) __threadfence_system();  // rows stored to a peer are complete before the kernel ends
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == kEpiWarps + 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (PROF && threadIdx.x == 0 && blockIdx.x < 256)
    g_wait_prof_fp8[(GATED ? 2048 : 0) + blockIdx.x * 8 + 5] = clock64() - t_kernel0;
}

}  // namespace

// defined in gemm_tcgen05.cu
int make_tensor_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes, int box_rows,
                       bool weights, int kbytes);
int device_sm_count();

namespace {

template <bool GATED, int MODE, int NS>
int launch(const GemmParams& g, int nbuf, cudaStream_t st) {
  constexpr int MAX_SMEM = kMaxSmem;
  static_assert(smem_bytes(3, 2, kMaxStagedKBlocks, 1024) <= kMaxSmem, "scale buffers do not fit beside the ring");
  static PerDeviceOnce once_attr;  // the opt-in to > 48 KB of dynamic shared memory is per device
  const cudaError_t attr_err = per_device_once(once_attr, [] {
    return cudaFuncSetAttribute(grouped_gemm_tcgen05_fp8_kernel<GATED, MODE, NS>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
  });
  if (attr_err != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", MAX_SMEM, cudaGetErrorString(attr_err));
  const int SMEM_BYTES = smem_bytes(NS, nbuf, (int)(g.k / 128), g.num_experts);
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
  p.nbuf = nbuf;
  p.spin = getenv("FMOE_FP8_SPIN") ? atoi(getenv("FMOE_FP8_SPIN")) : 0;
  p.debug = (MODE == 2 && getenv("FMOE_FP8_DEBUG")) ? atoi(getenv("FMOE_FP8_DEBUG")) : 0;

  const int64_t max_tiles = g.max_blocks * p.n_tiles;
  const int sms = device_sm_count();
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(sms > 0 ? sms : 148, max_tiles));
  p.group_m = pick_group_m(BM, g.k);
  grouped_gemm_tcgen05_fp8_kernel<GATED, MODE, NS><<<grid, kThreads, SMEM_BYTES, st>>>(map_a, map_b, p);
  return launch_status("grouped_gemm_tcgen05_fp8_kernel");
}

}  // namespace

bool gemm_tcgen05_fp8_supports(const GemmParams& p, bool gated) {
  if (p.dtype != FMOE_E4M3 || p.out_dtype != FMOE_BF16) return false;
  if (p.bias || p.activation == FMOE_ACT_SWIGLU_OAI) return false;  // bf16-only variant
  if (p.block_size != BM || p.a_gather) return false;
  if (p.k <= 0 || p.k % 128 != 0 || p.n <= 0 || p.n % 128 != 0) return false;
  if (p.k / 128 > kMaxStagedKBlocks) return false;  // a tile's block scales are staged in shared memory beside the ring
  if (!p.a_scale || !p.w_scale) return false;
  if (!aligned16(p.a) || !aligned16(p.w) || !(aligned16(p.out) && (p.out || (!gated && p.out_rows)))) return false;
  if ((int64_t)p.num_experts * (gated ? 2 * p.n : p.n) >= (1ll << 31) || p.a_rows >= (1ll << 31)) return false;
  if (p.max_blocks >= (1ll << 24) || p.num_experts > 1024) return false;
  return true;
}

int read_wait_profile_fp8(long long* host_out, int n) {
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(host_out, g_wait_prof_fp8, sizeof(long long) * (size_t)n));
  return FMOE_OK;
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
                "tcgen05 fp8 gemm: needs e4m3 in, bf16 out, block_size 128, sorted input rows, n a multiple of 128, "
                "k a multiple of 128 up to 8192");
  if (p.max_blocks <= 0) return FMOE_OK;
  static const int mode = getenv("FMOE_FP8_DEBUG") ? 2 : (getenv("FMOE_TC_PROFILE") ? 1 : 0);
  // ring depth and scale buffers by what fits in shared memory (FMOE_FP8_STAGES=3 forces the three-stage ring)
  const int kblocks = (int)(p.k / 128);
  const char* force = getenv("FMOE_FP8_STAGES");
  int stages = 3, nbuf = 2;
  if (!(force && atoi(force) == 3)) {
    // measured on DeepSeek-V3 T=16384: down GEMM (K = 2048) 3.89 -> 3.78 ms with the fourth stage; the gate/up GEMM
    // (K = 7168) has room for it only with a single scale buffer and was slower that way (5.94 -> 6.27 ms)
    if (smem_bytes(4, 2, kblocks, p.num_experts) <= kMaxSmem) stages = 4;
  }
  auto go = [&](auto gated_c, auto mode_c) {
    constexpr bool G = decltype(gated_c)::value;
    constexpr int M = decltype(mode_c)::value;
    return stages == 4 ? launch<G, M, 4>(p, nbuf, st) : launch<G, M, 3>(p, nbuf, st);
  };
  using T = std::true_type;
  using F = std::false_type;
  if (mode == 2) return gated ? go(T{}, std::integral_constant<int, 2>{}) : go(F{}, std::integral_constant<int, 2>{});
  if (mode == 1) return gated ? go(T{}, std::integral_constant<int, 1>{}) : go(F{}, std::integral_constant<int, 1>{});
  return gated ? go(T{}, std::integral_constant<int, 0>{}) : go(F{}, std::integral_constant<int, 0>{});
}

}  // namespace fmoe
