// Large-M grouped GEMM for sm_100a: persistent, warp-specialised, TMA -> shared
// memory -> tcgen05.mma -> TMEM, epilogue from TMEM.
//
//   tile      : 128 sorted rows (one moe_align block of one expert) x 256 accumulator columns
//   K step    : 128 bytes per row (64 bf16), one 128-byte swizzle atom; 4 MMAs of K=16 per step
//   pipeline  : 4 shared-memory stages (A 16 KB + B 32 KB each), full/empty mbarriers
//   TMEM      : 512 columns = two 128x256 fp32 accumulators, so the epilogue of tile i
//               overlaps the main loop of tile i+1
//   warps     : 0-3 epilogue (TMEM lane quarter = warp id), 4 TMA producer, 5 MMA issuer
//   schedule  : static round-robin over (n_tile, m_block) with m_block fastest, so CTAs that
//               run at the same time share the weight tile through L2
//
// gemm1 (gated): the 256 accumulator columns are 128 gate rows of W and the
// matching 128 up rows, so silu(gate)*up is applied in the epilogue and only
// [rows, I] is written.  gemm2: 256 plain columns, multiplied by the row's top-k
// weight and scattered to the row's flat slot.
//
// Cluster size 1, every CTA loads its own tiles.  (A variant on CTA pairs, cta_group::2 with 256-row tiles, was built and
// measured: it tied with this kernel on every shape tried and was taken out again.)  Every mbarrier wait is bounded; on expiry the
// kernel records a code in a device status word, leaves its loops, frees TMEM and returns.
#include "gemm.cuh"
#include "ptx_sm100.cuh"

#include <cstdlib>
#include <mutex>

namespace fmoe {

__device__ int g_device_status = 0;  // 0 = fine; otherwise (role << 8 | site) of the first wait that gave up
// Optional wait-time profile (FMOE_TC_PROFILE=1): per CTA {tiles, mma wait acc, mma wait data, producer wait, epilogue wait, epilogue busy}
__device__ long long g_wait_prof[256 * 8];

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
// Ring geometry for KB bytes of K per stage row.  KB = 128 (64 bf16, 128-byte swizzle, 4 stages of 48 KB) is the
// one in use; a 9-stage ring of 64-byte rows (64-byte swizzle) was measured 35-40 % slower on B200 and an L2
// prefetch of the weight boxes 6-15 % slower, so neither is built.
template <int KB>
struct Ring {
  static constexpr int KBYTES = KB;
  static_assert(KB == 128, "only the 128-byte ring is built");
  static constexpr int STAGES = 4;
  static constexpr int A_BYTES = BM * KB;
  static constexpr int B_BYTES = BN * KB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;  // + expert table
};
constexpr int TMEM_COLS = 512;
constexpr int kThreads = 192;

struct TcParams {
  const int32_t* sorted_token_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_post_padded;
  const float* row_scale;
  const float* a_scale;   // F8: [rows] f32, one scale per (sorted) input row; or per token (a_scale_gather)
  int32_t a_scale_gather;
  const float* w_scale;   // F8: [E, w_rows] f32, one scale per output channel
  const float* bias;      // optional [E, w_rows] f32
  float act_alpha, act_limit;
  void* out;
  void* const* out_rows;  // down projection: optional per-slot row addresses (may be peer memory)
  int64_t numel;
  int64_t n;           // gemm1: I, gemm2: H
  int64_t w_rows;      // rows of W per expert
  int64_t sorted_cap;
  int32_t num_experts;
  int32_t k_steps;     // ceil(K*elem / 128)
  int32_t n_tiles;
  int32_t max_blocks;
  int32_t activation;
  int32_t group_m;
  int32_t profile;
  int32_t l2_hints;    // 1: TMA loads carry L2 eviction priorities (weights evict_first, activation rows evict_last)
  int32_t debug;       // timing experiments only (results are wrong).  bit 0: no TMA loads, the MMA warp never waits for
                       // data; bit 1: no MMAs (the ring and its barriers alone); bit 2: B read as an N-major operand;
                       // bit 3: every load fetches the first tile (all L2 hits); bit 4: the ring re-arms a stage as soon as
                       // its own data has landed and the MMA warp never waits (both run, uncoupled)
  int32_t ring_depth;  // experiment: stages of the ring in use (default all)
  float* split_partials;    // tail split: [CTAs][128][256] f32 partial accumulators (NULL: no split)
  int32_t* split_counters;  // tail split: [CTAs] arrivals per split tile, zero at launch
  int32_t split_max;        // tail split: most K slices per tile (< 2: no split)
  int32_t top_k;       // gather mode: input row of slot s is s / top_k
  int32_t a_rows;      // gather mode: rows of the input tensor (a row index >= a_rows reads zeros)
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_device_status, 0, code); }

// Bounded wait whose verdict is uniform across the warp, so that the role loops never diverge around
// their __syncwarp() points.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
}

__device__ __forceinline__ bool warp_wait_relaxed(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait_relaxed(bar, parity));
}

// Work units of one CTA.  Tiles are dealt round-robin; when the last round has work for at most half of the CTAs
// (the CTAs are bound by their own rate, so a part-filled round costs as much as a full one), each of its tiles is
// cut into S slices along K (S a power of two) that S neighbouring CTAs compute.  The S partial accumulators are then
// summed by all S CTAs together: CTA s owns the s-th strip of the tile's columns, publishes the other strips of its
// partial in global memory, waits until all S have done so, adds the other CTAs' partials of its strip in slice
// order (a fixed order: results do not depend on timing) and runs the epilogue on the strip.
struct UnitPlan {
  int64_t total, rounds, left;
  int grid, b, S, k_steps;
  __host__ __device__ __forceinline__ void init(int64_t total_tiles, int k_steps_, int max_split, int grid_, int b_) {
    total = total_tiles;
    k_steps = k_steps_;
    grid = grid_;
    b = b_;
    S = 1;
    rounds = (total + grid - 1) / grid;
    left = total - (rounds - 1) * grid;
    if (total > 0 && max_split >= 2 && left * 2 <= grid) {
      int s = (int)(max_split < grid / left ? max_split : grid / left);
      s = s < k_steps / 8 ? s : k_steps / 8;
      while (s & (s - 1)) s &= s - 1;  // largest power of two below
      if (s >= 2) S = s;
    }
  }
  // unit `it` of this CTA: tile, K steps [ks0, ks1), slice (always 0 for whole tiles); false past the last unit
  __host__ __device__ __forceinline__ bool get(int64_t it, int64_t* tile, int* ks0, int* ks1, int* slice) const {
    *ks0 = 0;
    *ks1 = k_steps;
    *slice = 0;
    if (S == 1 || it < rounds - 1) {
      *tile = b + it * grid;
      return *tile < total;
    }
    if (it > rounds - 1 || b >= left * S) return false;
    *tile = (rounds - 1) * grid + b / S;
    *slice = b % S;
    *ks0 = (int)((int64_t)k_steps * *slice / S);
    *ks1 = (int)((int64_t)k_steps * (*slice + 1) / S);
    return true;
  }
  __host__ __device__ __forceinline__ bool is_split(int64_t it) const { return S > 1 && it == rounds - 1; }
};

__device__ __forceinline__ void store_partial32(const uint32_t (&r)[32], float* dst) {
#pragma unroll
  for (int q = 0; q < 8; ++q)
    __stcg(reinterpret_cast<float4*>(dst) + q, make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                           __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
}
__device__ __forceinline__ void add_partial32(uint32_t (&r)[32], const float* src) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(src) + q);
    r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + v.x);
    r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + v.y);
    r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + v.z);
    r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + v.w);
  }
}
__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// GATHER: the A operand is the un-permuted [a_rows, K] input; the producer warp fetches row
// sorted_token_ids[p] / top_k for sorted position p with TMA gather4 (32 lanes x 4 rows = one 128-row stage),
// padding positions read row a_rows, which is outside the tensor and arrives as zeros.
// EXTRA: the epilogue adds a bias and/or applies the swiglu_oai unit; a separate instantiation, so that the plain
// silu/gelu kernels keep their register allocation.
// BNMAJ: the weights are [E, K, N] (N contiguous: the layout the reference operator takes, w1 [E,H,2I] / w2 [E,I,H])
// and are read in place as an N-major B operand.  A stage's B part is four TMA boxes of 64 K rows x 64 columns
// (128 bytes, one swizzle atom wide) from a 3-D map [E, K, N]: K rows past the expert's last and columns past N are
// zero-filled by TMA.  In shared memory the boxes are 8 KB apart (the descriptor's leading byte offset), groups of
// 8 K rows 1 KB apart (its stride byte offset), and one MMA's 16 K rows are 2 KB.
// F8: e4m3 operands with per-row activation scales and per-output-channel weight scales (per-channel w8a8): the
// same pipeline with 128 K elements per stage and kind::f8f6f4 MMAs; the scales multiply the finished accumulator
// in the epilogue, so nothing is folded per K block.
template <bool GATED, int KB, bool GATHER, bool EXTRA, bool BNMAJ, bool F8>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const TcParams p) {
  constexpr int KBYTES = Ring<KB>::KBYTES, STAGES = Ring<KB>::STAGES, A_BYTES = Ring<KB>::A_BYTES,
                B_BYTES = Ring<KB>::B_BYTES, STAGE_BYTES = Ring<KB>::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;        // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;     // [2] MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  int32_t* expert_table = reinterpret_cast<int32_t*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&acc_full[a], 1);
      ptx::mbar_init(&acc_empty[a], 128);
    }
    ptx::fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 5) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  const int used_blocks = min((int)(*p.num_tokens_post_padded / BM), p.max_blocks);
  const int64_t total_tiles = (int64_t)used_blocks * p.n_tiles;
  ptx::tc_fence_before_sync();
  build_expert_table(expert_table, p.num_experts, p.expert_ids, used_blocks);  // ends with __syncthreads()
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  TileCursor cursor;
  const int k_steps = p.k_steps;
  UnitPlan plan;
  plan.init(total_tiles, k_steps, p.split_partials ? min(p.split_max, GATED ? 4 : 8) : 0, (int)gridDim.x, (int)blockIdx.x);

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    long long prof_a = 0;
    // coordinates of a tile; looked up one tile ahead so that the index loads never stall the ring
    auto tile_rows = [&](int64_t tile, int32_t* row_a, int32_t* row_b0, int32_t* row_b1) {
      int m_blk, n_tile, e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &e);
      *row_a = m_blk * BM;
      if constexpr (BNMAJ) {  // first column of the tile, expert
        *row_b0 = GATED ? n_tile * 128 : n_tile * 256;
        *row_b1 = e;
      } else {
        *row_b0 = (int32_t)((int64_t)e * p.w_rows + (GATED ? (int64_t)n_tile * 128 : (int64_t)n_tile * 256));
        *row_b1 = GATED ? (int32_t)(*row_b0 + p.n) : *row_b0 + 128;
      }
    };
    // gather mode: the four input rows this lane fetches for sorted positions row_a + 4*lane .. +3
    auto lane_rows = [&](int32_t row_a) {
      int4 s = *reinterpret_cast<const int4*>(p.sorted_token_ids + row_a + 4 * lane);
      auto src = [&](int32_t slot) { return (slot >= 0 && slot < p.numel) ? slot / p.top_k : p.a_rows; };
      return make_int4(src(s.x), src(s.y), src(s.z), src(s.w));
    };
    const uint64_t pol_w = ptx::l2_policy_evict_first(), pol_a = ptx::l2_policy_evict_last();
    int32_t row_a = 0, row_b0 = 0, row_b1 = 0, nrow_a = 0, nrow_b0 = 0, nrow_b1 = 0;
    int4 src_rows = make_int4(0, 0, 0, 0), nsrc_rows = src_rows;
    int64_t tile, ntile;
    int ks0, ks1, slice, nks0 = 0, nks1 = 0, nslice;
    bool have = plan.get(0, &tile, &ks0, &ks1, &slice);
    if (have) {
      tile_rows(tile, &row_a, &row_b0, &row_b1);
      if constexpr (GATHER) src_rows = lane_rows(row_a);
    }
    for (int64_t it = 0; have && alive && !(p.debug & 1); ++it) {
      const bool has_next = plan.get(it + 1, &ntile, &nks0, &nks1, &nslice);
      for (int ks = ks0; ks < ks1; ++ks) {
        const long long tp0 = p.profile ? clock64() : 0;
        const bool okp = warp_wait((p.debug & 16) ? &full_bar[stage] : &empty_bar[stage], phase ^ 1);
        if (p.profile) prof_a += clock64() - tp0;
        if (!okp) {
          report(0x100 | stage);
          alive = false;
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int32_t x = ks * (KBYTES / (F8 ? 1 : 2));  // element coordinate
          if (p.debug & 8) row_a = row_b0 = row_b1 = 0;  // experiment: every CTA loads the same tiles (L2 hits)
          if constexpr (BNMAJ) {
            ptx::tma_load_2d(sa, &map_a, x, row_a, &full_bar[stage]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int32_t col = GATED ? row_b0 + (j & 1) * 64 + (j >> 1) * (int32_t)p.n : row_b0 + j * 64;
              ptx::tma_load_3d(sb + j * (B_BYTES / 4), &map_b, col, x, row_b1, &full_bar[stage]);
            }
          } else if (p.l2_hints) {
            if constexpr (!GATHER) ptx::tma_load_2d_hint(sa, &map_a, x, row_a, &full_bar[stage], pol_a);
            ptx::tma_load_2d_hint(sb, &map_b, x, row_b0, &full_bar[stage], pol_w);
            ptx::tma_load_2d_hint(sb + B_BYTES / 2, &map_b, x, row_b1, &full_bar[stage], pol_w);
          } else {
            if constexpr (!GATHER) ptx::tma_load_2d(sa, &map_a, x, row_a, &full_bar[stage]);
            ptx::tma_load_2d(sb, &map_b, x, row_b0, &full_bar[stage]);
            ptx::tma_load_2d(sb + B_BYTES / 2, &map_b, x, row_b1, &full_bar[stage]);
          }
        }
        __syncwarp();
        if constexpr (GATHER) {
          // after lane 0 armed the barrier: every lane brings its 4 rows (4 x 128 B) of the stage
          ptx::tma_gather4_2d(smem + stage * STAGE_BYTES + lane * (4 * KBYTES), &map_a, ks * (KBYTES / 2), src_rows.x,
                              src_rows.y, src_rows.z, src_rows.w, &full_bar[stage]);
        }
        if (ks == ks0 && has_next) {
          tile_rows(ntile, &nrow_a, &nrow_b0, &nrow_b1);
          if constexpr (GATHER) nsrc_rows = lane_rows(nrow_a);
        }
        if (++stage == p.ring_depth) {
          stage = 0;
          phase ^= 1;
        }
      }
      row_a = nrow_a;
      row_b0 = nrow_b0;
      row_b1 = nrow_b1;
      src_rows = nsrc_rows;
      have = has_next;
      ks0 = nks0;
      ks1 = nks1;
    }
    if (p.profile && lane == 0 && blockIdx.x < 256) g_wait_prof[blockIdx.x * 8 + 3] = prof_a;
    // drain: do not leave while our own bulk copies may still be landing in shared memory
    if (alive && !(p.debug & 1)) {
      for (int s = 0; s < p.ring_depth; ++s) {
        // the consumer releases a stage only after its data arrived, so waiting for every
        // stage to be free again covers all outstanding copies
        if (!warp_wait((p.debug & 16) ? &full_bar[stage] : &empty_bar[stage], phase ^ 1)) {
          report(0x180 | stage);
          break;
        }
        if (++stage == p.ring_depth) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc =
        ptx::make_idesc(F8 ? /*e4m3*/ 0 : /*bf16*/ 1, BM, BN) | (BNMAJ ? (1u << 16) : 0u);  // bit 16: B is N-major
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool alive = true;
    long long prof_acc = 0, prof_data = 0;
    int64_t tile;
    int ks0, ks1, slice;
    for (int64_t it = 0; alive && plan.get(it, &tile, &ks0, &ks1, &slice); ++it) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const long long tm0 = p.profile ? clock64() : 0;
      const bool oka = warp_wait(&acc_empty[acc], acc_phase ^ 1);
      if (p.profile) prof_acc += clock64() - tm0;
      if (!oka) {
        report(0x200 | acc);
        alive = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int ks = ks0; ks < ks1; ++ks) {
        const long long tm1 = p.profile ? clock64() : 0;
        const bool okd = (p.debug & 17) ? true : warp_wait(&full_bar[stage], phase);
        if (p.profile) prof_data += clock64() - tm1;
        if (!okd) {
          report(0x240 | stage);
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = ptx::smem_desc_sw128(sa);
          const uint64_t db = ptx::smem_desc_sw128(sa + A_BYTES);
          if constexpr (F8) {
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk)  // 32 bytes of K per MMA (32 e4m3)
              ptx::mma_f8f6f4_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, ((ks - ks0) | kk) != 0);
            ptx::mma_commit(&empty_bar[stage]);
          } else if constexpr (BNMAJ) {
            const uint64_t dbn = ptx::smem_desc_sw128_lbo(sa + A_BYTES, B_BYTES / 4, 1024);
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk)
              ptx::mma_f16_ss(d_tmem, da + 2 * kk, dbn + (2048 >> 4) * kk, idesc, ((ks - ks0) | kk) != 0);
            ptx::mma_commit(&empty_bar[stage]);
          } else if (p.debug & 2) {
            ptx::mbar_arrive(&empty_bar[stage]);
          } else if (p.debug & 4) {
            // B as an N-major operand: 64 columns (128 B) x 8 K rows per swizzle atom, atoms of the next 8 K rows
            // 1024 B on, of the next 64 columns 8192 B on; 16 K rows per MMA = 2048 B
            const uint64_t dbn = ptx::smem_desc_sw128_lbo(sa + A_BYTES, 8192, 1024);
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk)
              ptx::mma_f16_ss(d_tmem, da + 2 * kk, dbn + 128 * kk, idesc | (1u << 16), ((ks - ks0) | kk) != 0);
            if (!(p.debug & 1)) ptx::mma_commit(&empty_bar[stage]);
          } else {
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk) {
              // 32 bytes of K per MMA (16 bf16): advance the start address by 32 B = 2 units
              ptx::mma_f16_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, ((ks - ks0) | kk) != 0);
            }
            if (!(p.debug & 17)) ptx::mma_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
          }
        }
        __syncwarp();
        if (++stage == p.ring_depth) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (alive && lane == 0) ptx::mma_commit(&acc_full[acc]);
      __syncwarp();
    }
    if (p.profile && lane == 0 && blockIdx.x < 256) {
      g_wait_prof[blockIdx.x * 8 + 0] = local;
      g_wait_prof[blockIdx.x * 8 + 1] = prof_acc;
      g_wait_prof[blockIdx.x * 8 + 2] = prof_data;
    }
  } else {
    // ---------------- epilogue (warps 0-3) ----------------
    int local = 0;
    bool alive = true;
    long long prof_wait = 0, prof_busy = 0;
    const int row = warp * 32 + lane;
    int64_t tile;
    int ks0, ks1, slice;
    for (int64_t it = 0; alive && plan.get(it, &tile, &ks0, &ks1, &slice); ++it) {
      int m_blk, n_tile, tile_e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &tile_e);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const int64_t pos = (int64_t)m_blk * BM + row;
      const int32_t slot = (pos < p.sorted_cap) ? p.sorted_token_ids[pos] : -1;
      const bool valid = slot >= 0 && slot < p.numel;
      float rs = (valid && p.row_scale) ? p.row_scale[slot] : 1.0f;
      if constexpr (F8)  // activation scale of this row: by sorted position, or by the token the slot belongs to
        rs *= p.a_scale_gather ? (valid ? p.a_scale[slot / p.top_k] : 0.f) : ((pos < p.sorted_cap) ? p.a_scale[pos] : 0.f);
      const float* wsc = F8 ? p.w_scale + (int64_t)tile_e * p.w_rows + (int64_t)n_tile * (GATED ? 128 : 256) : nullptr;
      // bias entries of this tile's columns (the same for every row: broadcast loads)
      const float* bias = (EXTRA && p.bias)
                              ? p.bias + (int64_t)tile_e * p.w_rows +
                                    (int64_t)n_tile * (GATED ? 128 : 256)
                              : nullptr;
      const long long te0 = p.profile ? clock64() : 0;
      const bool oke = warp_wait_relaxed(&acc_full[acc], acc_phase);
      const long long te1 = p.profile ? clock64() : 0;
      prof_wait += te1 - te0;
      if (!oke) {
        report(0x300 | acc);
        alive = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(warp * 32) << 16);
      // tail split: this CTA runs the epilogue on chunks [c_begin, c_end) of the tile's columns (32 accumulator
      // columns per chunk; gated: gate chunk c and up chunk c together); bufs + o * BM * BN is row `row` of the
      // partial accumulator that slice o published
      constexpr int NCH = GATED ? 4 : 8;
      const bool split = plan.is_split(it);
      const int S = split ? plan.S : 1;
      const int c_begin = slice * NCH / S, c_end = (slice + 1) * NCH / S;
      const int tail_index = plan.b / plan.S;
      const float* bufs = p.split_partials + ((int64_t)tail_index * S * BM + row) * BN;
      if (split) {
        float* mine = p.split_partials + (((int64_t)tail_index * S + slice) * BM + row) * BN;
#pragma unroll 1
        for (int c = 0; c < NCH; ++c) {
          if (c >= c_begin && c < c_end) continue;
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          store_partial32(r, mine + c * 32);
          if constexpr (GATED) {
            ptx::tmem_ld_32x32b_x32(taddr + 128 + c * 32, r);
            ptx::tmem_ld_wait();
            store_partial32(r, mine + 128 + c * 32);
          }
        }
        __threadfence();  // the strips are visible device-wide before this warp counts as arrived
        __syncwarp();
        if (lane == 0) atomicAdd(p.split_counters + tail_index, 1);
        // every epilogue warp of every slice has published: 4 * S arrivals
        const long long t0 = clock64();
        bool ok = true;
        while (ld_acquire_gpu(p.split_counters + tail_index) < 4 * S) {
          if (clock64() - t0 > 2000000000ll) {
            ok = false;
            break;
          }
          __nanosleep(64);
        }
        if (!__all_sync(0xffffffffu, ok)) {
          report(0x380 | acc);
          alive = false;
          break;
        }
      }
      if constexpr (GATED) {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + pos * p.n + (int64_t)n_tile * 128;
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t g[32], u[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, g);
          ptx::tmem_ld_32x32b_x32(taddr + 128 + c * 32, u);
          ptx::tmem_ld_wait();
          for (int o = 0; o < S; ++o) {
            if (o == slice) continue;
            add_partial32(g, bufs + (int64_t)o * BM * BN + c * 32);
            add_partial32(u, bufs + (int64_t)o * BM * BN + 128 + c * 32);
          }
          // the last column tile of an intermediate size that is not a multiple of 128 is cut at I (its surplus
          // accumulator columns hold products with rows of W that belong to the up half or to the next expert)
          if (pos < p.sorted_cap && (int64_t)n_tile * 128 + c * 32 < p.n) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
              // bias of the 8 gate and 8 up columns of this piece: four 16-byte broadcast loads
              float bgv[8], buv[8];
              if ((EXTRA && bias) || F8) {
                // bias (EXTRA) or channel scales (F8) of the 8 gate and 8 up columns: 16-byte broadcast loads
                const float* vec = F8 ? wsc : bias;
                const float4* pg = reinterpret_cast<const float4*>(vec + c * 32 + v * 8);
                const float4* pu = reinterpret_cast<const float4*>(vec + p.n + c * 32 + v * 8);
                const float4 g0 = __ldg(pg), g1 = __ldg(pg + 1), u0 = __ldg(pu), u1 = __ldg(pu + 1);
                bgv[0] = g0.x; bgv[1] = g0.y; bgv[2] = g0.z; bgv[3] = g0.w;
                bgv[4] = g1.x; bgv[5] = g1.y; bgv[6] = g1.z; bgv[7] = g1.w;
                buv[0] = u0.x; buv[1] = u0.y; buv[2] = u0.z; buv[3] = u0.w;
                buv[4] = u1.x; buv[5] = u1.y; buv[6] = u1.z; buv[7] = u1.w;
              } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) bgv[q] = buv[q] = 0.f;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int i = v * 8 + j * 2;
                float o0, o1;
                if constexpr (EXTRA) {
                  o0 = gated_output<true>(__uint_as_float(g[i]), __uint_as_float(u[i]), bgv[2 * j], buv[2 * j], rs,
                                          p.activation, p.act_alpha, p.act_limit);
                  o1 = gated_output<true>(__uint_as_float(g[i + 1]), __uint_as_float(u[i + 1]), bgv[2 * j + 1],
                                          buv[2 * j + 1], rs, p.activation, p.act_alpha, p.act_limit);
                } else if constexpr (F8) {
                  // (accumulator * row scale) * channel scale, then the activation
                  o0 = act_mul_fast(__uint_as_float(g[i]) * rs * bgv[2 * j], __uint_as_float(u[i]) * rs * buv[2 * j],
                                    p.activation);
                  o1 = act_mul_fast(__uint_as_float(g[i + 1]) * rs * bgv[2 * j + 1],
                                    __uint_as_float(u[i + 1]) * rs * buv[2 * j + 1], p.activation);
                } else {
                  o0 = act_mul_fast(__uint_as_float(g[i]) * rs, __uint_as_float(u[i]) * rs, p.activation);
                  o1 = act_mul_fast(__uint_as_float(g[i + 1]) * rs, __uint_as_float(u[i + 1]) * rs, p.activation);
                }
                w[j] = pack_bf16x2(o0, o1);
              }
              dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      } else {
        __nv_bfloat16* obase = !valid ? nullptr
                               : p.out_rows ? reinterpret_cast<__nv_bfloat16*>(p.out_rows[slot])
                                            : reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)slot * p.n;
        __nv_bfloat16* orow = obase + (int64_t)n_tile * 256;
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          for (int o = 0; o < S; ++o)
            if (o != slice) add_partial32(r, bufs + (int64_t)o * BM * BN + c * 32);
          if (obase && (int64_t)n_tile * 256 + c * 32 < p.n) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
              float bv[8];
              if ((EXTRA && bias) || F8) {
                const float4* pb = reinterpret_cast<const float4*>((F8 ? wsc : bias) + c * 32 + v * 8);
                const float4 b0 = __ldg(pb), b1 = __ldg(pb + 1);
                bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
              } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) bv[q] = 0.f;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int i = v * 8 + j * 2;
                if constexpr (F8)
                  w[j] = pack_bf16x2(__uint_as_float(r[i]) * rs * bv[2 * j], __uint_as_float(r[i + 1]) * rs * bv[2 * j + 1]);
                else
                  w[j] = pack_bf16x2((__uint_as_float(r[i]) + bv[2 * j]) * rs, (__uint_as_float(r[i + 1]) + bv[2 * j + 1]) * rs);
              }
              dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      // accumulator may be overwritten by the MMA warp from here on
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&acc_empty[acc]);
      if (p.profile) prof_busy += clock64() - te1;
    }
    if (p.out_rows) __threadfence_system();  // rows stored to a peer are complete before the kernel ends
    if (p.profile && threadIdx.x == 0 && blockIdx.x < 256) {
      g_wait_prof[blockIdx.x * 8 + 4] = prof_wait;
      g_wait_prof[blockIdx.x * 8 + 5] = prof_busy;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ----------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace

// SM count of the current device (cached per device ordinal).
int device_sm_count() {
  static std::mutex mu;
  static int sm_count[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev < 0 || dev >= kMaxDevices) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  return sm_count[dev];
}

// Host-side view of the work-unit plan (the same code the kernels run), for tests.
int tail_plan_unit(int64_t total_tiles, int k_steps, int max_split, int grid, int cta, int64_t it, int64_t* out) {
  UnitPlan plan;
  plan.init(total_tiles, k_steps, max_split, grid, cta);
  int64_t tile = 0;
  int ks0 = 0, ks1 = 0, slice = 0;
  if (!plan.get(it, &tile, &ks0, &ks1, &slice)) return 0;
  out[0] = tile;
  out[1] = ks0;
  out[2] = ks1;
  out[3] = slice;
  out[4] = plan.is_split(it) ? plan.S : 1;
  return 1;
}

int64_t gemm_tcgen05_split_workspace_bytes() {
  const int sms = device_sm_count();
  return 1024 + (int64_t)std::min(std::max(sms, 1), 256) * BM * BN * 4;
}

// 2-D row-major [rows, cols] tensor of `elem_bytes` elements; box = kbytes (128 or 64) x box_rows, swizzle of the same width.
int make_tensor_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes, int box_rows,
                       bool weights, int kbytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(kbytes / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  kbytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  weights ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return FMOE_OK;
}

// bf16 weights [E, K, N] with N contiguous; box = 64 columns (128 bytes, the swizzle width) x 64 K rows of one expert.
int make_tensor_map_nmajor(CUtensorMap* map, const void* base, int64_t experts, int64_t k, int64_t n) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)k, (cuuint64_t)experts};
  cuuint64_t strides[2] = {(cuuint64_t)n * 2, (cuuint64_t)n * (cuuint64_t)k * 2};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled (N-major weights) failed with code %d", (int)r);
  return FMOE_OK;
}

namespace {

template <bool GATED, int KB, bool GATHER, bool EXTRA, bool BNMAJ = false, bool F8 = false>
int launch(const GemmParams& g, cudaStream_t st) {
  constexpr int ELEM = F8 ? 1 : 2;
  constexpr int KBYTES = KB;
  constexpr int MAX_SMEM = Ring<KB>::SMEM_BYTES + expert_table_bytes(1024);
  const int SMEM_BYTES = Ring<KB>::SMEM_BYTES + expert_table_bytes(g.num_experts);
  const int sm_count = device_sm_count();
  static PerDeviceOnce once_attr;  // the opt-in to > 48 KB of dynamic shared memory is per device
  const cudaError_t attr_err = per_device_once(once_attr, [] {
    return cudaFuncSetAttribute(grouped_gemm_tcgen05_kernel<GATED, KB, GATHER, EXTRA, BNMAJ, F8>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
  });
  if (attr_err != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", SMEM_BYTES, cudaGetErrorString(attr_err));

  const int64_t w_rows = GATED ? 2 * g.n : g.n;
  CUtensorMap map_a, map_b;
  int rc = make_tensor_map_2d(&map_a, g.a, g.a_rows, g.k, ELEM, GATHER ? 1 : BM, false, KB);
  if (rc) return rc;
  if constexpr (BNMAJ) rc = make_tensor_map_nmajor(&map_b, g.w, g.num_experts, g.k, w_rows);
  else rc = make_tensor_map_2d(&map_b, g.w, (int64_t)g.num_experts * w_rows, g.k, ELEM, 128, true, KB);
  if (rc) return rc;

  TcParams p;
  p.sorted_token_ids = g.sorted_token_ids;
  p.expert_ids = g.expert_ids;
  p.num_tokens_post_padded = g.num_tokens_post_padded;
  p.row_scale = g.row_scale;
  p.a_scale = g.a_scale;
  p.a_scale_gather = g.a_scale_gather;
  p.w_scale = g.w_scale;
  p.bias = g.bias;
  p.act_alpha = g.act_alpha;
  p.act_limit = g.act_limit;
  p.out = g.out;
  p.out_rows = GATED ? nullptr : g.out_rows;
  p.numel = g.numel;
  p.n = g.n;
  p.w_rows = w_rows;
  p.sorted_cap = g.sorted_cap;
  p.num_experts = g.num_experts;
  p.k_steps = (int)ceil_div<int64_t>(g.k * ELEM, KBYTES);
  p.n_tiles = (int)ceil_div<int64_t>(g.n, GATED ? 128 : 256);
  p.max_blocks = (int)g.max_blocks;
  p.activation = g.activation;
  p.top_k = g.top_k;
  p.a_rows = (int32_t)g.a_rows;

  const int64_t max_tiles = g.max_blocks * p.n_tiles;
  unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(sm_count > 0 ? sm_count : 148, max_tiles));
  if (const char* cap = getenv("FMOE_TC_MAX_CTAS")) grid = std::max(1u, std::min(grid, (unsigned)atoi(cap)));  // experiment
  p.group_m = pick_group_m(BM, g.k * ELEM);
  p.profile = getenv("FMOE_TC_PROFILE") != nullptr;
  p.debug = getenv("FMOE_TC_DEBUG") ? atoi(getenv("FMOE_TC_DEBUG")) : 0;
  p.l2_hints = getenv("FMOE_TC_L2_HINTS") ? atoi(getenv("FMOE_TC_L2_HINTS")) : 0;
  // tail split: counters (1 KB, cleared before every launch) + one 128x256 f32 partial per CTA
  p.split_partials = nullptr;
  p.split_counters = nullptr;
  p.split_max = 0;
  const char* split_env = getenv("FMOE_TC_SPLIT_TAIL");  // "0": off (read per launch, tests flip it)
  const bool split_off = split_env && atoi(split_env) == 0;
  // one partial per CTA must fit: the scratch is sized for the SM count, the grid never exceeds it
  const bool split_fits = g.split_ws_bytes >= 1024 + (int64_t)grid * BM * BN * 4 && grid <= 256;
  if (g.split_ws && !split_off && split_fits && aligned16(g.split_ws)) {
    p.split_counters = reinterpret_cast<int32_t*>(g.split_ws);
    p.split_partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g.split_ws) + 1024);
    p.split_max = 8;
    FMOE_CUDA_OK(cudaMemsetAsync(g.split_ws, 0, 1024, st));
  }
  p.ring_depth = Ring<KB>::STAGES;
  if (const char* d = getenv("FMOE_TC_RING_DEPTH")) p.ring_depth = std::max(1, std::min(Ring<KB>::STAGES, atoi(d)));
  grouped_gemm_tcgen05_kernel<GATED, KB, GATHER, EXTRA, BNMAJ, F8><<<grid, kThreads, SMEM_BYTES, st>>>(map_a, map_b, p);
  return launch_status("grouped_gemm_tcgen05_kernel");
}

}  // namespace

bool gemm_tcgen05_supports(const GemmParams& p, bool gated) {
  const bool f8 = p.dtype == FMOE_E4M3 && p.scale_mode == FMOE_SCALE_CHANNEL;
  if ((p.dtype != FMOE_BF16 && !f8) || p.out_dtype != FMOE_BF16) return false;
  // e4m3 with per-row / per-channel scales: plain kernels, K-major weights, sorted input rows
  if (f8 && (p.a_gather || p.bias || p.w_layout != FMOE_W_K_MAJOR || !p.a_scale || !p.w_scale || !aligned16(p.w_scale) ||
             (gated && p.activation == FMOE_ACT_SWIGLU_OAI)))
    return false;
  if (p.block_size != BM) return false;
  // gather mode: gate/up GEMM only; one int4 of sorted ids per lane
  if (p.a_gather && (!gated || p.top_k < 1 || !aligned16(p.sorted_token_ids))) return false;
  if (p.w_layout != FMOE_W_K_MAJOR && p.w_layout != FMOE_W_N_MAJOR) return false;
  // weights in the reference operator's [E, K, N] layout: plain kernels only (no row gather, bias or swiglu_oai)
  if (p.w_layout == FMOE_W_N_MAJOR && (p.a_gather || p.bias || (gated && p.activation == FMOE_ACT_SWIGLU_OAI))) return false;
  if (p.bias && !aligned16(p.bias)) return false;  // 16-byte bias loads in the epilogue (n % 32 == 0 holds already)
  if (p.k <= 0 || (p.k * (f8 ? 1 : 2)) % 16 != 0) return false;  // TMA row stride must be a multiple of 16 bytes
  if (p.n <= 0 || p.n % 32 != 0) return false;  // 64-byte epilogue stores; column tiles are cut at n in 32-column pieces
  if (!aligned16(p.a) || !aligned16(p.w) || !(aligned16(p.out) && (p.out || (!gated && p.out_rows)))) return false;
  if ((int64_t)p.num_experts * (gated ? 2 * p.n : p.n) >= (1ll << 31) || p.a_rows >= (1ll << 31)) return false;
  if (p.max_blocks >= (1ll << 24) || p.num_experts > 1024) return false;
  return true;
}

int gemm_tcgen05(const GemmParams& p, bool gated, cudaStream_t st) {
  if (!gemm_tcgen05_supports(p, gated))
    return fail(FMOE_ERR_UNSUPPORTED,
                "tcgen05 gemm: needs bf16 in/out (or e4m3 in with per-channel scales), block_size 128, input-row gather only for the gate/up gemm, "
                "n %% %d == 0, 16-byte aligned pointers (got dtype=%d block=%d a_gather=%d n=%lld k=%lld)",
                32, p.dtype, p.block_size, p.a_gather, (long long)p.n, (long long)p.k);
  if (p.max_blocks <= 0) return FMOE_OK;
  const bool extra = p.bias != nullptr || (gated && p.activation == FMOE_ACT_SWIGLU_OAI);
  if (p.dtype == FMOE_E4M3)
    return gated ? launch<true, 128, false, false, false, true>(p, st) : launch<false, 128, false, false, false, true>(p, st);
  if (p.w_layout == FMOE_W_N_MAJOR)
    return gated ? launch<true, 128, false, false, true>(p, st) : launch<false, 128, false, false, true>(p, st);
  if (p.a_gather) return extra ? launch<true, 128, true, true>(p, st) : launch<true, 128, true, false>(p, st);
  if (gated) return extra ? launch<true, 128, false, true>(p, st) : launch<true, 128, false, false>(p, st);
  return extra ? launch<false, 128, false, true>(p, st) : launch<false, 128, false, false>(p, st);
}

namespace {
// Self-test of the time-out path: waits on a barrier that nobody signals, with a short limit.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_barrier_init();
  }
  __syncthreads();
  if (!ptx::mbar_wait_limit(&bar, 0, limit_cycles) && threadIdx.x == 0) report(0xE00);
}
}  // namespace

int launch_bounded_wait_selftest(long long limit_cycles, cudaStream_t st) {
  bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(limit_cycles);
  return launch_status("bounded_wait_selftest_kernel");
}

int read_wait_profile(long long* host_out, int n) {
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(host_out, g_wait_prof, sizeof(long long) * (size_t)n));
  return FMOE_OK;
}

int status_word_fp8(int* out, bool clear);
int status_word_ep(int* out, bool clear);

// First non-zero status word of the translation units that keep one (tcgen05 kernels, expert-parallel
// exchange); all are cleared.
int read_and_clear_device_status(cudaStream_t st, int* status_out) {
  int zero = 0, a = 0, b = 0, d = 0;
  FMOE_CUDA_OK(cudaStreamSynchronize(st));
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(&a, g_device_status, sizeof(int)));
  if (a != 0) FMOE_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
  int rc = status_word_fp8(&b, true);
  if (rc) return rc;
  rc = status_word_ep(&d, true);
  if (rc) return rc;
  *status_out = a ? a : (b ? b : d);
  return FMOE_OK;
}

}  // namespace fmoe
