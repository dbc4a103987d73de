// Large-M bf16 grouped GEMM on CTA pairs (cluster of 2, tcgen05 cta_group::2).
//
// With one CTA per 128x256 tile every K=16 MMA reads 12 KB of shared memory in 128 clocks while TMA
// writes as much: shared-memory bandwidth caps that kernel at about two thirds of the tensor rate.
// Here two CTAs of a cluster share one 256x256 tile: each holds its own 128 rows of A and HALF of the
// B tile (128 of the 256 weight rows), one tcgen05.mma of M=256 spans both, so per CTA the MMA reads
// 8 KB per 128 clocks and TMA writes 8 KB.
//
//   tile     : 256 sorted rows (one moe_align block of 256 rows of one expert) x 256 accumulator columns
//   stage    : A 128x64 bf16 (16 KB) + B-half 128x64 bf16 (16 KB) per CTA; 6 stages
//   TMEM     : 512 columns per CTA = two 128x256 fp32 accumulators (rows of this CTA)
//   CTA 0    : issues all MMAs; its full barriers collect the bytes of both CTAs' loads
//   both     : TMA producer warp (own A rows, own half of B), 4 epilogue warps (own rows)
// gemm1: CTA 0 loads the 128 gate rows, CTA 1 the matching 128 up rows, so accumulator columns
// [0,128) are gate and [128,256) up, as in the single-CTA kernel.
//
// Every load has a single destination CTA (no load is broadcast to several CTAs); completion of the MMAs is
// signalled to each CTA with its own tcgen05.commit.  mbarrier waits are bounded as in the other tcgen05 kernels;
// the two cluster-wide barriers (after set-up, before TMEM release) are reached by every thread on every path.
#include "gemm.cuh"
#include "ptx_sm100.cuh"

#include <cstdlib>
#include <mutex>

namespace fmoe {

// This translation unit's status word (device code is not linked across files); read by status_word_pair().
__device__ int g_device_status_pair = 0;
// Optional wait-time profile (FMOE_TC_PROFILE=1), same columns as the single-CTA kernel's: per CTA
// {tiles, mma wait acc, mma wait data, producer wait, epilogue wait, epilogue busy, -, -}
__device__ long long g_wait_prof_pair[256 * 8];
int make_tensor_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes, int box_rows,
                       bool weights, int kbytes);
int device_sm_count();

namespace {

constexpr int BM = 128;       // rows per CTA
constexpr int PAIR_M = 256;   // rows per tile
constexpr int BN = 256;
constexpr int KBYTES = 128;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * KBYTES;        // 16 KB
constexpr int BH_BYTES = (BN / 2) * KBYTES;  // 16 KB: this CTA's half of B
constexpr int STAGE_BYTES = A_BYTES + BH_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int kThreads = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct PairParams {
  const int32_t* sorted_token_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_post_padded;
  const float* row_scale;
  void* out;
  int64_t numel;
  int64_t n;
  int64_t w_rows;
  int64_t sorted_cap;
  int32_t num_experts;
  int32_t k_steps;
  int32_t n_tiles;
  int32_t max_blocks;  // blocks of 256 rows
  int32_t activation;
  int32_t group_m;
  int32_t profile;
  int32_t debug;  // timing experiment only (results are wrong): 1 = no TMA loads, the MMA warp never waits for data
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_device_status_pair, 0, code); }
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
}

__device__ __forceinline__ bool warp_wait_relaxed(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, ptx::mbar_wait_relaxed(bar, parity));
}

template <bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                 const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES] used in CTA 0: both producers -> MMA
  uint64_t* empty_bar = bars + STAGES;            // [STAGES] per CTA: MMA -> this CTA's producer
  uint64_t* acc_full = bars + 2 * STAGES;         // [2] per CTA: MMA -> this CTA's epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;    // [2] used in CTA 0: both epilogues -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  int32_t* expert_table = reinterpret_cast<int32_t*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 2);   // one arrive.expect_tx from each CTA's producer
      ptx::mbar_init(&empty_bar[s], 1);  // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&acc_full[a], 1);
      ptx::mbar_init(&acc_empty[a], 256);  // 128 epilogue threads of each CTA
    }
    ptx::fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 5) {
    ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  const int used_blocks = min((int)(*p.num_tokens_post_padded / PAIR_M), p.max_blocks);
  const int64_t total_tiles = (int64_t)used_blocks * p.n_tiles;
  ptx::tc_fence_before_sync();
  build_expert_table(expert_table, p.num_experts, p.expert_ids, used_blocks);  // ends with __syncthreads()
  ptx::cluster_sync_all();  // the other CTA's barriers exist before anything is signalled across
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  TileCursor cursor;
  const int k_steps = p.k_steps;

  if (warp == 4) {
    // ---------------- TMA producer (both CTAs) ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    long long prof_p = 0;
    auto tile_rows = [&](int64_t tile, int32_t* row_a, int32_t* row_b) {
      int m_blk, n_tile, e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &e);
      *row_a = m_blk * PAIR_M + (int)rank * BM;
      const int64_t b0 = (int64_t)e * p.w_rows + (GATED ? (int64_t)n_tile * 128 : (int64_t)n_tile * 256);
      *row_b = (int32_t)(leader ? b0 : (GATED ? b0 + p.n : b0 + 128));
    };
    int32_t row_a = 0, row_b = 0, nrow_a = 0, nrow_b = 0;
    if ((int64_t)cluster_id < total_tiles) tile_rows(cluster_id, &row_a, &row_b);
    for (int64_t tile = cluster_id; tile < total_tiles && alive && p.debug != 1; tile += num_clusters) {
      const bool has_next = tile + num_clusters < total_tiles;
      for (int ks = 0; ks < k_steps; ++ks) {
        const long long tp0 = p.profile ? clock64() : 0;
        const bool okp = warp_wait(&empty_bar[stage], phase ^ 1);
        if (p.profile) prof_p += clock64() - tp0;
        if (!okp) {
          report(0x900 | stage);
          alive = false;
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * STAGE_BYTES;
          // the full barrier of this stage in CTA 0 collects both CTAs' bytes
          const uint32_t bar0 = ptx::smem_u32(&full_bar[stage]) & ~ptx::kPeerRankBit;
          ptx::mbar_arrive_expect_tx_cluster(bar0, STAGE_BYTES);
          const int32_t x = ks * (KBYTES / 2);
          ptx::tma_load_2d_pair(sa, &map_a, x, row_a, bar0);
          ptx::tma_load_2d_pair(sa + A_BYTES, &map_b, x, row_b, bar0);
        }
        __syncwarp();
        if (ks == 0 && has_next) tile_rows(tile + num_clusters, &nrow_a, &nrow_b);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      row_a = nrow_a;
      row_b = nrow_b;
    }
    if (p.profile && lane == 0 && blockIdx.x < 256) g_wait_prof_pair[blockIdx.x * 8 + 3] = prof_p;
    if (alive && p.debug != 1) {  // drain: every stage this CTA filled has been consumed
      for (int s = 0; s < STAGES; ++s) {
        if (!warp_wait(&empty_bar[stage], phase ^ 1)) {
          report(0x980 | stage);
          break;
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer (CTA 0 only) ----------------
    if (leader) {
      constexpr uint32_t idesc = ptx::make_idesc(/*bf16*/ 1, PAIR_M, BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool alive = true;
      long long prof_acc = 0, prof_data = 0;
      for (int64_t tile = cluster_id; tile < total_tiles && alive; tile += num_clusters) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ++local;
        const long long tm0 = p.profile ? clock64() : 0;
        const bool oka = warp_wait(&acc_empty[acc], acc_phase ^ 1);
        if (p.profile) prof_acc += clock64() - tm0;
        if (!oka) {
          report(0xA00 | acc);
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          const long long tm1 = p.profile ? clock64() : 0;
          const bool okd = p.debug == 1 ? true : warp_wait(&full_bar[stage], phase);
          if (p.profile) prof_data += clock64() - tm1;
          if (!okd) {
            report(0xA40 | stage);
            alive = false;
            break;
          }
          ptx::tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
            const uint64_t da = ptx::smem_desc_sw128(sa);
            const uint64_t db = ptx::smem_desc_sw128(sa + A_BYTES);
#pragma unroll
            for (int kk = 0; kk < KBYTES / 32; ++kk)
              ptx::mma_f16_ss_pair(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (ks | kk) != 0);
            // the stage is free in both CTAs once these MMAs have read it
            const uint32_t eb = ptx::smem_u32(&empty_bar[stage]);
            if (p.debug != 1) {
              ptx::mma_commit_pair(eb);
              ptx::mma_commit_pair(eb | ptx::kPeerRankBit);
            }
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (alive && lane == 0) {
          const uint32_t fb = ptx::smem_u32(&acc_full[acc]);
          ptx::mma_commit_pair(fb);
          ptx::mma_commit_pair(fb | ptx::kPeerRankBit);
        }
        __syncwarp();
      }
      if (p.profile && lane == 0 && blockIdx.x < 256) {
        g_wait_prof_pair[blockIdx.x * 8 + 0] = local;
        g_wait_prof_pair[blockIdx.x * 8 + 1] = prof_acc;
        g_wait_prof_pair[blockIdx.x * 8 + 2] = prof_data;
      }
    }
  } else {
    // ---------------- epilogue (warps 0-3, both CTAs, own 128 rows) ----------------
    int local = 0;
    bool alive = true;
    long long prof_wait = 0, prof_busy = 0;
    const int row = warp * 32 + lane;
    for (int64_t tile = cluster_id; tile < total_tiles && alive; tile += num_clusters) {
      int m_blk, n_tile, tile_e;
      cursor.locate(tile, p.n_tiles, p.group_m, p.num_experts, p.expert_ids, expert_table, &m_blk, &n_tile, &tile_e);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const int64_t pos = (int64_t)m_blk * PAIR_M + (int64_t)rank * BM + row;
      const int32_t slot = (pos < p.sorted_cap) ? p.sorted_token_ids[pos] : -1;
      const bool valid = slot >= 0 && slot < p.numel;
      const float rs = (valid && p.row_scale) ? p.row_scale[slot] : 1.0f;
      const long long te0 = p.profile ? clock64() : 0;
      const bool oke = warp_wait_relaxed(&acc_full[acc], acc_phase);
      const long long te1 = p.profile ? clock64() : 0;
      prof_wait += te1 - te0;
      if (!oke) {
        report(0xB00 | acc);
        alive = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(warp * 32) << 16);
      if constexpr (GATED) {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + pos * p.n + (int64_t)n_tile * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, g);
          ptx::tmem_ld_32x32b_x32(taddr + 128 + c * 32, u);
          ptx::tmem_ld_wait();
          if (pos < p.sorted_cap) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int i = v * 8 + j * 2;
                float o0 = act_mul_fast(__uint_as_float(g[i]) * rs, __uint_as_float(u[i]) * rs, p.activation);
                float o1 = act_mul_fast(__uint_as_float(g[i + 1]) * rs, __uint_as_float(u[i + 1]) * rs, p.activation);
                w[j] = pack_bf16x2(o0, o1);
              }
              dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      } else {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)(valid ? slot : 0) * p.n +
                              (int64_t)n_tile * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          if (valid && (int64_t)n_tile * 256 + c * 32 < p.n) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int i = v * 8 + j * 2;
                w[j] = pack_bf16x2(__uint_as_float(r[i]) * rs, __uint_as_float(r[i + 1]) * rs);
              }
              dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      // this thread is done with the accumulator: tell CTA 0's MMA warp
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_cluster(ptx::smem_u32(&acc_empty[acc]) & ~ptx::kPeerRankBit);
      if (p.profile) prof_busy += clock64() - te1;
    }
    if (p.profile && threadIdx.x == 0 && blockIdx.x < 256) {
      g_wait_prof_pair[blockIdx.x * 8 + 4] = prof_wait;
      g_wait_prof_pair[blockIdx.x * 8 + 5] = prof_busy;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // nobody signals into a CTA that has left, and both are done with TMEM
  if (warp == 5) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool GATED>
int launch(const GemmParams& g, cudaStream_t st) {
  static PerDeviceOnce once_attr;  // the opt-in to > 48 KB of dynamic shared memory is per device
  const cudaError_t attr_err = per_device_once(once_attr, [] {
    return cudaFuncSetAttribute(grouped_gemm_tcgen05_pair_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                SMEM_BYTES + expert_table_bytes(1024));
  });
  if (attr_err != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", SMEM_BYTES, cudaGetErrorString(attr_err));
  const int64_t w_rows = GATED ? 2 * g.n : g.n;
  CUtensorMap map_a, map_b;
  int rc = make_tensor_map_2d(&map_a, g.a, g.a_rows, g.k, 2, BM, false, 128);
  if (rc) return rc;
  rc = make_tensor_map_2d(&map_b, g.w, (int64_t)g.num_experts * w_rows, g.k, 2, 128, true, 128);
  if (rc) return rc;
  PairParams p;
  p.sorted_token_ids = g.sorted_token_ids;
  p.expert_ids = g.expert_ids;
  p.num_tokens_post_padded = g.num_tokens_post_padded;
  p.row_scale = g.row_scale;
  p.out = g.out;
  p.numel = g.numel;
  p.n = g.n;
  p.w_rows = w_rows;
  p.sorted_cap = g.sorted_cap;
  p.num_experts = g.num_experts;
  p.k_steps = (int)ceil_div<int64_t>(g.k * 2, KBYTES);
  p.n_tiles = (int)ceil_div<int64_t>(g.n, GATED ? 128 : 256);
  p.max_blocks = (int)g.max_blocks;
  p.activation = g.activation;

  const int64_t max_tiles = g.max_blocks * p.n_tiles;
  const int sms = device_sm_count();
  const int64_t pairs = std::max<int64_t>(1, std::min<int64_t>((sms > 0 ? sms : 148) / 2, max_tiles));
  p.group_m = pick_group_m(PAIR_M, g.k * 2);
  p.profile = getenv("FMOE_TC_PROFILE") != nullptr;
  p.debug = getenv("FMOE_TC_DEBUG") ? atoi(getenv("FMOE_TC_DEBUG")) : 0;
  grouped_gemm_tcgen05_pair_kernel<GATED><<<(unsigned)(2 * pairs), kThreads, SMEM_BYTES + expert_table_bytes(g.num_experts), st>>>(
      map_a, map_b, p);
  return launch_status("grouped_gemm_tcgen05_pair_kernel");
}

}  // namespace

bool gemm_tcgen05_pair_supports(const GemmParams& p, bool gated) {
  if (p.dtype != FMOE_BF16 || p.out_dtype != FMOE_BF16) return false;
  if (p.block_size != PAIR_M || p.a_gather) return false;
  if (p.bias || p.activation == FMOE_ACT_SWIGLU_OAI || p.out_rows) return false;
  if (p.k <= 0 || (p.k * 2) % 16 != 0) return false;
  if (p.n <= 0 || p.n % (gated ? 128 : 32) != 0) return false;
  if (!aligned16(p.a) || !aligned16(p.w) || !aligned16(p.out)) return false;
  if ((int64_t)p.num_experts * (gated ? 2 * p.n : p.n) >= (1ll << 31) || p.a_rows >= (1ll << 31)) return false;
  if (p.max_blocks >= (1ll << 23) || p.num_experts > 1024) return false;
  return true;
}

int read_wait_profile_pair(long long* host_out, int n) {
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(host_out, g_wait_prof_pair, sizeof(long long) * (size_t)n));
  return FMOE_OK;
}

int status_word_pair(int* out, bool clear) {
  int zero = 0;
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(out, g_device_status_pair, sizeof(int)));
  if (clear && *out != 0) FMOE_CUDA_OK(cudaMemcpyToSymbol(g_device_status_pair, &zero, sizeof(int)));
  return FMOE_OK;
}

int gemm_tcgen05_pair(const GemmParams& p, bool gated, cudaStream_t st) {
  if (!gemm_tcgen05_pair_supports(p, gated))
    return fail(FMOE_ERR_UNSUPPORTED,
                "tcgen05 pair gemm: needs bf16 in/out, block_size 256, input rows already in sorted order, "
                "n %% %d == 0, 16-byte aligned pointers",
                gated ? 128 : 32);
  if (p.max_blocks <= 0) return FMOE_OK;
  return gated ? launch<true>(p, st) : launch<false>(p, st);
}

}  // namespace fmoe
