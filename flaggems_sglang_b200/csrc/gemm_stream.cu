// Small-M grouped GEMM: the weights are streamed from HBM exactly once per token
// block, straight from global memory into mma.sync fragments (no shared-memory
// staging), with 16-byte loads that cover whole 64-byte row segments per quad.
//
// Orientation is swapped: a 16-row slab of W is the A operand (m16), a group of
// 8 tokens is the B operand (n8).  Since the reduction index may be permuted
// freely as long as both operands agree, lane (g = lane/4, t = lane%4) loads the
// 16 contiguous bytes at k-offset 16*t of its row and feeds them to two
// consecutive MMAs; both operands use the same byte -> k assignment.
//
// One work item = one token block (8*NTG rows of one expert) x one slab pair of W rows.
// By default one warp owns an item over the whole K range; when a launch has too few
// items to fill the GPU, 2/4/8 warps of a CTA share an item, split K in chunks of 128 and
// are reduced through shared memory in a fixed order (bit-reproducible).  gemm1 pairs 16
// gate rows with the matching 16 up rows so that silu(gate)*up is applied in registers.
#include <cstdlib>

#include "gemm.cuh"

namespace fmoe {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int RT = 2;  // 16-row slabs of W per CTA

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// EB: bytes per element (2 = bf16, 1 = e4m3 with 128-block scales)
// A work item is (token block b, slab pair s); W = 1, 2, 4 or 8 warps share an item and split its K
// range (interleaved 128-k chunks).  W is chosen by the host so that the launch has enough warps to
// keep HBM busy; with W == 1 a warp owns its item end to end and the CTA never synchronises.
// CTAs per SM the register allocation must allow: the kernel hides HBM latency with resident warps
constexpr int min_ctas(int eb, int ntg) { return (ntg == 1 || (ntg == 2 && eb == 2)) ? 2 : 1; }

// RAGGED (bf16 only): K is not a multiple of 128, the loads of the last chunk that fall past the row read as zero.
// A separate instantiation, so that the predicates never touch the load schedule of the common case.
template <int EB, int NTG, bool GATED, typename OutT, bool RAGGED>
__global__ void __launch_bounds__(kThreads, min_ctas(EB, NTG))
grouped_gemm_stream_kernel(GemmParams p, int W, int n_slabs) {
  pdl_entry();
  constexpr int BM = 8 * NTG;
  constexpr int U = (EB == 2) ? 4 : 2;      // 64-byte steps per 128-k chunk
  constexpr int FRAG = RT * NTG * 4 * 32;   // accumulator words per warp
  extern __shared__ float s_red[];          // [kWarps][FRAG], only when W > 1

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int items_per_cta = kWarps / W;
  const int64_t item = (int64_t)blockIdx.x * items_per_cta + warp / W;
  const int part = warp % W;
  const int64_t b = item / n_slabs;
  const int slab = (int)(item % n_slabs);
  bool active = b < p.max_blocks && b * BM < (int64_t)*p.num_tokens_post_padded;
  int e = active ? p.expert_ids[b] : -1;
  active = active && e >= 0 && e < p.num_experts;
  if (W == 1 && !active) return;  // no barrier is ever reached on this path

  const int64_t K = p.k;
  const int64_t w_rows = GATED ? 2 * p.n : p.n;
  const int64_t n0 = (int64_t)slab * (GATED ? 16 : 32);
  const int64_t kblocks = (K + 127) / 128;  // bf16: the last chunk may be partial (its loads past K read as zero)
  const int64_t row_bytes = K * EB;

  float acc[RT][NTG][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int q = 0; q < NTG; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rt][q][i] = 0.f;

  // flat slots of the tokens this lane touches: token g of each group feeds the B fragment,
  // tokens 2t and 2t+1 are the accumulator columns (scales, epilogue)
  int32_t slot_t[NTG][2];
#pragma unroll
  for (int q = 0; q < NTG; ++q) slot_t[q][0] = slot_t[q][1] = -1;

  if (active) {
    // W row of this lane for slab rt, half h (fragment rows g and g+8); clamped so loads stay in bounds
    const uint8_t* wptr[RT][2];
    int64_t slab_row0[RT];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
      slab_row0[rt] = GATED ? (rt == 0 ? n0 : p.n + n0) : n0 + 16 * rt;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        int64_t row = min(slab_row0[rt] + g + 8 * h, w_rows - 1);
        wptr[rt][h] = reinterpret_cast<const uint8_t*>(p.w) + (((int64_t)e * w_rows + row) * K) * EB + t * 16;
      }
    }
    const uint8_t* xptr[NTG];
    const float* sa_ptr[NTG][2];
#pragma unroll
    for (int q = 0; q < NTG; ++q) {
      const int64_t pos_g = b * BM + q * 8 + g;
      const int32_t sg = p.sorted_token_ids[pos_g];
      const bool okg = sg >= 0 && sg < p.numel;
      const int64_t ar = okg ? (p.a_gather ? (int64_t)(sg / p.top_k) : pos_g) : -1;
      xptr[q] = ar >= 0 ? reinterpret_cast<const uint8_t*>(p.a) + ar * K * EB + t * 16 : nullptr;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int64_t pos_t = b * BM + q * 8 + 2 * t + j;
        const int32_t st = p.sorted_token_ids[pos_t];
        const bool okt = st >= 0 && st < p.numel;
        slot_t[q][j] = okt ? st : -1;
        if constexpr (EB == 1) {
          const int64_t art = okt ? (p.a_gather ? (int64_t)(st / p.top_k) : pos_t) : -1;
          sa_ptr[q][j] = art >= 0 ? p.a_scale + art * kblocks : nullptr;
        }
      }
    }
    const float* sw_ptr[RT];
    if constexpr (EB == 1) {
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
        sw_ptr[rt] = p.w_scale + ((int64_t)e * (w_rows / 128) + min(slab_row0[rt], w_rows - 1) / 128) * kblocks;
    }

    // The W fragments of a chunk live in registers; as soon as the MMAs of one 64-byte step have consumed
    // theirs, the same registers are reloaded with that step of the warp's NEXT chunk, so loads stay in
    // flight while the rest of the chunk is computed (a warp that loaded a whole chunk, waited and then
    // computed kept HBM busy only half of the time).  The block scales of the next chunk travel the same way.
    uint4 wq[RT][U][2];
    float sw_c[RT], sa_c[NTG][2];
    // wptr walks one chunk ahead of xptr: it always points at the chunk whose fragments are loaded next
    const int64_t step = (int64_t)W * 128 * EB;
    // byte offset, inside a row, of the chunk the W pointers / the x pointers stand at (bounds of a partial last chunk)
    int64_t w_off = (int64_t)part * 128 * EB + t * 16, x_off = w_off;
    constexpr bool ragged = RAGGED;
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int h = 0; h < 2; ++h) wptr[rt][h] += (int64_t)part * 128 * EB;
#pragma unroll
    for (int q = 0; q < NTG; ++q)
      if (xptr[q]) xptr[q] += (int64_t)part * 128 * EB;
    auto load_w_step = [&](int u) {
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          wq[rt][u][h] = (!ragged || w_off + u * 64 < row_bytes) ? ldg_stream_v4(wptr[rt][h] + u * 64) : make_uint4(0, 0, 0, 0);
    };
    auto load_scales = [&](int64_t chunk) {
      if constexpr (EB == 1) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) sw_c[rt] = sw_ptr[rt][chunk];
#pragma unroll
        for (int q = 0; q < NTG; ++q)
#pragma unroll
          for (int j = 0; j < 2; ++j) sa_c[q][j] = sa_ptr[q][j] ? sa_ptr[q][j][chunk] : 0.f;
      }
    };
    auto bump_w = [&]() {
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int h = 0; h < 2; ++h) wptr[rt][h] += step;
      w_off += step;
    };
    if (part < kblocks) {
#pragma unroll
      for (int u = 0; u < U; ++u) load_w_step(u);
      load_scales(part);
      bump_w();
    }
#pragma unroll 1
    for (int64_t chunk = part; chunk < kblocks; chunk += W) {
      const bool has_next = chunk + W < kblocks;
      float part_acc[RT][NTG][4];
      if constexpr (EB == 1) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
          for (int q = 0; q < NTG; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) part_acc[rt][q][i] = 0.f;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int q = 0; q < NTG; ++q) {
          uint4 xq = (xptr[q] && (!ragged || x_off + u * 64 < row_bytes)) ? ldg_cached_v4(xptr[q] + u * 64)
                                                                            : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            if constexpr (EB == 2) {
              mma_bf16_16816(acc[rt][q], wq[rt][u][0].x, wq[rt][u][1].x, wq[rt][u][0].y, wq[rt][u][1].y, xq.x, xq.y);
              mma_bf16_16816(acc[rt][q], wq[rt][u][0].z, wq[rt][u][1].z, wq[rt][u][0].w, wq[rt][u][1].w, xq.z, xq.w);
            } else {
              mma_e4m3_16832(part_acc[rt][q], wq[rt][u][0].x, wq[rt][u][1].x, wq[rt][u][0].y, wq[rt][u][1].y, xq.x, xq.y);
              mma_e4m3_16832(part_acc[rt][q], wq[rt][u][0].z, wq[rt][u][1].z, wq[rt][u][0].w, wq[rt][u][1].w, xq.z, xq.w);
            }
          }
        }
        if (has_next) load_w_step(u);
      }
      bump_w();
#pragma unroll
      for (int q = 0; q < NTG; ++q)
        if (xptr[q]) xptr[q] += step;
      x_off += step;
      if constexpr (EB == 1) {
        // acc += partial * (activation scale of the token) * (weight scale of the slab) for this 128-k block
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
          for (int q = 0; q < NTG; ++q) {
            const float s0 = sa_c[q][0] * sw_c[rt];
            const float s1 = sa_c[q][1] * sw_c[rt];
            acc[rt][q][0] = fmaf(part_acc[rt][q][0], s0, acc[rt][q][0]);
            acc[rt][q][1] = fmaf(part_acc[rt][q][1], s1, acc[rt][q][1]);
            acc[rt][q][2] = fmaf(part_acc[rt][q][2], s0, acc[rt][q][2]);
            acc[rt][q][3] = fmaf(part_acc[rt][q][3], s1, acc[rt][q][3]);
          }
        }
        if (has_next) load_scales(chunk + W);
      }
    }
  }

  if (W > 1) {
    // fixed-order reduction over the W warps of the item (bit-reproducible)
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int q = 0; q < NTG; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) s_red[warp * FRAG + ((rt * NTG + q) * 4 + i) * 32 + lane] = acc[rt][q][i];
    __syncthreads();
    if (part != 0 || !active) return;
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int q = 0; q < NTG; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float s = 0.f;
          for (int w = 0; w < W; ++w) s += s_red[(warp + w) * FRAG + ((rt * NTG + q) * 4 + i) * 32 + lane];
          acc[rt][q][i] = s;
        }
  }

  // epilogue from registers.  Accumulator word i of lane (g,t): W row g + 8*(i>>1) of the slab, token 2t + (i&1).
  OutT* out = reinterpret_cast<OutT*>(p.out);
#pragma unroll
  for (int q = 0; q < NTG; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int32_t slot = slot_t[q][i & 1];
      if (slot < 0) continue;
      const float rs = p.row_scale ? p.row_scale[slot] : 1.0f;
      const int col = g + 8 * (i >> 1);
      const float* bias = p.bias ? p.bias + (int64_t)e * w_rows : nullptr;
      if constexpr (GATED) {
        if (n0 + col < p.n)
          out[(b * BM + q * 8 + 2 * t + (i & 1)) * p.n + n0 + col] = from_f32<OutT>(gated_output<false>(
              acc[0][q][i], acc[1][q][i], bias ? bias[n0 + col] : 0.f, bias ? bias[p.n + n0 + col] : 0.f, rs,
              p.activation, p.act_alpha, p.act_limit));
      } else {
        OutT* orow = p.out_rows ? reinterpret_cast<OutT*>(p.out_rows[slot]) : out + (int64_t)slot * p.n;
        if (!orow) continue;
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
          if (n0 + rt * 16 + col < p.n)
            orow[n0 + rt * 16 + col] = from_f32<OutT>((acc[rt][q][i] + (bias ? bias[n0 + rt * 16 + col] : 0.f)) * rs);
      }
    }
  if (p.out_rows) __threadfence_system();  // rows stored to a peer are complete before the kernel ends
}

// Warps per item: enough warps in flight to cover HBM latency, but at least two 128-k chunks per warp.
int pick_ksplit(int64_t items, int64_t kblocks, int elem_bytes) {
  // FMOE_STREAM_W=1|2|4|8 forces the split (tuning aid)
  if (const char* env = getenv("FMOE_STREAM_W")) {
    int w = atoi(env);
    if (w == 1 || w == 2 || w == 4 || w == 8) return w;
  }
  // Measured on B200: with 2-byte elements a warp touches 256 contiguous bytes of a row per step and, for long
  // reductions (Mixtral: 32 and 112 chunks of 128), HBM streams best when the warps of a CTA walk one row range
  // together (W = 8 gives 2 KB runs).  For short reductions (Qwen3 2048 / 768, the reference's test shape 1280 /
  // 3072) an 8-way split leaves a warp two chunks and a reduction: W = 2 measured 0.224 -> 0.196 ms at Qwen3 T=32 and
  // 0.272 -> 0.222 ms at the reference shape T=17; the work-item rule below raises it when a launch has few items
  // (T=1: W = 4).  With 1-byte elements W = 1 measured fastest at every size tried (also with 256-byte chunks).
  int W = 1;
  if (elem_bytes == 2) W = kblocks >= 32 ? 8 : (kblocks >= 4 ? 2 : 1);
  const int64_t target = 148 * 16;
  while (W < kWarps && items * W < target && kblocks / (2 * W) >= 2) W *= 2;
  return W;
}

template <int EB, int NTG, bool GATED>
int launch(const GemmParams& p, cudaStream_t st) {
  const int n_slabs = (int)ceil_div<int64_t>(p.n, GATED ? 16 : 32);
  const int64_t items = p.max_blocks * n_slabs;
  const int W = pick_ksplit(items, (p.k + 127) / 128, EB);
  const int64_t ctas = ceil_div<int64_t>(items, kWarps / W);
  if (ctas >= (1ll << 31)) return fail(FMOE_ERR_UNSUPPORTED, "stream gemm: too many work items");
  const size_t smem = W > 1 ? sizeof(float) * kWarps * RT * NTG * 4 * 32 : 0;
  dim3 grid((unsigned)ctas);
  const bool ragged = EB == 2 && (p.k % 128) != 0;
  if constexpr (EB == 2) {
    if (ragged) {
      if (p.out_dtype == FMOE_F32)
        launch_pdl(grouped_gemm_stream_kernel<EB, NTG, GATED, float, true>, grid, dim3(kThreads), smem, st, p, W, n_slabs);
      else
        launch_pdl(grouped_gemm_stream_kernel<EB, NTG, GATED, __nv_bfloat16, true>, grid, dim3(kThreads), smem, st, p, W, n_slabs);
      return launch_status("grouped_gemm_stream_kernel");
    }
  }
  if (p.out_dtype == FMOE_F32)
    launch_pdl(grouped_gemm_stream_kernel<EB, NTG, GATED, float, false>, grid, dim3(kThreads), smem, st, p, W, n_slabs);
  else
    launch_pdl(grouped_gemm_stream_kernel<EB, NTG, GATED, __nv_bfloat16, false>, grid, dim3(kThreads), smem, st, p, W, n_slabs);
  return launch_status("grouped_gemm_stream_kernel");
}

template <int EB, bool GATED>
int launch_ntg(const GemmParams& p, cudaStream_t st) {
  switch (p.block_size) {
    case 8: return launch<EB, 1, GATED>(p, st);
    case 16: return launch<EB, 2, GATED>(p, st);
    case 32: return launch<EB, 4, GATED>(p, st);
  }
  return fail(FMOE_ERR_UNSUPPORTED, "stream gemm: block_size must be 8, 16 or 32 (got %d)", p.block_size);
}

}  // namespace

bool gemm_stream_supports(const GemmParams& p, bool gated) {
  if (p.dtype != FMOE_BF16 && p.dtype != FMOE_E4M3) return false;
  if (p.out_dtype != FMOE_BF16 && p.out_dtype != FMOE_F32) return false;
  if (p.block_size != 8 && p.block_size != 16 && p.block_size != 32) return false;
  if (p.k <= 0 || (p.dtype == FMOE_E4M3 ? p.k % 128 != 0 : p.k % 8 != 0)) return false;  // 16-byte loads; e4m3: scale blocks
  if (p.n <= 0 || p.n % 16 != 0) return false;
  if (gated && p.dtype == FMOE_E4M3 && p.n % 128 != 0) return false;  // up rows must start on a scale block
  if (!aligned16(p.a) || !aligned16(p.w)) return false;
  return true;
}

int gemm_stream(const GemmParams& p, bool gated, cudaStream_t st) {
  if (!gemm_stream_supports(p, gated))
    return fail(FMOE_ERR_UNSUPPORTED,
                "stream gemm: needs bf16/e4m3 inputs, k %% 8 == 0 (e4m3: 128), n %% 16 == 0, block_size in {8,16,32}, "
                "16-byte aligned a and w (got dtype=%d k=%lld n=%lld block=%d)",
                p.dtype, (long long)p.k, (long long)p.n, p.block_size);
  if (p.max_blocks <= 0) return FMOE_OK;
  if (p.dtype == FMOE_BF16) return gated ? launch_ntg<2, true>(p, st) : launch_ntg<2, false>(p, st);
  return gated ? launch_ntg<1, true>(p, st) : launch_ntg<1, false>(p, st);
}

}  // namespace fmoe
