// Plain CUDA-core grouped GEMM: one thread per output column, sequential K loop.
// It exists for fp32 inputs and as an independent on-device cross-check of the
// tensor-core kernels; it accepts every shape the ABI allows.
#include "gemm.cuh"

namespace fmoe {
namespace {

template <typename T>
struct Elem;
template <>
struct Elem<float> { static constexpr bool kScaled = false; };
template <>
struct Elem<__nv_bfloat16> { static constexpr bool kScaled = false; };
template <>
struct Elem<__nv_fp8_e4m3> { static constexpr bool kScaled = true; };

template <typename AT, bool GATED, typename OutT>
__global__ void __launch_bounds__(128)
grouped_gemm_simt_kernel(GemmParams p) {
  const int64_t b = blockIdx.y;
  const int64_t used = *p.num_tokens_post_padded;
  if (b * p.block_size >= used) return;
  const int e = p.expert_ids[b];
  if (e < 0 || e >= p.num_experts) return;
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.n) return;
  const int64_t w_rows = GATED ? 2 * p.n : p.n;  // rows of w per expert
  const AT* w = reinterpret_cast<const AT*>(p.w) + (int64_t)e * w_rows * p.k;
  const AT* wg = w + c * p.k;
  const AT* wu = GATED ? w + (p.n + c) * p.k : nullptr;
  const int64_t kblocks = ceil_div<int64_t>(p.k, 128);
  const float* swg = nullptr;
  const float* swu = nullptr;
  if constexpr (Elem<AT>::kScaled) {
    const float* sw = p.w_scale + (int64_t)e * (w_rows / 128) * kblocks;
    swg = sw + (c / 128) * kblocks;
    if (GATED) swu = sw + ((p.n + c) / 128) * kblocks;
  }
  for (int r = 0; r < p.block_size; ++r) {
    const int64_t pos = b * p.block_size + r;
    const int32_t slot = p.sorted_token_ids[pos];
    if (slot < 0 || slot >= p.numel) continue;
    const int64_t arow = p.a_gather ? slot / p.top_k : pos;
    const AT* a = reinterpret_cast<const AT*>(p.a) + arow * p.k;
    float acc_g = 0.f, acc_u = 0.f;
    for (int64_t kb = 0; kb < kblocks; ++kb) {
      float pg = 0.f, pu = 0.f;
      const int64_t k1 = min(p.k, (kb + 1) * 128);
      for (int64_t k = kb * 128; k < k1; ++k) {
        float av = to_f32(a[k]);
        pg = fmaf(av, to_f32(wg[k]), pg);
        if (GATED) pu = fmaf(av, to_f32(wu[k]), pu);
      }
      if constexpr (Elem<AT>::kScaled) {
        float sa = p.a_scale[arow * kblocks + kb];
        acc_g += pg * (sa * swg[kb]);
        if (GATED) acc_u += pu * (sa * swu[kb]);
      } else {
        acc_g += pg;
        acc_u += pu;
      }
    }
    const float rs = p.row_scale ? p.row_scale[slot] : 1.0f;
    const float* bias = p.bias ? p.bias + (int64_t)e * w_rows : nullptr;
    if constexpr (GATED) {
      reinterpret_cast<OutT*>(p.out)[pos * p.n + c] = from_f32<OutT>(gated_output<false>(
          acc_g, acc_u, bias ? bias[c] : 0.f, bias ? bias[p.n + c] : 0.f, rs, p.activation, p.act_alpha, p.act_limit));
    } else {
      reinterpret_cast<OutT*>(p.out)[(int64_t)slot * p.n + c] = from_f32<OutT>((acc_g + (bias ? bias[c] : 0.f)) * rs);
    }
  }
}

template <typename AT, bool GATED>
int launch(const GemmParams& p, cudaStream_t st) {
  if (p.max_blocks <= 0 || p.n <= 0) return FMOE_OK;
  dim3 grid((unsigned)ceil_div<int64_t>(p.n, 128), (unsigned)p.max_blocks);
  if (p.out_dtype == FMOE_F32)
    grouped_gemm_simt_kernel<AT, GATED, float><<<grid, 128, 0, st>>>(p);
  else if (p.out_dtype == FMOE_BF16)
    grouped_gemm_simt_kernel<AT, GATED, __nv_bfloat16><<<grid, 128, 0, st>>>(p);
  else
    return fail(FMOE_ERR_UNSUPPORTED, "simt gemm: out_dtype must be f32 or bf16");
  return launch_status("grouped_gemm_simt_kernel");
}

}  // namespace

int gemm_simt(const GemmParams& p, bool gated, cudaStream_t st) {
  if (p.max_blocks > 65535) return fail(FMOE_ERR_UNSUPPORTED, "simt gemm: more than 65535 blocks");
  switch (p.dtype) {
    case FMOE_F32: return gated ? launch<float, true>(p, st) : launch<float, false>(p, st);
    case FMOE_BF16: return gated ? launch<__nv_bfloat16, true>(p, st) : launch<__nv_bfloat16, false>(p, st);
    case FMOE_E4M3: return gated ? launch<__nv_fp8_e4m3, true>(p, st) : launch<__nv_fp8_e4m3, false>(p, st);
  }
  return fail(FMOE_ERR_INVALID_ARG, "simt gemm: unknown dtype %d", p.dtype);
}

}  // namespace fmoe
