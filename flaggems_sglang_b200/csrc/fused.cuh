// Internal: workspace plan and launcher of the one-call expert computation (fused.cu).
#pragma once
#include "common.cuh"

namespace fmoe {

struct FusedPlan {
  int variant, block, act_elem;
  int64_t numel, cap, nblk, max_blocks, total;
  // byte offsets into the workspace (-1: not used)
  int64_t off_sorted, off_expert, off_npp, off_align_ws, align_ws_bytes, off_xs, off_xs_scale, off_xt, off_xt_scale, off_act, off_actq, off_actq_scale, off_z;
  int64_t off_split, split_bytes;  // tail-split scratch of the bf16 tcgen05 GEMMs
};

// e4m3 with the tcgen05 kernels: quantise each token row once ([T,H]) and copy bytes and scales into the sorted
// order, instead of quantising every one of the T*top_k sorted rows (the quantiser is division-bound, the copy is
// not).  The scale rows must be a multiple of 16 bytes for the copy kernel.
inline bool fp8_quant_once(int64_t top_k, int64_t H) { return top_k >= 2 && H % 512 == 0; }

int pick_variant(int dtype, int64_t numel, int E, int64_t I, int64_t H, int forced, int* variant, int* block);
int plan_fused(const fmoe_fused_args& a, FusedPlan* plan);
// Enqueues the whole computation using `ws` (at least plan.total bytes, 256-byte aligned) as scratch.
int run_fused(const fmoe_fused_args& a, const FusedPlan& plan, uint8_t* ws, void* stream);

}  // namespace fmoe
