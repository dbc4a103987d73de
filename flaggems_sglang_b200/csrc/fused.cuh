// Internal: workspace plan and launcher of the one-call expert computation (fused.cu).
#pragma once
#include "common.cuh"

namespace fmoe {

struct FusedPlan {
  int variant, block, act_elem;
  int64_t numel, cap, nblk, max_blocks, total;
  // byte offsets into the workspace (-1: not used)
  int64_t off_sorted, off_expert, off_npp, off_align_ws, align_ws_bytes, off_xs, off_xs_scale, off_act, off_actq, off_actq_scale, off_z;
};

int pick_variant(int dtype, int64_t numel, int E, int64_t I, int64_t H, int forced, int* variant, int* block);
int plan_fused(const fmoe_fused_args& a, FusedPlan* plan);
// Enqueues the whole computation using `ws` (at least plan.total bytes, 256-byte aligned) as scratch.
int run_fused(const fmoe_fused_args& a, const FusedPlan& plan, uint8_t* ws, void* stream);

}  // namespace fmoe
