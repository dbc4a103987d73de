// fmoe_fused_experts: the whole expert computation behind one C call.  Host-side orchestration only:
// it carves the caller's workspace and enqueues the kernels of the other files on the given stream.
#include "fused.cuh"

#include <nvtx3/nvToolsExt.h>

namespace fmoe {

int pick_variant(int dtype, int64_t numel, int E, int64_t I, int64_t H, int forced, int* variant, int* block) {
  if (dtype == FMOE_F32) {
    if (forced != FMOE_VARIANT_AUTO && forced != FMOE_VARIANT_SIMT)
      return fail(FMOE_ERR_UNSUPPORTED, "fp32 inputs run on the simt kernels only");
    *variant = FMOE_VARIANT_SIMT;
    *block = 16;
    return FMOE_OK;
  }
  if (dtype != FMOE_BF16 && dtype != FMOE_E4M3) return fail(FMOE_ERR_INVALID_ARG, "unknown dtype %d", dtype);
  const int64_t active = std::max<int64_t>(1, std::min<int64_t>(E, numel));
  const double rows = (double)numel / (double)active;  // rows per active expert if routing were uniform
  // bf16: the tensor-core kernels cut their last column tile / zero-fill their last K step, the streaming kernel
  // masks its last 128-k chunk, so sizes such as 2880 (GPT-OSS) stay off the plain CUDA-core kernel
  const bool stream_ok = dtype == FMOE_BF16 ? (H % 16 == 0 && I % 16 == 0) : (H % 128 == 0 && I % 128 == 0);
  // e4m3: a tile's block scales are staged in shared memory, which bounds the reduction length at 8192
  const bool tc_ok = dtype == FMOE_BF16 ? (I % 32 == 0 && H % 32 == 0)
                                        : (I % 128 == 0 && H % 128 == 0 && I <= 8192 && H <= 8192);
  int v = forced;
  if (v == FMOE_VARIANT_AUTO) {
    // measured on B200: up to 4 rows per expert the two families tie (both stream the weights once at ~90 % of
    // HBM bandwidth) and the streaming kernel wins on tile quantisation for a handful of experts; above that the
    // 128-row tensor-core tiles win (DeepSeek-V3 T=256: 1.49 against 2.11 ms)
    if (stream_ok && (rows <= 4.0 || !tc_ok)) v = FMOE_VARIANT_STREAM;
    else if (tc_ok) v = FMOE_VARIANT_TCGEN05;
    else v = FMOE_VARIANT_SIMT;
  }
  switch (v) {
    case FMOE_VARIANT_TCGEN05:
      if (!tc_ok) return fail(FMOE_ERR_UNSUPPORTED, "tcgen05 kernels need I %% 32 == 0 and H %% 32 == 0 (e4m3: multiples of 128, up to 8192)");
      *block = 128;
      break;
    case FMOE_VARIANT_STREAM:
      if (!stream_ok) return fail(FMOE_ERR_UNSUPPORTED, "stream kernels need H and I to be multiples of 16 (128 for e4m3)");
      *block = rows <= 4.0 ? 8 : (rows <= 12.0 ? 16 : 32);
      break;
    case FMOE_VARIANT_SIMT:
      *block = 16;
      break;
    default:
      return fail(FMOE_ERR_INVALID_ARG, "unknown variant %d", forced);
  }
  *variant = v;
  return FMOE_OK;
}

namespace {
inline int64_t up256(int64_t v) { return (v + 255) & ~int64_t(255); }

// The single-CTA bf16 tcgen05 gate/up kernel can fetch its input rows by TMA gather4 instead of reading a
// sorted copy of the hidden states.  Measured on B200 the gather costs more than the copy saves (32 four-row
// TMA instructions per 16 KB stage against one tiled load: gate/up 4.07 ms against 1.67 ms at Mixtral
// T=4096, 1.03 against 0.39 ms at Qwen3 T=8192), so the copy is the default and FMOE_TC_GATHER4=1 selects
// the gather (it saves the cap x H workspace).
inline bool tc_gathers_input(int variant, int dtype) {
  static const bool gather4 = getenv("FMOE_TC_GATHER4") != nullptr;
  return variant == FMOE_VARIANT_TCGEN05 && dtype == FMOE_BF16 && gather4;
}
}

int plan_fused(const fmoe_fused_args& a, FusedPlan* pl) {
  if (a.struct_size != sizeof(fmoe_fused_args))
    return fail(FMOE_ERR_INVALID_ARG, "fused_experts: fmoe_fused_args.struct_size is %u, this library's struct has %zu "
                "bytes (binding built against another header?)", a.struct_size, sizeof(fmoe_fused_args));
  FMOE_REQUIRE(a.num_experts >= 1 && a.num_experts <= 1024 && a.top_k >= 1, "fused_experts: bad E or top_k");
  FMOE_REQUIRE(a.T >= 0 && a.H >= 1 && a.I >= 1, "fused_experts: bad sizes T=%lld H=%lld I=%lld", (long long)a.T,
               (long long)a.H, (long long)a.I);
  FMOE_REQUIRE(a.dtype == FMOE_F32 || a.dtype == FMOE_BF16 || a.dtype == FMOE_E4M3, "fused_experts: unknown dtype %d", a.dtype);
  FMOE_REQUIRE(a.activation == FMOE_ACT_SILU || a.activation == FMOE_ACT_GELU || a.activation == FMOE_ACT_SWIGLU_OAI,
               "fused_experts: unknown activation %d", a.activation);
  if (a.b1 || a.b2 || a.activation == FMOE_ACT_SWIGLU_OAI)
    FMOE_REQUIRE(a.dtype != FMOE_E4M3,
                 "fused_experts: bias and the swiglu_oai activation are not available with e4m3 weights");
  const bool channel = a.dtype == FMOE_E4M3 && a.scale_mode == FMOE_SCALE_CHANNEL;
  if (a.dtype == FMOE_E4M3) {
    FMOE_REQUIRE(a.scale_mode == FMOE_SCALE_BLOCK128 || a.scale_mode == FMOE_SCALE_CHANNEL,
                 "fused_experts: unknown scale_mode %d", a.scale_mode);
    if (channel) {
      FMOE_REQUIRE(a.H % 32 == 0 && a.I % 32 == 0 && a.H <= 16384 && a.I <= 16384,
                   "fused_experts: per-channel e4m3 needs H and I to be multiples of 32, up to 16384");
      if (a.variant != FMOE_VARIANT_AUTO && a.variant != FMOE_VARIANT_TCGEN05)
        return fail(FMOE_ERR_UNSUPPORTED, "fused_experts: per-channel e4m3 runs on the TCGEN05 kernels only");
    } else {
      FMOE_REQUIRE(a.H % 128 == 0 && a.I % 128 == 0, "fused_experts: e4m3 needs H and I to be multiples of 128");
    }
  }
  FMOE_REQUIRE(a.w_layout == FMOE_W_K_MAJOR || a.w_layout == FMOE_W_N_MAJOR, "fused_experts: unknown w_layout %d", a.w_layout);
  const bool n_major = a.w_layout == FMOE_W_N_MAJOR;
  if (n_major && (a.dtype != FMOE_BF16 || a.b1 || a.b2 || a.activation == FMOE_ACT_SWIGLU_OAI ||
                  (a.variant != FMOE_VARIANT_AUTO && a.variant != FMOE_VARIANT_TCGEN05)))
    return fail(FMOE_ERR_UNSUPPORTED, "fused_experts: [E,H,2I] / [E,I,H] weights (FMOE_W_N_MAJOR) need bf16, the TCGEN05 "
                "kernels, no bias and no swiglu_oai");
  FusedPlan& p = *pl;
  p.numel = a.T * a.top_k;
  int rc = FMOE_OK;
  if (channel) {  // one kernel family: bf16-style tcgen05 pipeline on e4m3 operands, 128-row blocks
    p.variant = FMOE_VARIANT_TCGEN05;
    p.block = 128;
  } else {
    rc = pick_variant(a.dtype, p.numel, a.num_experts, a.I, a.H, n_major ? FMOE_VARIANT_TCGEN05 : a.variant, &p.variant,
                      &p.block);
  }
  if (rc) return rc;
  p.cap = p.numel + (int64_t)a.num_experts * (p.block - 1);
  p.nblk = ceil_div<int64_t>(p.cap, p.block);
  p.max_blocks = std::min<int64_t>(p.cap / p.block, p.numel);
  const int64_t eb = a.dtype == FMOE_F32 ? 4 : 2;  // element size of hidden / out / z
  const bool fp8 = a.dtype == FMOE_E4M3;
  const bool tc = p.variant == FMOE_VARIANT_TCGEN05;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    int64_t o = off;
    off += up256(bytes);
    return o;
  };
  p.off_sorted = take(p.cap * 4);
  p.off_expert = take(p.nblk * 4);
  p.off_npp = take(16);
  p.align_ws_bytes = fmoe_moe_align_workspace_bytes(p.numel, a.num_experts);
  p.off_align_ws = take(p.align_ws_bytes);
  p.off_xs = p.off_xs_scale = p.off_xt = p.off_xt_scale = p.off_actq = p.off_actq_scale = p.off_split = -1;
  p.split_bytes = 0;
  if (channel) {
    // every sorted row is quantised with its own scale; the activation likewise
    p.off_xs = take(p.cap * a.H);
    p.off_xs_scale = take(p.cap * 4);
    if (a.top_k >= 2 && a.H % 16 == 0) {  // each token row quantised once, its bytes copied into the sorted order
      p.off_xt = take(a.T * a.H);
      p.off_xt_scale = take(a.T * 4);
    }
    p.act_elem = 2;
    p.off_act = take(p.cap * a.I * 2);
    p.off_actq = take(p.cap * a.I);
    p.off_actq_scale = take(p.cap * 4);
    p.split_bytes = fmoe_gemm_split_workspace_bytes();
    p.off_split = take(p.split_bytes);
  } else if (fp8) {
    const int64_t xrows = tc ? p.cap : a.T;
    p.off_xs = take(xrows * a.H);
    p.off_xs_scale = take(xrows * (a.H / 128) * 4);
    if (tc && fp8_quant_once(a.top_k, a.H)) {
      p.off_xt = take(a.T * a.H);
      p.off_xt_scale = take(a.T * (a.H / 128) * 4);
    }
    p.act_elem = tc ? 2 : 4;  // bf16 from the tcgen05 epilogue, fp32 from the streaming kernel
    p.off_act = take(p.cap * a.I * p.act_elem);
    p.off_actq = take(p.cap * a.I);
    p.off_actq_scale = take(p.cap * (a.I / 128) * 4);
  } else {
    if (tc && !(tc_gathers_input(p.variant, a.dtype) && !n_major)) p.off_xs = take(p.cap * a.H * eb);
    if (tc && a.dtype == FMOE_BF16) {
      p.split_bytes = fmoe_gemm_split_workspace_bytes();
      p.off_split = take(p.split_bytes);
    }
    p.act_elem = (int)eb;
    p.off_act = take(p.cap * a.I * eb);
  }
  p.off_z = a.no_combine ? -1 : take(p.numel * a.H * eb);
  p.total = off;
  return FMOE_OK;
}

namespace {
// Optional per-stage timing (fmoe_debug_stage_events): events of the calling thread's NEXT fused call.
thread_local void* const* t_stage_events = nullptr;
thread_local int t_stage_count = 0;

// NVTX range per stage of the layer (header-only NVTX 3: a no-op branch unless a profiler is attached).  The range that
// is open when the function returns, on an error too, is closed by the destructor.
struct StageRange {
  bool open = false;
  void next(const char* name) {
    if (open) nvtxRangePop();
    nvtxRangePushA(name);
    open = true;
  }
  ~StageRange() {
    if (open) nvtxRangePop();
  }
};
const char* const kStageNames[7] = {"fmoe.align",       "fmoe.gather_quant", "fmoe.gemm1_act", "fmoe.act_quant",
                                    "fmoe.gemm2",       "fmoe.moe_sum",      "fmoe.done"};
}  // namespace

int run_fused(const fmoe_fused_args& a, const FusedPlan& p, uint8_t* ws, void* stream) {
  void* const* stage_ev = t_stage_events;
  const int stage_n = t_stage_count;
  t_stage_events = nullptr;
  t_stage_count = 0;
  StageRange range;
  auto mark = [&](int i) {
    if (stage_ev && i < stage_n && stage_ev[i]) cudaEventRecord((cudaEvent_t)stage_ev[i], (cudaStream_t)stream);
    if (i < 6) range.next(kStageNames[i]);
  };
  if (a.T == 0) return FMOE_OK;
  FMOE_REQUIRE(a.hidden && a.w1 && a.w2 && a.topk_weights && a.topk_ids && (a.out || a.out_rows), "fused_experts: null pointer");
  if (a.out_rows) {
    FMOE_REQUIRE(a.no_combine && !a.zero_dropped, "fused_experts: out_rows needs no_combine = 1 and zero_dropped = 0");
    if (p.variant != FMOE_VARIANT_STREAM && p.variant != FMOE_VARIANT_TCGEN05)
      return fail(FMOE_ERR_UNSUPPORTED, "fused_experts: out_rows is taken by the STREAM and TCGEN05 kernels only");
  }
  const bool fp8 = a.dtype == FMOE_E4M3;
  const bool tc = p.variant == FMOE_VARIANT_TCGEN05;
  if (fp8) FMOE_REQUIRE(a.w1_scale && a.w2_scale, "fused_experts: e4m3 needs w1_scale and w2_scale");
  const int io = fp8 ? FMOE_BF16 : a.dtype;  // dtype of hidden / z / out
  const int64_t eb = io == FMOE_F32 ? 4 : 2;
  int32_t* sorted = reinterpret_cast<int32_t*>(ws + p.off_sorted);
  int32_t* experts = reinterpret_cast<int32_t*>(ws + p.off_expert);
  int32_t* npp = reinterpret_cast<int32_t*>(ws + p.off_npp);
  void* act = ws + p.off_act;
  void* z = a.no_combine ? a.out : (void*)(ws + p.off_z);
  auto st = (cudaStream_t)stream;

  mark(0);
  int rc = fmoe_moe_align_block_size_ws(a.topk_ids, p.numel, a.num_experts, p.block, sorted, p.cap, experts, p.nblk, npp,
                                        ws + p.off_align_ws, p.align_ws_bytes, stream);
  if (rc) return rc;
  mark(1);
  if (a.zero_dropped) FMOE_CUDA_OK(cudaMemsetAsync(z, 0, (size_t)(p.numel * a.H * eb), st));

  fmoe_gemm_args g{};
  g.struct_size = (uint32_t)sizeof(fmoe_gemm_args);
  g.w_layout = a.w_layout;
  g.variant = p.variant;
  g.num_experts = a.num_experts;
  g.top_k = a.top_k;
  g.block_size = p.block;
  g.numel = p.numel;
  g.sorted_cap = p.cap;
  g.max_blocks = p.max_blocks;
  g.sorted_token_ids = sorted;
  g.expert_ids = experts;
  g.num_tokens_post_padded = npp;

  if (p.off_split >= 0) {  // both GEMMs use it in turn (stream order)
    g.split_ws = ws + p.off_split;
    g.split_ws_bytes = p.split_bytes;
  }
  fmoe_gemm_args g1 = g, g2 = g;
  g1.n = a.I;
  g1.activation = a.activation;
  g1.act_alpha = a.act_alpha;
  g1.act_limit = a.act_limit;
  g1.bias = a.b1;
  g2.bias = a.b2;
  g1.k = a.H;
  g1.w = a.w1;
  g1.out = act;
  g1.row_scale = a.apply_router_weight_on_input ? a.topk_weights : nullptr;
  g2.n = a.H;
  g2.k = a.I;
  g2.w = a.w2;
  g2.out = z;
  g2.out_rows = a.out_rows;
  g2.a_gather = 0;
  g2.a_rows = p.cap;
  g2.row_scale = a.apply_router_weight_on_input ? nullptr : a.topk_weights;
  g2.out_dtype = io;

  if (!fp8) {
    g1.dtype = g1.out_dtype = g2.dtype = a.dtype;
    if (tc && p.off_xs >= 0) {
      void* xs = ws + p.off_xs;
      rc = fmoe_gather_rows(a.hidden, (int)eb, p.cap, a.H, sorted, a.top_k, p.numel, npp, xs, stream);
      if (rc) return rc;
      g1.a = xs;
      g1.a_rows = p.cap;
      g1.a_gather = 0;
    } else {
      g1.a = a.hidden;
      g1.a_rows = a.T;
      g1.a_gather = 1;
    }
    g2.a = act;
  } else {
    void* xq = ws + p.off_xs;
    float* xsc = reinterpret_cast<float*>(ws + p.off_xs_scale);
    const bool channel = a.scale_mode == FMOE_SCALE_CHANNEL;
    g1.scale_mode = g2.scale_mode = a.scale_mode;
    if (channel && p.off_xt >= 0) {
      void* xt = ws + p.off_xt;
      float* xtsc = reinterpret_cast<float*>(ws + p.off_xt_scale);
      rc = fmoe_quant_fp8_per_token(a.hidden, FMOE_BF16, a.T, a.H, nullptr, 1, 0, nullptr, xt, xtsc, stream);
      if (rc) return rc;
      rc = fmoe_gather_rows(xt, 1, p.cap, a.H, sorted, a.top_k, p.numel, npp, xq, stream);
      xsc = xtsc;  // the gate/up GEMM looks the scale up by token
      g1.a_scale_gather = 1;
    } else if (channel) {
      rc = fmoe_quant_fp8_per_token(a.hidden, FMOE_BF16, p.cap, a.H, sorted, a.top_k, p.numel, npp, xq, xsc, stream);
    } else if (tc && p.off_xt >= 0) {
      void* xt = ws + p.off_xt;
      float* xtsc = reinterpret_cast<float*>(ws + p.off_xt_scale);
      rc = fmoe_quant_fp8_group128(a.hidden, FMOE_BF16, a.T, a.H, nullptr, 1, 0, nullptr, xt, xtsc, stream);
      if (rc) return rc;
      rc = fmoe_gather_rows(xt, 1, p.cap, a.H, sorted, a.top_k, p.numel, npp, xq, stream);
      if (rc) return rc;
      rc = fmoe_gather_rows(xtsc, 4, p.cap, a.H / 128, sorted, a.top_k, p.numel, npp, xsc, stream);
    } else if (tc)
      rc = fmoe_quant_fp8_group128(a.hidden, FMOE_BF16, p.cap, a.H, sorted, a.top_k, p.numel, npp, xq, xsc, stream);
    else
      rc = fmoe_quant_fp8_group128(a.hidden, FMOE_BF16, a.T, a.H, nullptr, 1, 0, nullptr, xq, xsc, stream);
    if (rc) return rc;
    g1.dtype = g2.dtype = FMOE_E4M3;
    g1.out_dtype = p.act_elem == 2 ? FMOE_BF16 : FMOE_F32;
    g1.a = xq;
    g1.a_scale = xsc;
    g1.a_rows = tc ? p.cap : a.T;
    g1.a_gather = tc ? 0 : 1;
    g1.w_scale = a.w1_scale;
    g2.a = ws + p.off_actq;
    g2.a_scale = reinterpret_cast<float*>(ws + p.off_actq_scale);
    g2.w_scale = a.w2_scale;
  }
  mark(2);
  rc = fmoe_gemm1_silu(&g1, stream);
  if (rc) return rc;
  mark(3);
  if (fp8) {
    // padding positions of the sorted order (most of the rows at small T) are zero-filled, not quantised
    if (a.scale_mode == FMOE_SCALE_CHANNEL)
      rc = fmoe_quant_fp8_per_token(act, FMOE_BF16, p.cap, a.I, sorted, 0, p.numel, npp, ws + p.off_actq,
                                    reinterpret_cast<float*>(ws + p.off_actq_scale), stream);
    else
      rc = fmoe_quant_fp8_group128(act, g1.out_dtype, p.cap, a.I, sorted, 0, p.numel, npp, ws + p.off_actq,
                                   reinterpret_cast<float*>(ws + p.off_actq_scale), stream);
    if (rc) return rc;
  }
  mark(4);
  rc = fmoe_gemm2(&g2, stream);
  if (rc) return rc;
  mark(5);
  if (a.no_combine) return FMOE_OK;
  rc = fmoe_moe_sum(z, io, a.T, a.top_k, a.H, a.routed_scaling_factor == 0.f ? 1.0f : a.routed_scaling_factor, a.out, stream);
  mark(6);
  return rc;
}

}  // namespace fmoe

extern "C" int fmoe_pick_variant(int dtype, int64_t numel, int E, int64_t I, int64_t H, int forced_variant,
                                 int* variant_out, int* block_out) {
  if (!variant_out || !block_out) return fmoe::fail(FMOE_ERR_INVALID_ARG, "pick_variant: null output pointer");
  return fmoe::pick_variant(dtype, numel, E, I, H, forced_variant, variant_out, block_out);
}

extern "C" int fmoe_debug_stage_events(void* const* events, int n) {
  if (n < 0 || n > FMOE_STAGE_EVENTS || (n > 0 && !events))
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "stage events: need 0 <= n <= %d and a non-null array", FMOE_STAGE_EVENTS);
  fmoe::t_stage_events = n ? events : nullptr;
  fmoe::t_stage_count = n;
  return FMOE_OK;
}

extern "C" int64_t fmoe_fused_experts_workspace_bytes(const fmoe_fused_args* args) {
  if (!args) {
    fmoe::fail(FMOE_ERR_INVALID_ARG, "fused_experts: args is null");
    return -1;
  }
  fmoe::FusedPlan p;
  if (fmoe::plan_fused(*args, &p)) return -1;
  return p.total;
}

extern "C" int fmoe_fused_experts(const fmoe_fused_args* args, void* stream) {
  using namespace fmoe;
  if (!args) return fail(FMOE_ERR_INVALID_ARG, "fused_experts: args is null");
  FusedPlan p;
  int rc = plan_fused(*args, &p);
  if (rc) return rc;
  if (args->T == 0) return FMOE_OK;
  FMOE_REQUIRE(args->workspace && (reinterpret_cast<uintptr_t>(args->workspace) & 255u) == 0,
               "fused_experts: workspace must be non-null and 256-byte aligned");
  FMOE_REQUIRE(args->workspace_bytes >= p.total, "fused_experts: workspace too small (%lld < %lld bytes)",
               (long long)args->workspace_bytes, (long long)p.total);
  return run_fused(*args, p, reinterpret_cast<uint8_t*>(args->workspace), stream);
}
