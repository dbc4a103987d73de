/*
 * fmoe_b200 — C ABI of the B200 (sm_100a) fused-MoE kernels.
 *
 * The reference project (FlagGems-sglang) has no native boundary: its operator
 * is a Python function that launches Triton kernels.  Each entry point below
 * names the reference interface (file:line inside that project) whose work it
 * takes over, so a maintainer can bind it from the Python operator with ctypes.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; the caller owns
 *     all memory, and the compute entry points never allocate or free (workspaces are
 *     passed in); only fmoe_ep_buffer_create / _destroy allocate, at set-up time;
 *   - every function returns FMOE_OK (0) or an FMOE_ERR_* code; a human-readable
 *     message for the calling thread's last failure is at fmoe_last_error();
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, not awaited;
 *   - nothing here falls back to the CPU: without a CUDA device every compute
 *     entry point returns FMOE_ERR_CUDA.
 */
#ifndef FMOE_B200_H
#define FMOE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMOE_OK 0
#define FMOE_ERR_INVALID_ARG 1
#define FMOE_ERR_CUDA 2
#define FMOE_ERR_UNSUPPORTED 3
#define FMOE_ERR_DEVICE_TIMEOUT 4

/* element types of activations / weights */
#define FMOE_F32 0
#define FMOE_BF16 1
#define FMOE_E4M3 2

/* gated activation applied by gemm1 (g = gate accumulator, u = up accumulator, both after the optional bias) */
#define FMOE_ACT_SILU 0        /* silu(g*rs) * (u*rs): the row scale goes in first, as in the reference's gemm1 + silu pass */
#define FMOE_ACT_GELU 1        /* gelu(g*rs) * (u*rs) */
#define FMOE_ACT_SWIGLU_OAI 2  /* g' = min(g, limit), u' = clamp(u, -limit, limit) (limit > 0 only),
                                  s = g' / (1 + exp(-alpha*g')), out = (s*u' + s) * rs: the swiglu of the bias variant
                                  (src/flaggems_sglang/ops/fused_moe.py:235-325, third-party triton_kernels.swiglu);
                                  bias, activation, then row scale, the order of that path's GEMM epilogue */

/* grouped-GEMM kernel families (fmoe_gemm_args.variant) */
#define FMOE_VARIANT_AUTO 0
#define FMOE_VARIANT_SIMT 1    /* plain CUDA-core kernel; any shape; validation and fp32 */
#define FMOE_VARIANT_STREAM 2  /* small-M weight-streaming kernel, split-K over warps */
#define FMOE_VARIANT_TCGEN05 3 /* TMA + tcgen05/TMEM persistent kernel for large M */

/* ABI version: 2 = argument structs begin with struct_size; 3 = fmoe_gemm_args ends with split_ws / split_ws_bytes;
 * 4 = ... and scale_mode / a_scale_gather; fmoe_fused_args.scale_mode takes the place of a reserved word. */
int fmoe_version(void);
/* Message of the last error returned on the calling thread ("" if none). */
const char* fmoe_last_error(void);
/* Number of SMs of the current device (0 when there is no device). */
int fmoe_sm_count(void);

/*
 * Router: softmax over E experts, top-k, optional renormalisation.
 * Replaces the routing the reference's caller performs before the hook
 * (src/flaggems_sglang/ops/fused_moe.py:355-366 consumes topk_weights/topk_ids;
 * tests/test_fused_moe.py:38-41 builds them with softmax -> topk -> renormalise).
 * Ranking is on the raw logits, ties go to the lower expert index.  A NaN logit ranks as -inf (weight 0); a row
 * with no logit above -inf is routed as if all its logits were equal (ids 0..k-1, equal weights); a +inf logit
 * gives NaN weights as softmax does.  Every id written is inside [0, E).
 *   logits [T,E] f32 row-major -> topk_weights [T,k] f32, topk_ids [T,k] i32
 * Limits: 1 <= k <= 32, k <= E <= 1024.
 */
int fmoe_topk_softmax(const float* logits, int64_t T, int E, int k, int renormalize,
                      float* topk_weights, int32_t* topk_ids, void* stream);

/*
 * Router: DeepSeek-V3 style group-limited top-k on sigmoid scores with a
 * per-expert selection bias (same place in the reference as above; the
 * reference itself has no grouped router).
 *   s = sigmoid(logits); c = s + bias (bias may be NULL);
 *   group score = sum of the 2 largest c of the group; keep topk_group groups;
 *   ids = top-k of c inside kept groups; weights = s[ids], renormalised by
 *   (sum + 1e-20) when `renormalize`, then multiplied by `scale`.
 *   A NaN logit counts as -inf (s = 0), a NaN c (or NaN group score) as -inf; every id written is inside [0, E).
 * Limits: E <= 1024, E % n_group == 0, n_group <= 32, k <= 32.
 */
int fmoe_topk_grouped(const float* logits, const float* bias, int64_t T, int E, int k,
                      int n_group, int topk_group, int renormalize, float scale,
                      float* topk_weights, int32_t* topk_ids, void* stream);

/*
 * moe_align_block_size: sort the flat (token, slot) indices by expert and pad
 * every expert to a multiple of `block`.  Takes over the routing-table
 * construction of src/flaggems_sglang/ops/fused_moe.py:119-146.
 *   topk_ids [numel] i32 (ids outside [0,E) are dropped)
 *   sorted_token_ids [sorted_cap] i32, sorted_cap >= numel + E*(block-1); filled
 *       with the sentinel `numel`, then per expert its slots in ascending order
 *   expert_ids [expert_cap] i32, expert_cap >= ceil(sorted_cap/block); expert of
 *       each used block, -1 after the used blocks
 *   num_tokens_post_padded [1] i32
 * Limits: E <= 1024, numel < 2^31.
 */
int fmoe_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int E, int block,
                              int32_t* sorted_token_ids, int64_t sorted_cap,
                              int32_t* expert_ids, int64_t expert_cap,
                              int32_t* num_tokens_post_padded, void* stream);

/*
 * Same result with caller scratch: inputs of 8192 slots or more are processed by one CTA per 4096 slots
 * (three launches) instead of a single CTA.  workspace needs fmoe_moe_align_workspace_bytes(numel, E) bytes;
 * with workspace == NULL or a small input this is fmoe_moe_align_block_size.
 */
int64_t fmoe_moe_align_workspace_bytes(int64_t numel, int E);
int fmoe_moe_align_block_size_ws(const int32_t* topk_ids, int64_t numel, int E, int block,
                                 int32_t* sorted_token_ids, int64_t sorted_cap,
                                 int32_t* expert_ids, int64_t expert_cap,
                                 int32_t* num_tokens_post_padded, void* workspace, int64_t workspace_bytes,
                                 void* stream);

/*
 * Per-row, per-128-channel dynamic quantisation to e4m3 (the fp8 path the
 * reference rejects at src/flaggems_sglang/ops/fused_moe.py:170-185).
 *   x [rows_in, K] (in_dtype FMOE_BF16 or FMOE_F32), K % 128 == 0
 *   q [rows_out, K] e4m3, scale [rows_out, K/128] f32,
 *   scale = max(amax,1e-10)/448, q = rne(x/scale) saturated to +-448.
 * With row_map == NULL rows_out == rows_in and row r reads row r.  With a
 * row_map (sorted_token_ids) output row p reads input row row_map[p]/map_div
 * (map_div >= 1) or input row p itself (map_div == 0: the map only marks the
 * padding), and rows whose map entry is >= map_sentinel are written as zeros
 * (scale 1) without reading x.
 * Only rows p < *num_rows_dev are produced when num_rows_dev != NULL.
 */
int fmoe_quant_fp8_group128(const void* x, int in_dtype, int64_t rows_out, int64_t K,
                            const int32_t* row_map, int map_div, int64_t map_sentinel,
                            const int32_t* num_rows_dev, void* q, float* scale, void* stream);
/* Per-row dynamic quantisation with ONE scale per row (the activation side of per-channel w8a8: the reference's
 * `per_channel_quant` argument, src/flaggems_sglang/ops/fused_moe.py:160, asserted off there at :173-175):
 *   x [rows_in, K] bf16, K % 8 == 0, K <= 16384; q [rows_out, K] e4m3; scale [rows_out] f32,
 *   scale = max(amax / 448, 1 / (448 * 512)), q = rne(x / scale) saturated to +-448.
 * row_map / map_div / map_sentinel / num_rows_dev as for fmoe_quant_fp8_group128. */
int fmoe_quant_fp8_per_token(const void* x, int in_dtype, int64_t rows_out, int64_t K,
                             const int32_t* row_map, int map_div, int64_t map_sentinel,
                             const int32_t* num_rows_dev, void* q, float* scale, void* stream);

/*
 * Row gather into the padded expert-sorted order (bf16/f32 copy):
 *   out[p,:] = x[row_map[p]/map_div,:], zeros where row_map[p] >= map_sentinel,
 *   for p < *num_rows_dev.  elem_bytes is 2 or 4; K*elem_bytes % 16 == 0.
 */
int fmoe_gather_rows(const void* x, int elem_bytes, int64_t rows_out, int64_t K,
                     const int32_t* row_map, int map_div, int64_t map_sentinel,
                     const int32_t* num_rows_dev, void* out, void* stream);

/*
 * Grouped GEMMs over the expert-sorted token blocks.  Together they take over
 * the two matmul_ogs calls and the activation pass of
 * src/flaggems_sglang/ops/fused_moe.py:205-231.
 */
#define FMOE_SCALE_BLOCK128 0
#define FMOE_SCALE_CHANNEL 1
#define FMOE_W_K_MAJOR 0
#define FMOE_W_N_MAJOR 1
typedef struct fmoe_gemm_args {
  uint32_t struct_size;/* sizeof(fmoe_gemm_args) as the CALLER compiled it; a size the library does not know is
                          refused with FMOE_ERR_INVALID_ARG before any other field is read   */
  int32_t w_layout;    /* FMOE_W_K_MAJOR (0) | FMOE_W_N_MAJOR: see `w`                   */
  int32_t dtype;       /* FMOE_F32 | FMOE_BF16 | FMOE_E4M3: type of a and w            */
  int32_t out_dtype;   /* FMOE_F32 | FMOE_BF16 | FMOE_E4M3 (gemm1+TCGEN05 fp8 only)     */
  int32_t variant;     /* FMOE_VARIANT_*                                                 */
  int32_t num_experts; /* E                                                              */
  int32_t top_k;       /* k                                                              */
  int32_t block_size;  /* block used for sorted_token_ids / expert_ids                   */
  int32_t a_gather;    /* 1: row of `a` for sorted position p is slot/top_k ([T,K] input)
                          0: row of `a` is p itself (input already in sorted order)      */
  int32_t activation;  /* gemm1: FMOE_ACT_SILU | FMOE_ACT_GELU                          */
  int64_t numel;       /* T*k: sentinel in sorted_token_ids, number of output slots      */
  int64_t n;           /* gemm1: I (w has 2I rows per expert); gemm2: H                  */
  int64_t k;           /* reduction length: gemm1 H, gemm2 I                             */
  int64_t a_rows;      /* rows of `a`                                                    */
  int64_t sorted_cap;  /* length of sorted_token_ids                                     */
  int64_t max_blocks;  /* upper bound on used blocks the launch must cover               */
  const void* a;       /* [a_rows, k]                                                    */
  const float* a_scale;/* e4m3: [a_rows, k/128]                                          */
  const void* w;       /* FMOE_W_K_MAJOR: gemm1 [E, 2I, H]; gemm2 [E, H, I]; reduction dim contiguous (the
                          serving-side layout).  FMOE_W_N_MAJOR: gemm1 [E, H, 2I]; gemm2 [E, I, H], the layout
                          the reference operator takes (fused_moe.py:192-199), read in place by the bf16
                          TCGEN05 kernel as an N-major B operand; other kernels refuse it              */
  const float* w_scale;/* e4m3: [E, rows/128, k/128]                                     */
  const int32_t* sorted_token_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_post_padded;
  const float* row_scale; /* [numel] top-k weights by flat slot, or NULL                 */
  void* out;           /* gemm1: [sorted_cap, I] in sorted order; gemm2: [numel, H] by slot */
  float* out_scale;    /* gemm1 with out_dtype e4m3: [sorted_cap, I/128]                 */
  const float* bias;   /* optional f32 [E, rows of w per expert] added to the accumulator first:
                          gemm1 [E,2I] (gate entries then up entries), gemm2 [E,H].  SIMT, STREAM and bf16
                          TCGEN05 kernels                                                             */
  float act_alpha;     /* FMOE_ACT_SWIGLU_OAI                                                         */
  float act_limit;     /* FMOE_ACT_SWIGLU_OAI: clamp limit, <= 0 for none                             */
  void* const* out_rows; /* gemm2, optional: DEVICE array [numel] of row addresses; row `slot` is written
                            at out_rows[slot] instead of out + slot*H (NULL entry: row skipped).  The
                            addresses may be peer memory (expert-parallel combine fused into the
                            epilogue).  STREAM and TCGEN05 variants only.                          */
  void* split_ws;        /* optional scratch of fmoe_gemm_split_workspace_bytes() bytes (16-byte aligned, contents
                            irrelevant): lets the bf16 TCGEN05 kernel cut the tiles of a part-filled last round
                            along K over the idle CTAs.  NULL: every tile is computed by one CTA.  Results are
                            deterministic either way but differ in the last bits between the two.        */
  int64_t split_ws_bytes;
  int32_t scale_mode;    /* e4m3: FMOE_SCALE_BLOCK128 (a_scale [a_rows, k/128], w_scale [E, rows/128, k/128]) or
                            FMOE_SCALE_CHANNEL (a_scale [a_rows], one per row; w_scale [E, rows of w], one per output
                            channel; applied to the finished accumulator; bf16 out; TCGEN05 variant only)        */
  int32_t a_scale_gather;/* FMOE_SCALE_CHANNEL: 1 = a_scale is [tokens] and the scale of sorted position p is
                            a_scale[slot(p) / top_k] (rows quantised once per token, bytes copied into the sorted
                            order); 0 = a_scale is [a_rows], one per row of `a`                                 */
} fmoe_gemm_args;
int64_t fmoe_gemm_split_workspace_bytes(void);
/* Host-side view of the TCGEN05 kernels' work plan (no GPU needed): unit number `unit` of CTA `cta` in a launch of
 * `grid` CTAs over `total_tiles` tiles of `k_steps` K steps each, with at most `max_split` slices per tile (8 for the
 * down GEMM, 4 for the gate/up GEMM, 0 or 1 for no split).  Returns 1 and host_out = {tile, first K step, end K step,
 * slice, slices of this tile}, 0 past the CTA's last unit, -1 on bad arguments. */
int fmoe_debug_tail_plan(int64_t total_tiles, int k_steps, int max_split, int grid, int cta, int64_t unit,
                         int64_t* host_out);

/* gemm1: out[p, c] = act(acc[p, c]) * acc[p, I + c], acc = (a_row(p) . w[e(p)]^T) * row_scale. */
int fmoe_gemm1_silu(const fmoe_gemm_args* args, void* stream);
/* gemm2: out[slot(p), :] = (a[p, :] . w[e(p)]^T) * row_scale[slot(p)], rounded to out_dtype. */
int fmoe_gemm2(const fmoe_gemm_args* args, void* stream);

/*
 * moe_sum / combine: out[t,:] = round(sum_j z[t,j,:]) (fp32, j ascending), then
 * optionally out = round(out * scale) when scale != 1 (the hook's post-multiply,
 * src/flaggems_sglang/ops/fused_moe.py:415-420).  Takes over the grouped reduce
 * the reference's second matmul_ogs call ends with (:224-231).
 *   z [T, k, H], out [T, H]; dtype FMOE_BF16 or FMOE_F32; H*elem % 16 == 0.
 */
int fmoe_moe_sum(const void* z, int dtype, int64_t T, int k, int64_t H, float scale,
                 void* out, void* stream);
/* Same, then out = round(out + addend) with addend [T, H] of the same dtype (NULL: none): the shared expert's
 * output joins the routed experts' in the combine pass instead of in a separate `+=` over [T, H]. */
int fmoe_moe_sum_add(const void* z, int dtype, int64_t T, int k, int64_t H, float scale,
                     const void* addend, void* out, void* stream);

/*
 * Whole expert computation in one call: align -> [row gather / activation quantisation] -> gemm1+silu ->
 * [quantisation] -> gemm2 * weight -> moe_sum.  Takes over src/flaggems_sglang/ops/fused_moe.py:197-232
 * (`triton_kernel_fused_experts` body) and, with b1/b2 and FMOE_ACT_SWIGLU_OAI, :235-325
 * (`triton_kernel_fused_experts_with_bias`) on the serving-side layouts w1 [E,2I,H], w2 [E,H,I].
 * All intermediates live in the caller's `workspace` (size from fmoe_fused_experts_workspace_bytes);
 * nothing is allocated and the host is never synchronised.
 */
typedef struct fmoe_fused_args {
  uint32_t struct_size; /* sizeof(fmoe_fused_args) as the caller compiled it (checked like fmoe_gemm_args.struct_size) */
  int32_t w_layout;     /* FMOE_W_K_MAJOR: w1 [E,2I,H], w2 [E,H,I]; FMOE_W_N_MAJOR: w1 [E,H,2I], w2 [E,I,H] (bf16,
                           TCGEN05 kernels, no bias / swiglu_oai)                                          */
  int32_t dtype;        /* FMOE_F32 | FMOE_BF16: type of hidden/w1/w2/out; FMOE_E4M3: e4m3 weights with
                           128x128 scales, bf16 hidden/out, activations quantised per token per 128 channels */
  int32_t variant;      /* FMOE_VARIANT_* (AUTO: chosen from the shape)                                   */
  int32_t num_experts;  /* E                                                                              */
  int32_t top_k;        /* k                                                                              */
  int32_t apply_router_weight_on_input; /* 1: top-k weight scales the gemm1 input rows instead of gemm2's output */
  int32_t no_combine;   /* 1: out is [T,k,H] (rows by flat slot), no sum over k                            */
  int32_t zero_dropped; /* 1: slots whose id is outside [0,E) must read as zero (expert-parallel shards)  */
  int32_t activation;   /* FMOE_ACT_SILU | FMOE_ACT_GELU                                                  */
  int64_t T, H, I;
  float routed_scaling_factor; /* applied after the sum when != 1 (ignored with no_combine)              */
  int32_t scale_mode;   /* e4m3: FMOE_SCALE_BLOCK128 (0) or FMOE_SCALE_CHANNEL (w1_scale [E,2I], w2_scale [E,H], one
                           scale per output channel; activations quantised with one scale per token; TCGEN05 only) */
  const void* hidden;   /* [T,H]                                                                          */
  const void* w1;       /* [E,2I,H]                                                                       */
  const void* w2;       /* [E,H,I]                                                                        */
  const float* w1_scale;/* e4m3: [E,2I/128,H/128] (FMOE_SCALE_CHANNEL: [E,2I])                                */
  const float* w2_scale;/* e4m3: [E,H/128,I/128]  (FMOE_SCALE_CHANNEL: [E,H])                                 */
  const float* topk_weights; /* [T,k]                                                                     */
  const int32_t* topk_ids;   /* [T,k]                                                                     */
  void* out;            /* [T,H] or [T,k,H]                                                               */
  void* workspace;      /* 256-byte aligned                                                               */
  int64_t workspace_bytes;
  const float* b1;      /* optional f32 [E,2I] bias of the gate/up projection (gate entries then up entries)     */
  const float* b2;      /* optional f32 [E,H] bias of the down projection                                   */
  float act_alpha;      /* FMOE_ACT_SWIGLU_OAI                                                              */
  float act_limit;      /* FMOE_ACT_SWIGLU_OAI: clamp limit, <= 0 for none                                  */
  void* const* out_rows; /* with no_combine: optional DEVICE array [T*k] of row addresses that replace
                            out + slot*H (see fmoe_gemm_args.out_rows); `out` may then be NULL            */
} fmoe_fused_args;

/* Kernel family and moe_align block the AUTO choice takes for a shape.  forced_variant may be AUTO. */
int fmoe_pick_variant(int dtype, int64_t numel, int E, int64_t I, int64_t H, int forced_variant,
                      int* variant_out, int* block_out);
/* Bytes of workspace fmoe_fused_experts needs for these arguments (pointers are not read); < 0 on error. */
int64_t fmoe_fused_experts_workspace_bytes(const fmoe_fused_args* args);
int fmoe_fused_experts(const fmoe_fused_args* args, void* stream);

/*
 * fmoe_fused_experts for callers that cannot allocate device memory.  It has no counterpart in the
 * reference, which allocates its intermediates with torch on every call.
 *
 * Who needs it: code that runs the layer where cudaMalloc (or any allocator built on it) is off limits —
 * on a latency-critical thread that may not take the allocator's locks, or inside a host application that
 * owns all device memory and offers no scratch.  Same arguments and results as
 * fmoe_fused_experts, except that `workspace` / `workspace_bytes` are ignored: the intermediates go to an
 * array of FMOE_STATIC_SCRATCH_BYTES that is part of the library image, so every GPU that loads the
 * library gives up that much memory until the process exits.
 *
 *   - Problems whose workspace (fmoe_fused_experts_workspace_bytes) exceeds FMOE_STATIC_SCRATCH_BYTES are
 *     refused with FMOE_ERR_UNSUPPORTED; nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and remembers it.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it.  The
 *     kernels rewrite every index buffer they read and clear the per-slot outputs when `zero_dropped` is
 *     set, so no stale value is ever consumed; but two calls that overlap on the GPU (different streams
 *     without ordering between them) race on the array and give wrong results.  Serialise them.
 */
#define FMOE_STATIC_SCRATCH_BYTES (64ll << 20)
int64_t fmoe_static_scratch_bytes(void);
int fmoe_fused_experts_static(const fmoe_fused_args* args, void* stream);

/*
 * Expert-parallel token exchange over peer memory (one process per GPU, NVLink P2P stores).  No counterpart in
 * the reference, which has no expert parallelism (expert_map is asserted None,
 * src/flaggems_sglang/ops/fused_moe.py:176-178); the contract is "same numbers as the single-GPU op on the same
 * global batch".  Experts are sharded contiguously: rank j owns global experts [j*experts_per_rank,
 * (j+1)*experts_per_rank).
 *
 * Every rank owns a receive area that its peers write: rows [capacity, row bytes] (bf16 rows, or e4m3 rows with
 * scales [capacity, H/128] f32), weights [capacity] (f32), src [capacity] (two int32: source rank, source slot) and a
 * result area z [z_slots, H].  `peer_*` arguments are DEVICE arrays of `world` pointers, entry j = that area on
 * rank j (entry `rank` = this rank's own).  The kernels only store to peer memory and never wait on a peer; the
 * caller orders the phases across ranks with stream-ordered collectives:
 *
 *   fmoe_ep_expert_counts -> sort by expert (fmoe_moe_align_block_size, block 1, E = all experts) -> all-gather of
 *   `counts` into matrix[world * total_experts] (matrix[r*E + e] = rows rank r holds for global expert e) ->
 *   fmoe_ep_dispatch_sorted -> barrier -> fmoe_ep_recv_tables -> grouped GEMMs straight over the receive area
 *   (fmoe_gemm1_silu / fmoe_gemm2 with top_k = 1, a_gather = 0, numel = capacity) -> fmoe_ep_scatter_rows (or
 *   none: out_rows of fmoe_ep_recv_tables given to fmoe_gemm2) -> barrier -> fmoe_moe_sum over this rank's z.
 *
 * Rows land in the owner's area already in the padded expert-sorted order the grouped GEMMs read: the owner's
 * experts ascending, each starting at a multiple of `block`, inside an expert the ranks in rank order, inside a
 * rank ascending flat slot; the receiver runs no moe_align and no row copy.
 *
 * Misuse that only the device can see (an expert id outside [0, total_experts), a row beyond `capacity`, a
 * corrupt return address) is skipped, recorded, and returned by fmoe_check_device_status as
 * FMOE_ERR_INVALID_ARG; the result rows of skipped slots read as zero.
 */
#define FMOE_EP_IPC_HANDLE_BYTES 64
/* cudaMalloc + IPC handle of a receive area / open and close a peer's / free the own one. */
int fmoe_ep_buffer_create(int64_t bytes, void** ptr, void* ipc_handle /* FMOE_EP_IPC_HANDLE_BYTES, host */);
int fmoe_ep_buffer_open(const void* ipc_handle, void** ptr);
int fmoe_ep_buffer_close(void* ptr);
int fmoe_ep_buffer_destroy(void* ptr);
/* counts[e] = number of entries of topk_ids equal to e, e in [0, total_experts) (<= 1024). */
int fmoe_ep_expert_counts(const int32_t* topk_ids, int64_t numel, int total_experts, int32_t* counts, void* stream);
/* perm: the T*top_k (token, slot) positions sorted by expert (stable; invalid ids dropped).  Sends row
 * perm[p] / top_k of `rows` ([T, row_bytes]; with row_scales [T, scales_per_row] f32 for e4m3 rows) and its
 * weight / return address to the owner of its expert.  own_z: this rank's result area, whose rows of slots that
 * could not be sent are zeroed (NULL: not touched). */
int fmoe_ep_dispatch_sorted(const void* rows, int64_t row_bytes, const float* row_scales, int scales_per_row,
                            int64_t T, int top_k, const int32_t* topk_ids, const float* topk_weights,
                            const int32_t* perm, const int32_t* matrix, int rank, int world, int total_experts,
                            int experts_per_rank, int block, void* const* peer_rows, float* const* peer_scales,
                            float* const* peer_weights, void* const* peer_src, int64_t capacity, void* own_z,
                            int64_t z_row_bytes, void* stream);
/* Tables of this rank's receive area for the grouped GEMMs: sorted_token_ids [capacity] (row index, `capacity` for
 * padding rows), expert_ids [expert_cap >= capacity/block] (local expert of each used block, -1 after them),
 * num_tokens_post_padded [1].  With out_rows != NULL also out_rows[r] = peer_z[src[r].rank] + src[r].slot *
 * z_row_bytes for the received rows (NULL for padding): the table fmoe_gemm_args.out_rows takes, which makes the
 * down-projection epilogue store every result row straight into the slot buffer of the rank it came from. */
int fmoe_ep_recv_tables(const int32_t* matrix, int rank, int world, int total_experts, int experts_per_rank, int block,
                        int64_t capacity, const void* recv_src, int64_t z_slots, void* const* peer_z,
                        int64_t z_row_bytes, int32_t* sorted_token_ids, int32_t* expert_ids, int64_t expert_cap,
                        int32_t* num_tokens_post_padded, void** out_rows, void* stream);
/* z_rows[r] (expert output of received row r, r < *num_rows_dev) -> out_rows[r] (skipped when NULL). */
int fmoe_ep_scatter_rows(const void* z_rows, int64_t row_bytes, void* const* out_rows, const int32_t* num_rows_dev,
                         int64_t capacity, void* stream);

/*
 * Reads and clears the device-side status word that bounded waits inside the
 * tcgen05 kernels set when they give up, and the one of the expert-parallel
 * exchange kernels.  Synchronises `stream`.
 * Returns FMOE_OK, FMOE_ERR_DEVICE_TIMEOUT or FMOE_ERR_INVALID_ARG.
 */
int fmoe_check_device_status(void* stream);

/*
 * Self-test of the time-out reporting: launches a one-warp kernel that waits, for at most `limit_cycles`
 * clock cycles, on a barrier nobody signals; it gives up, records a status code and returns, so the next
 * fmoe_check_device_status returns FMOE_ERR_DEVICE_TIMEOUT and the context stays usable.  No counterpart in
 * the reference (it has no device-side waits).
 */
int fmoe_selftest_bounded_wait(int64_t limit_cycles, void* stream);

/*
 * Diagnostic: per-stage device timing of the calling thread's NEXT fmoe_fused_experts / _static call.
 * `events` is a HOST array of n cudaEvent_t handles (created by the caller with timing enabled, NULL entries
 * are skipped) that stays valid until that call returns; the call records them on its stream at the stage
 * boundaries and forgets the array:
 *   [0] start  [1] align done  [2] input rows gathered / quantised  [3] gate/up GEMM done
 *   [4] activations quantised (e4m3 only)  [5] down GEMM done  [6] sum done
 * n = 0 cancels.  No counterpart in the reference (it times whole calls, benchmark/performance_utils.py:365-377).
 */
#define FMOE_STAGE_EVENTS 7
int fmoe_debug_stage_events(void* const* events, int n);

/*
 * Diagnostic: with the environment variable FMOE_TC_PROFILE set, the bf16 tcgen05 kernel records, per
 * CTA, clock cycles spent waiting {tiles, MMA on accumulator, MMA on data, producer on free stage,
 * epilogue on accumulator, epilogue busy, -, -}.  Copies the last launch's n values (8 per CTA, at most
 * 256 CTAs) to HOST memory.  No counterpart in the reference.
 */
int fmoe_debug_tcgen05_wait_profile(int64_t* host_out, int n);
/* Same for the kernel family `variant`: FMOE_VARIANT_TCGEN05 (bf16) or -FMOE_VARIANT_TCGEN05 for the e4m3 kernel, whose columns are {tiles, MMA waits for a TMEM partial, MMA waits for data, producer waits,
 * fold waits, fold busy, kernel cycles, epilogue cycles}: 256 x 8 values of the last down GEMM, then 256 x 8 of the
 * last gate/up GEMM (n up to 4096). */
int fmoe_debug_wait_profile(int variant, int64_t* host_out, int n);

#ifdef __cplusplus
}
#endif
#endif /* FMOE_B200_H */
