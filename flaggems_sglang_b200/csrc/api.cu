// extern "C" entry points that are not tied to a single kernel file: error
// reporting, device queries and the grouped-GEMM dispatcher.
#include <cstdlib>

#include "gemm.cuh"

namespace fmoe {

bool pdl_enabled() {
  static const bool on = [] {
    const char* env = getenv("FMOE_PDL");
    return !(env && env[0] == '0');
  }();
  return on;
}

char* last_error_buffer() {
  static thread_local char buf[kErrBufSize] = {0};
  return buf;
}

namespace {

int validate_gemm(const GemmParams& a, bool gated, const char* who) {
  FMOE_REQUIRE(a.dtype == FMOE_F32 || a.dtype == FMOE_BF16 || a.dtype == FMOE_E4M3, "%s: unknown dtype %d", who, a.dtype);
  FMOE_REQUIRE(a.num_experts >= 1 && a.top_k >= 1 && a.block_size >= 1, "%s: bad E/top_k/block_size", who);
  FMOE_REQUIRE(a.activation == FMOE_ACT_SILU || a.activation == FMOE_ACT_GELU || a.activation == FMOE_ACT_SWIGLU_OAI,
               "%s: unknown activation %d", who, a.activation);
  FMOE_REQUIRE(a.w_layout == FMOE_W_K_MAJOR || a.w_layout == FMOE_W_N_MAJOR, "%s: unknown w_layout %d", who, a.w_layout);
  if (a.w_layout == FMOE_W_N_MAJOR) {
    if (a.dtype != FMOE_BF16 || (a.variant != FMOE_VARIANT_AUTO && a.variant != FMOE_VARIANT_TCGEN05))
      return fail(FMOE_ERR_UNSUPPORTED, "%s: [E,K,N] weights (FMOE_W_N_MAJOR) are read by the bf16 TCGEN05 kernel only", who);
  }
  if (a.bias || a.activation == FMOE_ACT_SWIGLU_OAI)
    FMOE_REQUIRE(a.dtype != FMOE_E4M3, "%s: bias and the swiglu_oai activation are not available with e4m3 weights", who);
  FMOE_REQUIRE(a.numel >= 0 && a.n >= 1 && a.k >= 1, "%s: bad sizes numel=%lld n=%lld k=%lld", who,
               (long long)a.numel, (long long)a.n, (long long)a.k);
  FMOE_REQUIRE(a.max_blocks >= 0 && a.max_blocks * a.block_size <= a.sorted_cap,
               "%s: max_blocks*block_size (%lld) exceeds sorted_cap (%lld)", who,
               (long long)(a.max_blocks * a.block_size), (long long)a.sorted_cap);
  if (a.max_blocks == 0 || a.numel == 0) return FMOE_OK;
  FMOE_REQUIRE(a.a && a.w && (a.out || (!gated && a.out_rows)) && a.sorted_token_ids && a.expert_ids &&
                   a.num_tokens_post_padded,
               "%s: null pointer", who);
  if (a.out_rows)
    FMOE_REQUIRE(!gated && (a.variant == FMOE_VARIANT_STREAM || a.variant == FMOE_VARIANT_TCGEN05),
                 "%s: out_rows is taken by gemm2 with the STREAM or TCGEN05 variant only", who);
  if (a.dtype == FMOE_E4M3) {
    FMOE_REQUIRE(a.a_scale && a.w_scale, "%s: e4m3 needs a_scale and w_scale", who);
    FMOE_REQUIRE(a.scale_mode == FMOE_SCALE_BLOCK128 || a.scale_mode == FMOE_SCALE_CHANNEL, "%s: unknown scale_mode %d",
                 who, a.scale_mode);
    if (a.scale_mode == FMOE_SCALE_CHANNEL) {
      if (a.variant != FMOE_VARIANT_AUTO && a.variant != FMOE_VARIANT_TCGEN05)
        return fail(FMOE_ERR_UNSUPPORTED, "%s: per-channel e4m3 scales are taken by the TCGEN05 kernel only", who);
      FMOE_REQUIRE(a.k % 16 == 0 && a.n % 32 == 0, "%s: per-channel e4m3 needs k %% 16 == 0 and n %% 32 == 0", who);
    } else {
      FMOE_REQUIRE(a.k % 128 == 0 && a.n % 128 == 0, "%s: e4m3 needs k and n to be multiples of 128", who);
    }
  }
  if (!a.a_gather)
    FMOE_REQUIRE(a.a_rows >= a.max_blocks * a.block_size, "%s: a has %lld rows, the launch covers %lld", who,
                 (long long)a.a_rows, (long long)(a.max_blocks * a.block_size));
  else
    FMOE_REQUIRE(a.a_rows * a.top_k >= a.numel, "%s: a has %lld rows but numel/top_k needs more", who,
                 (long long)a.a_rows);
  return FMOE_OK;
}

int dispatch_gemm(const fmoe_gemm_args* args, bool gated, void* stream, const char* who) {
  if (!args) return fail(FMOE_ERR_INVALID_ARG, "%s: args is null", who);
  if (args->struct_size != sizeof(fmoe_gemm_args))
    return fail(FMOE_ERR_INVALID_ARG, "%s: fmoe_gemm_args.struct_size is %u, this library's struct has %zu bytes "
                "(binding built against another header?)", who, args->struct_size, sizeof(fmoe_gemm_args));
  const GemmParams& a = *args;
  int rc = validate_gemm(a, gated, who);
  if (rc) return rc;
  if (a.max_blocks == 0 || a.numel == 0) return FMOE_OK;
  auto st = (cudaStream_t)stream;
  int variant = a.variant;
  if (a.w_layout == FMOE_W_N_MAJOR || (a.dtype == FMOE_E4M3 && a.scale_mode == FMOE_SCALE_CHANNEL)) {
    variant = FMOE_VARIANT_TCGEN05;
  } else if (variant == FMOE_VARIANT_AUTO) {
    if (gemm_tcgen05_supports(a, gated) || gemm_tcgen05_fp8_supports(a, gated))
      variant = FMOE_VARIANT_TCGEN05;
    else if (gemm_stream_supports(a, gated))
      variant = FMOE_VARIANT_STREAM;
    else
      variant = FMOE_VARIANT_SIMT;
  }
  switch (variant) {
    case FMOE_VARIANT_SIMT: return gemm_simt(a, gated, st);
    case FMOE_VARIANT_STREAM: return gemm_stream(a, gated, st);
    case FMOE_VARIANT_TCGEN05:
      return (a.dtype == FMOE_E4M3 && a.scale_mode == FMOE_SCALE_BLOCK128) ? gemm_tcgen05_fp8(a, gated, st)
                                                                           : gemm_tcgen05(a, gated, st);
  }
  return fail(FMOE_ERR_INVALID_ARG, "%s: unknown variant %d", who, a.variant);
}

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_version(void) { return 4; }

extern "C" int64_t fmoe_gemm_split_workspace_bytes(void) { return fmoe::gemm_tcgen05_split_workspace_bytes(); }

extern "C" int fmoe_debug_tail_plan(int64_t total_tiles, int k_steps, int max_split, int grid, int cta, int64_t unit,
                                    int64_t* host_out) {
  if (!host_out || grid < 1 || cta < 0 || cta >= grid || total_tiles < 0 || k_steps < 1 || unit < 0) return -1;
  return fmoe::tail_plan_unit(total_tiles, k_steps, max_split, grid, cta, unit, host_out);
}

extern "C" const char* fmoe_last_error(void) { return fmoe::last_error_buffer(); }

extern "C" int fmoe_sm_count(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

extern "C" int fmoe_gemm1_silu(const fmoe_gemm_args* args, void* stream) {
  return fmoe::dispatch_gemm(args, true, stream, "gemm1_silu");
}

extern "C" int fmoe_gemm2(const fmoe_gemm_args* args, void* stream) {
  return fmoe::dispatch_gemm(args, false, stream, "gemm2");
}

namespace fmoe {
int read_wait_profile(long long* host_out, int n);
int read_wait_profile_fp8(long long* host_out, int n);
int launch_bounded_wait_selftest(long long limit_cycles, cudaStream_t st);
}  // namespace fmoe

extern "C" int fmoe_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
  if (limit_cycles < 1 || limit_cycles > 2000000000ll) return fmoe::fail(FMOE_ERR_INVALID_ARG, "selftest: limit out of range");
  return fmoe::launch_bounded_wait_selftest(limit_cycles, (cudaStream_t)stream);
}

extern "C" int fmoe_debug_tcgen05_wait_profile(int64_t* host_out, int n) {
  if (!host_out || n < 0 || n > 256 * 8) return fmoe::fail(FMOE_ERR_INVALID_ARG, "wait profile: bad buffer");
  return fmoe::read_wait_profile(reinterpret_cast<long long*>(host_out), n);
}

extern "C" int fmoe_debug_wait_profile(int variant, int64_t* host_out, int n) {
  if (!host_out || n < 0 || n > (variant == -FMOE_VARIANT_TCGEN05 ? 2 : 1) * 256 * 8) return fmoe::fail(FMOE_ERR_INVALID_ARG, "wait profile: bad buffer");
  if (variant == FMOE_VARIANT_TCGEN05) return fmoe::read_wait_profile(reinterpret_cast<long long*>(host_out), n);
  if (variant == -FMOE_VARIANT_TCGEN05) return fmoe::read_wait_profile_fp8(reinterpret_cast<long long*>(host_out), n);
  return fmoe::fail(FMOE_ERR_INVALID_ARG, "wait profile: variant %d keeps none", variant);
}

extern "C" int fmoe_check_device_status(void* stream) {
  int status = 0;
  int rc = fmoe::read_and_clear_device_status((cudaStream_t)stream, &status);
  if (rc) return rc;
  if ((status & 0xF00) == 0xA00)
    return fmoe::fail(FMOE_ERR_INVALID_ARG,
                      "expert-parallel exchange skipped rows (site code 0x%x: 0xA00 expert id out of range, "
                      "0xA01 receive capacity exceeded, 0xA02 bad return address)", status);
  if (status != 0)
    return fmoe::fail(FMOE_ERR_DEVICE_TIMEOUT, "a bounded wait inside a tcgen05 kernel gave up (site code 0x%x)", status);
  return FMOE_OK;
}
