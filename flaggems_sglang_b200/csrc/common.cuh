// Shared host/device helpers for the fmoe_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/fmoe_b200.h"

namespace fmoe {

// Thread-local message buffer behind fmoe_last_error().
char* last_error_buffer();
constexpr int kErrBufSize = 512;

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), kErrBufSize, fmt, ap);
  va_end(ap);
  return code;
}

#define FMOE_REQUIRE(cond, ...)                                  \
  do {                                                           \
    if (!(cond)) return ::fmoe::fail(FMOE_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

#define FMOE_CUDA_OK(expr)                                                        \
  do {                                                                            \
    cudaError_t err__ = (expr);                                                   \
    if (err__ != cudaSuccess)                                                     \
      return ::fmoe::fail(FMOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(FMOE_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(err));
  return FMOE_OK;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// The kernels of a decode-sized layer call run for a few microseconds each, so the gap between two launches
// is a visible share of the call.  Kernels launched through launch_pdl() may be scheduled while their
// predecessor on the stream is still running; each of them starts with pdl_entry(), which first lets its own
// successor be scheduled and then waits until the predecessor grid has completed and its writes are visible.
// Nothing is read or written before that wait, so the data flow is the one of ordinary stream order.
// FMOE_PDL=0 turns the launch attribute off (plain stream serialisation).
bool pdl_enabled();

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_entry() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // the error is picked up by launch_status()
}
#endif

// One-time set-up that is a property of a DEVICE (cudaFuncSetAttribute, the SM count): runs once per device
// ordinal, with that device current, so a process that drives several GPUs configures each of them.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
};
template <typename Fn>
inline cudaError_t per_device_once(PerDeviceOnce& st, Fn fn) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return fn();
  std::lock_guard<std::mutex> lock(st.mu);
  if (st.done[dev]) return cudaSuccess;
  err = fn();
  if (err == cudaSuccess) st.done[dev] = true;
  return err;
}

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) {
  return (a + b - 1) / b;
}

// ---- element conversions -------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__nv_fp8_e4m3 v) { return float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ uint8_t f32_to_e4m3_bits(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// RN(v / s) for many v and one s: with r = RN(1/s), two residual corrections of v*r give the correctly rounded
// quotient (Markstein), the same bits as an IEEE division, in 5 instructions per element.  The caller falls back to
// __fdiv_rn when the group holds an infinity (the residual would be inf - inf).
__device__ __forceinline__ float div_by_shared(float v, float s, float r) {
  float q = v * r;
  q = fmaf(fmaf(-q, s, v), r, q);
  q = fmaf(fmaf(-q, s, v), r, q);
  return q;
}

// silu(g) * u exactly as the reference kernel writes it: (g / (1 + exp(-g))) * u in fp32
// (FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:62).
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdiv_rn(g, 1.0f + expf(-g)) * u;
}

// Gated activation of gemm1's epilogue: act(g) * u.  0 = silu (default), 1 = gelu (erf form), as the
// reference's two activations (src/flaggems_sglang/ops/fused_moe.py:217-220).
__device__ __forceinline__ float act_mul(float g, float u, int activation) {
  if (activation == FMOE_ACT_GELU) return 0.5f * g * (1.0f + erff(g * 0.70710678118654752f)) * u;
  return silu_mul(g, u);
}

// Same with the hardware approximations (ex2 / rcp based, relative error ~1e-6, far below the bf16
// rounding of the result): the exact IEEE division and expf cost ~50 instructions per output, which made
// the epilogue of the large-M kernels as long as a short main loop.
__device__ __forceinline__ float act_mul_fast(float g, float u, int activation) {
  if (activation == FMOE_ACT_GELU) return 0.5f * g * (1.0f + erff(g * 0.70710678118654752f)) * u;
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Output of the gate/up projection for one column: accumulators g, u of the gate and up rows, their biases
// (0 without), the row scale, the activation and its parameters.  See FMOE_ACT_* for the order of operations.
// FAST selects the ex2/rcp based forms (bf16 epilogues of the large-M kernels).
template <bool FAST>
__device__ __forceinline__ float gated_output(float g, float u, float bg, float bu, float rs, int activation,
                                              float alpha, float limit) {
  g += bg;
  u += bu;
  if (activation == FMOE_ACT_SWIGLU_OAI) {
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fmaxf(-limit, fminf(u, limit));
    }
    const float s = FAST ? __fdividef(g, 1.0f + __expf(-alpha * g)) : __fdiv_rn(g, 1.0f + expf(-alpha * g));
    return fmaf(s, u, s) * rs;
  }
  return FAST ? act_mul_fast(g * rs, u * rs, activation) : act_mul(g * rs, u * rs, activation);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Streaming 16-byte load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// 16-byte load through L1 (small operands re-read by every warp of the CTA).
__device__ __forceinline__ uint4 ldg_cached_v4(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

}  // namespace fmoe
