// fmoe_fused_experts_static: the one-call expert computation for callers that must not allocate.
//
// Some callers of this library cannot call cudaMalloc at the point where they run an MoE layer: a real-time
// serving loop that forbids allocator calls on its hot thread, or an embedding process whose memory pool is owned by someone else
// and hands out no scratch.  For them the intermediates of fmoe_fused_experts (sorted index buffers, the
// activation between the two GEMMs, the per-slot outputs) live in a fixed array in device memory that is
// part of this library's image instead of a caller-provided workspace.
#include <mutex>

#include "fused.cuh"

namespace fmoe {
namespace {

constexpr int64_t kStaticScratchBytes = FMOE_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Held by every GPU that loads the library, from load until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
uint8_t* g_scratch_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, with that device current.
int static_scratch_for_current_device(uint8_t** out) {
  int dev = -1;
  FMOE_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FMOE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess)
      return fail(FMOE_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(err));
    if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255u) != 0)
      return fail(FMOE_ERR_CUDA, "static scratch has an unusable device address %p", ptr);
    g_scratch_ptr[dev] = static_cast<uint8_t*>(ptr);
  }
  *out = g_scratch_ptr[dev];
  return FMOE_OK;
}

}  // namespace
}  // namespace fmoe

extern "C" int64_t fmoe_static_scratch_bytes(void) { return fmoe::kStaticScratchBytes; }

extern "C" int fmoe_fused_experts_static(const fmoe_fused_args* args, void* stream) {
  using namespace fmoe;
  if (!args) return fail(FMOE_ERR_INVALID_ARG, "fused_experts_static: args is null");
  FusedPlan plan;
  int rc = plan_fused(*args, &plan);
  if (rc) return rc;
  if (plan.total > kStaticScratchBytes)
    return fail(FMOE_ERR_UNSUPPORTED,
                "fused_experts_static: this problem needs %lld bytes of scratch, the built-in array holds %lld; "
                "use fmoe_fused_experts with a caller workspace",
                (long long)plan.total, (long long)kStaticScratchBytes);
  if (args->T == 0) return FMOE_OK;
  uint8_t* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  return run_fused(*args, plan, scratch, stream);
}
