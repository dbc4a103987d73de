// Expert-parallel token exchange over peer memory (NVLink / NVSwitch, plain P2P stores).
//
// Every rank owns one receive area that its peers can write: rows [capacity, H], and per row the local
// expert id, the gate weight and the return address (source rank, source slot); plus a result area
// z [slots, H] that the expert ranks write back into.  The kernels here only *store* to peer memory and
// never wait on a peer: ordering between ranks comes from stream-ordered collectives issued by the host
// layer between the phases (count all-gather before the dispatch, a barrier after the dispatch and after
// the combine), so there is no spin-wait that could hang.
//
//   fmoe_ep_route      dest rank of every (token, slot) pair + rows per destination
//   fmoe_ep_dispatch   row p of the destination-sorted order -> peer dest, at the offset the count matrix gives
//   fmoe_ep_mask_tail  receive-area ids past the received rows := -1 (ignored by moe_align_block_size); optionally
//                      the table of return addresses that lets the down-projection epilogue store its rows
//                      straight into the source ranks' z (fmoe_gemm_args.out_rows)
//   fmoe_ep_combine    expert output row r -> z[slot] of the rank that sent row r (when the GEMM did not)
//
// The reference has no expert parallelism (expert_map is asserted None,
// FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:176-178).
#include "common.cuh"

namespace fmoe {

// This translation unit's status word; read by status_word_ep().
__device__ int g_device_status_ep = 0;

namespace {

constexpr int kMaxWorld = 64;

__device__ __forceinline__ void report_ep(int code) { atomicCAS(&g_device_status_ep, 0, code); }

__global__ void __launch_bounds__(1024)
ep_route_kernel(const int32_t* __restrict__ ids, int64_t numel, int experts_per_rank, int world,
                int32_t* __restrict__ dest, int32_t* __restrict__ counts) {
  __shared__ int hist[kMaxWorld];
  for (int j = threadIdx.x; j < world; j += blockDim.x) hist[j] = 0;
  __syncthreads();
  const int64_t total_experts = (int64_t)experts_per_rank * world;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t id = ids[i];
    int d = world;  // out of range: dropped by the sort, and reported
    if (id >= 0 && id < total_experts) {
      d = id / experts_per_rank;
      atomicAdd(&hist[d], 1);
    } else {
      report_ep(0xA00);
    }
    dest[i] = d;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < world; j += blockDim.x)
    if (hist[j]) atomicAdd(&counts[j], hist[j]);
}

// matrix[i*world + j] = rows rank i sends to rank j.  Rows from rank i occupy, in rank j's receive area, the
// range starting at sum_{i' < i} matrix[i'][j], in the order of the sender's destination-sorted list.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4* __restrict__ hidden, int64_t vec_per_row, int top_k, const int32_t* __restrict__ ids,
                   const float* __restrict__ weights, const int32_t* __restrict__ perm,
                   const int32_t* __restrict__ matrix, int rank, int world, int experts_per_rank,
                   uint4* const* __restrict__ peer_rows, int32_t* const* __restrict__ peer_ids,
                   float* const* __restrict__ peer_weights, int2* const* __restrict__ peer_src, int64_t capacity) {
  __shared__ int64_t s_start[kMaxWorld + 1];  // first position of destination j in this rank's sorted list
  __shared__ int64_t s_base[kMaxWorld];       // first row of this rank's range in destination j's receive area
  if (threadIdx.x == 0) {
    int64_t acc = 0;
    for (int j = 0; j < world; ++j) {
      s_start[j] = acc;
      acc += matrix[rank * world + j];
    }
    s_start[world] = acc;
  }
  if (threadIdx.x < world) {
    int64_t base = 0;
    for (int i = 0; i < rank; ++i) base += matrix[i * world + threadIdx.x];
    s_base[threadIdx.x] = base;
  }
  __syncthreads();
  const int64_t sent = s_start[world];
  for (int64_t p = blockIdx.x; p < sent; p += gridDim.x) {
    const int32_t slot = perm[p];
    const int32_t id = ids[slot];
    const int j = id / experts_per_rank;
    const int64_t row = s_base[j] + (p - s_start[j]);
    if (row >= capacity) {
      if (threadIdx.x == 0) report_ep(0xA01);
      continue;
    }
    const uint4* src = hidden + (int64_t)(slot / top_k) * vec_per_row;
    uint4* dst = peer_rows[j] + row * vec_per_row;
    for (int64_t c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = __ldg(src + c);
    if (threadIdx.x == 0) {
      peer_ids[j][row] = id - j * experts_per_rank;
      peer_weights[j][row] = weights[slot];
      peer_src[j][row] = make_int2(rank, slot);
    }
  }
  __threadfence_system();
}

__device__ __forceinline__ int64_t rows_received(const int32_t* matrix, int rank, int world) {
  int64_t total = 0;
  for (int i = 0; i < world; ++i) total += matrix[i * world + rank];
  return total;
}

__global__ void __launch_bounds__(256)
ep_mask_tail_kernel(int32_t* __restrict__ recv_ids, const int32_t* __restrict__ matrix, int rank, int world,
                    int64_t capacity, const int2* __restrict__ recv_src, int64_t z_slots,
                    uint8_t* const* __restrict__ peer_z, int64_t row_bytes, void** __restrict__ out_rows) {
  const int64_t total = min(rows_received(matrix, rank, world), capacity);
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < capacity; r += (int64_t)gridDim.x * blockDim.x) {
    if (r >= total) {
      recv_ids[r] = -1;
      if (out_rows) out_rows[r] = nullptr;
    } else if (out_rows) {
      const int2 s = recv_src[r];
      const bool ok = s.x >= 0 && s.x < world && s.y >= 0 && s.y < z_slots;
      if (!ok) report_ep(0xA02);
      out_rows[r] = ok ? peer_z[s.x] + (int64_t)s.y * row_bytes : nullptr;
    }
  }
}

__global__ void __launch_bounds__(256)
ep_combine_kernel(const uint4* __restrict__ z, int64_t vec_per_row, const int2* __restrict__ recv_src,
                  const int32_t* __restrict__ matrix, int rank, int world, int64_t capacity, int64_t z_slots,
                  uint4* const* __restrict__ peer_z) {
  const int64_t total = min(rows_received(matrix, rank, world), capacity);
  for (int64_t r = blockIdx.x; r < total; r += gridDim.x) {
    const int2 s = recv_src[r];
    if (s.x < 0 || s.x >= world || s.y < 0 || s.y >= z_slots) {
      if (threadIdx.x == 0) report_ep(0xA02);
      continue;
    }
    const uint4* src = z + r * vec_per_row;
    uint4* dst = peer_z[s.x] + (int64_t)s.y * vec_per_row;
    for (int64_t c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = __ldg(src + c);
  }
  __threadfence_system();
}

}  // namespace

int status_word_ep(int* out, bool clear) {
  int zero = 0;
  FMOE_CUDA_OK(cudaMemcpyFromSymbol(out, g_device_status_ep, sizeof(int)));
  if (clear && *out != 0) FMOE_CUDA_OK(cudaMemcpyToSymbol(g_device_status_ep, &zero, sizeof(int)));
  return FMOE_OK;
}

}  // namespace fmoe

extern "C" int fmoe_ep_buffer_create(int64_t bytes, void** ptr, void* ipc_handle) {
  using namespace fmoe;
  static_assert(sizeof(cudaIpcMemHandle_t) == FMOE_EP_IPC_HANDLE_BYTES, "handle size");
  FMOE_REQUIRE(bytes > 0 && ptr && ipc_handle, "ep_buffer_create: bad arguments");
  void* p = nullptr;
  FMOE_CUDA_OK(cudaMalloc(&p, (size_t)bytes));
  cudaError_t err = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(ipc_handle), p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return fail(FMOE_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(err));
  }
  *ptr = p;
  return FMOE_OK;
}

extern "C" int fmoe_ep_buffer_open(const void* ipc_handle, void** ptr) {
  using namespace fmoe;
  FMOE_REQUIRE(ipc_handle && ptr, "ep_buffer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  FMOE_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FMOE_OK;
}

extern "C" int fmoe_ep_buffer_close(void* ptr) {
  using namespace fmoe;
  if (ptr) FMOE_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return FMOE_OK;
}

extern "C" int fmoe_ep_buffer_destroy(void* ptr) {
  using namespace fmoe;
  if (ptr) FMOE_CUDA_OK(cudaFree(ptr));
  return FMOE_OK;
}

extern "C" int fmoe_ep_route(const int32_t* topk_ids, int64_t numel, int experts_per_rank, int world, int32_t* dest,
                             int32_t* counts, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(world >= 1 && world <= kMaxWorld && experts_per_rank >= 1, "ep_route: need 1 <= world <= %d and experts_per_rank >= 1", kMaxWorld);
  FMOE_REQUIRE(numel >= 0 && counts, "ep_route: bad arguments");
  auto st = (cudaStream_t)stream;
  FMOE_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * world, st));
  if (numel == 0) return FMOE_OK;
  FMOE_REQUIRE(topk_ids && dest, "ep_route: null pointer");
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(numel, 4096), 148);
  ep_route_kernel<<<grid, 1024, 0, st>>>(topk_ids, numel, experts_per_rank, world, dest, counts);
  return launch_status("ep_route_kernel");
}

extern "C" int fmoe_ep_dispatch(const void* hidden, int elem_bytes, int64_t T, int64_t H, int top_k,
                                const int32_t* topk_ids, const float* topk_weights, const int32_t* perm,
                                const int32_t* matrix, int rank, int world, int experts_per_rank,
                                void* const* peer_rows, int32_t* const* peer_ids, float* const* peer_weights,
                                void* const* peer_src, int64_t capacity, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "ep_dispatch: bad rank %d of %d", rank, world);
  FMOE_REQUIRE(top_k >= 1 && experts_per_rank >= 1 && capacity >= 0, "ep_dispatch: bad top_k / experts_per_rank / capacity");
  FMOE_REQUIRE((elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4) && H > 0 && (H * elem_bytes) % 16 == 0,
               "ep_dispatch: row size must be a multiple of 16 bytes");
  if (T <= 0) return FMOE_OK;
  FMOE_REQUIRE(hidden && topk_ids && topk_weights && perm && matrix && peer_rows && peer_ids && peer_weights && peer_src,
               "ep_dispatch: null pointer");
  FMOE_REQUIRE(aligned16(hidden), "ep_dispatch: hidden must be 16-byte aligned");
  const unsigned grid = (unsigned)std::min<int64_t>(T * top_k, 148 * 8);
  ep_dispatch_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)hidden, H * elem_bytes / 16, top_k, topk_ids, topk_weights, perm, matrix, rank, world,
      experts_per_rank, (uint4* const*)peer_rows, peer_ids, peer_weights, (int2* const*)peer_src, capacity);
  return launch_status("ep_dispatch_kernel");
}

extern "C" int fmoe_ep_mask_tail(int32_t* recv_ids, const int32_t* matrix, int rank, int world, int64_t capacity,
                                 const void* recv_src, int64_t z_slots, void* const* peer_z, int64_t row_bytes,
                                 void** out_rows, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "ep_mask_tail: bad rank %d of %d", rank, world);
  if (capacity <= 0) return FMOE_OK;
  FMOE_REQUIRE(recv_ids && matrix, "ep_mask_tail: null pointer");
  if (out_rows)
    FMOE_REQUIRE(recv_src && peer_z && row_bytes > 0 && row_bytes % 16 == 0 && z_slots >= 0,
                 "ep_mask_tail: out_rows needs recv_src, peer_z and a row size that is a multiple of 16 bytes");
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(capacity, 256), 148 * 4);
  ep_mask_tail_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(recv_ids, matrix, rank, world, capacity,
                                                              (const int2*)recv_src, z_slots,
                                                              (uint8_t* const*)peer_z, row_bytes, out_rows);
  return launch_status("ep_mask_tail_kernel");
}

extern "C" int fmoe_ep_combine(const void* z_rows, int elem_bytes, int64_t H, const void* recv_src,
                               const int32_t* matrix, int rank, int world, int64_t capacity, int64_t z_slots,
                               void* const* peer_z, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "ep_combine: bad rank %d of %d", rank, world);
  FMOE_REQUIRE((elem_bytes == 2 || elem_bytes == 4) && H > 0 && (H * elem_bytes) % 16 == 0,
               "ep_combine: row size must be a multiple of 16 bytes");
  if (capacity <= 0) return FMOE_OK;
  FMOE_REQUIRE(z_rows && recv_src && matrix && peer_z && aligned16(z_rows), "ep_combine: null or misaligned pointer");
  const unsigned grid = (unsigned)std::min<int64_t>(capacity, 148 * 8);
  ep_combine_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)z_rows, H * elem_bytes / 16,
                                                            (const int2*)recv_src, matrix, rank, world, capacity,
                                                            z_slots, (uint4* const*)peer_z);
  return launch_status("ep_combine_kernel");
}
