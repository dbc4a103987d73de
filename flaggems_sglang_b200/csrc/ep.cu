// Expert-parallel token exchange over peer memory (NVLink / NVSwitch, plain P2P stores).
//
// Every rank owns one receive area that its peers can write: rows [capacity, row bytes] (bf16, or e4m3 with a
// [capacity, H/128] scale area), and per row the gate weight and the return address (source rank, source slot);
// plus a result area z [slots, H] that the expert ranks write back into.  Rows arrive ALREADY in the padded
// expert-sorted order the grouped GEMMs consume: the ranks all-gather their per-expert row counts, and every
// sender computes from that matrix where, in the owner's receive area, its rows of an expert belong.  The
// receiver therefore runs neither moe_align nor a row copy (nor, for e4m3, a quantisation pass: the sender
// quantises each token once and ships bytes + scales).
//
// The kernels here only *store* to peer memory and never wait on a peer: ordering between ranks comes from
// stream-ordered collectives issued by the host layer between the phases (count all-gather before the
// dispatch, a barrier after the dispatch and after the combine), so there is no spin-wait that could hang.
//
//   fmoe_ep_expert_counts    rows per global expert of this rank's (token, slot) pairs
//   fmoe_ep_dispatch_sorted  this rank's rows, sorted by expert -> the owners' receive areas
//   fmoe_ep_recv_tables      sorted_token_ids / expert_ids / num_tokens_post_padded of the receive area and the
//                            table of return addresses (fmoe_gemm_args.out_rows)
//   fmoe_ep_scatter_rows     expert output row r -> its return address (when the down projection did not store it)
//
// The reference has no expert parallelism (expert_map is asserted None,
// FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:176-178).
#include "common.cuh"

namespace fmoe {

// This translation unit's status word; read by status_word_ep().
__device__ int g_device_status_ep = 0;

namespace {

constexpr int kMaxWorld = 64;
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ void report_ep(int code) { atomicCAS(&g_device_status_ep, 0, code); }

__global__ void __launch_bounds__(1024)
ep_expert_counts_kernel(const int32_t* __restrict__ ids, int64_t numel, int total_experts, int32_t* __restrict__ counts) {
  __shared__ int hist[kMaxExperts];
  for (int j = threadIdx.x; j < total_experts; j += blockDim.x) hist[j] = 0;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t id = ids[i];
    if (id >= 0 && id < total_experts)
      atomicAdd(&hist[id], 1);
    else
      report_ep(0xA00);  // dropped: the slot's result row reads as zero
  }
  __syncthreads();
  for (int j = threadIdx.x; j < total_experts; j += blockDim.x)
    if (hist[j]) atomicAdd(&counts[j], hist[j]);
}

// Layout of rank j's receive area, from the count matrix m[r * E + e] (rows rank r holds for global expert e):
// its experts in ascending order, expert e starting at the block-aligned row
//     base(e) = sum over the owner's experts e' < e of round_up(total(e'), block),  total(e) = sum_r m[r][e]
// and, inside the expert, the ranks' rows in rank order (rank r's first row at base(e) + sum_{r' < r} m[r'][e]),
// each rank's rows in the order of its expert-sorted list (ascending flat slot).
struct AreaLayout {
  int32_t base[kMaxExperts];   // first row of expert e in its owner's area
  int32_t total[kMaxExperts];  // rows of expert e over all ranks
};

// All threads of the CTA; ends with __syncthreads().
__device__ __forceinline__ void build_layout(AreaLayout& L, const int32_t* __restrict__ m, int world, int total_experts,
                                             int experts_per_rank, int block) {
  for (int e = threadIdx.x; e < total_experts; e += blockDim.x) {
    int t = 0;
    for (int r = 0; r < world; ++r) t += m[r * total_experts + e];
    L.total[e] = t;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < world; j += blockDim.x) {  // one thread per owner: its experts in order
    int acc = 0;
    for (int e = j * experts_per_rank; e < (j + 1) * experts_per_rank; ++e) {
      L.base[e] = acc;
      acc += (L.total[e] + block - 1) / block * block;
    }
  }
  __syncthreads();
}

// perm: this rank's (token, slot) positions sorted by expert (stable), `sent` of them valid.
__global__ void __launch_bounds__(256)
ep_dispatch_sorted_kernel(const uint4* __restrict__ rows_in, int64_t vec_per_row, const float* __restrict__ scales_in,
                          int scales_per_row, int top_k, const int32_t* __restrict__ ids,
                          const float* __restrict__ weights, const int32_t* __restrict__ perm, int64_t numel,
                          const int32_t* __restrict__ matrix, int rank, int world, int total_experts,
                          int experts_per_rank, int block, uint4* const* __restrict__ peer_rows,
                          float* const* __restrict__ peer_scales, float* const* __restrict__ peer_weights,
                          int2* const* __restrict__ peer_src, int64_t capacity, uint4* __restrict__ own_z,
                          int64_t z_vec_per_row) {
  __shared__ AreaLayout L;
  __shared__ int32_t s_first[kMaxExperts];  // first row, in the owner's area, of THIS rank's rows of expert e
  __shared__ int32_t s_start[kMaxExperts];  // first position of expert e in this rank's sorted list
  __shared__ int32_t s_sent;
  build_layout(L, matrix, world, total_experts, experts_per_rank, block);
  for (int e = threadIdx.x; e < total_experts; e += blockDim.x) {
    int off = 0;
    for (int r = 0; r < rank; ++r) off += matrix[r * total_experts + e];
    s_first[e] = L.base[e] + off;
  }
  // exclusive prefix of this rank's own counts: per-thread chunks, then a serial pass over the chunk sums
  __shared__ int32_t s_chunk[256];
  const int per_thread = (total_experts + blockDim.x - 1) / blockDim.x;
  {
    int acc = 0;
    for (int i = 0; i < per_thread; ++i) {
      const int e = threadIdx.x * per_thread + i;
      if (e < total_experts) {
        s_start[e] = acc;
        acc += matrix[rank * total_experts + e];
      }
    }
    s_chunk[threadIdx.x] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      const int v = s_chunk[t];
      s_chunk[t] = acc;
      acc += v;
    }
    s_sent = acc;
  }
  __syncthreads();
  for (int i = 0; i < per_thread; ++i) {
    const int e = threadIdx.x * per_thread + i;
    if (e < total_experts) s_start[e] += s_chunk[threadIdx.x];
  }
  __syncthreads();
  const int64_t sent = s_sent;
  for (int64_t p = blockIdx.x; p < numel; p += gridDim.x) {
    if (p >= sent) {
      // positions past the valid ones: slots whose expert id is out of range.  Their result rows must read as zero.
      // (perm holds the sentinel there, so the slot is found from the ids: done once, by the scan below.)
      break;
    }
    const int32_t slot = perm[p];
    const int32_t e = ids[slot];
    const int j = e / experts_per_rank;
    const int64_t row = (int64_t)s_first[e] + (p - s_start[e]);
    if (row >= capacity) {  // receive area too small for this batch: dropped and reported, result row zero
      if (threadIdx.x == 0) report_ep(0xA01);
      if (own_z)
        for (int64_t c = threadIdx.x; c < z_vec_per_row; c += blockDim.x) own_z[(int64_t)slot * z_vec_per_row + c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int64_t tok = slot / top_k;
    const uint4* src = rows_in + tok * vec_per_row;
    uint4* dst = peer_rows[j] + row * vec_per_row;
    for (int64_t c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = __ldg(src + c);
    if (scales_in) {
      const float* ssrc = scales_in + tok * scales_per_row;
      float* sdst = peer_scales[j] + row * scales_per_row;
      for (int c = threadIdx.x; c < scales_per_row; c += blockDim.x) sdst[c] = __ldg(ssrc + c);
    }
    if (threadIdx.x == 0) {
      peer_weights[j][row] = weights[slot];
      peer_src[j][row] = make_int2(rank, slot);
    }
  }
  // slots with an expert id outside [0, total_experts) were never sent: zero their result rows
  if (own_z && sent < numel) {
    for (int64_t s = blockIdx.x; s < numel; s += gridDim.x) {
      const int32_t e = ids[s];
      if (e >= 0 && e < total_experts) continue;
      for (int64_t c = threadIdx.x; c < z_vec_per_row; c += blockDim.x) own_z[s * z_vec_per_row + c] = make_uint4(0, 0, 0, 0);
    }
  }
  __threadfence_system();
}

// Tables of this rank's receive area.  `sentinel` (= capacity) marks padding rows in sorted_ids.
__global__ void __launch_bounds__(256)
ep_recv_tables_kernel(const int32_t* __restrict__ matrix, int rank, int world, int total_experts, int experts_per_rank,
                      int block, int64_t capacity, const int2* __restrict__ recv_src, int64_t z_slots,
                      uint8_t* const* __restrict__ peer_z, int64_t row_bytes, int32_t* __restrict__ sorted_ids,
                      int32_t* __restrict__ expert_ids, int64_t expert_cap, int32_t* __restrict__ npp,
                      void** __restrict__ out_rows) {
  __shared__ AreaLayout L;
  build_layout(L, matrix, world, total_experts, experts_per_rank, block);
  const int e0 = rank * experts_per_rank;
  const int last = e0 + experts_per_rank - 1;
  int64_t used = (int64_t)L.base[last] + (L.total[last] + block - 1) / block * block;
  if (used > capacity) used = capacity / block * block;  // the senders dropped (and reported) the rows beyond the area
  if (blockIdx.x == 0 && threadIdx.x == 0) *npp = (int32_t)used;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < capacity; r += (int64_t)gridDim.x * blockDim.x) {
    // local expert whose segment starts at or before row r (bases ascend)
    int lo = 0, hi = experts_per_rank - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((int64_t)L.base[e0 + mid] <= r) lo = mid; else hi = mid - 1;
    }
    const int32_t base = L.base[e0 + lo], total = L.total[e0 + lo];
    const bool in_use = r < used;
    const bool valid = in_use && r < (int64_t)base + total;
    sorted_ids[r] = valid ? (int32_t)r : (int32_t)capacity;
    if (out_rows) {
      void* dst = nullptr;
      if (valid) {
        const int2 s = recv_src[r];
        const bool ok = s.x >= 0 && s.x < world && s.y >= 0 && s.y < z_slots;
        if (!ok) report_ep(0xA02);
        if (ok) dst = peer_z[s.x] + (int64_t)s.y * row_bytes;
      }
      out_rows[r] = dst;
    }
    if (r % block == 0) {
      const int64_t padded_end = (int64_t)base + (total + block - 1) / block * block;
      expert_ids[r / block] = (in_use && r < padded_end) ? lo : -1;
    }
  }
  if (blockIdx.x == 0)
    for (int64_t b = capacity / block + threadIdx.x; b < expert_cap; b += blockDim.x) expert_ids[b] = -1;
}

__global__ void __launch_bounds__(256)
ep_scatter_rows_kernel(const uint4* __restrict__ z, int64_t vec_per_row, void* const* __restrict__ out_rows,
                       const int32_t* __restrict__ npp, int64_t capacity) {
  const int64_t used = min((int64_t)*npp, capacity);
  for (int64_t r = blockIdx.x; r < used; r += gridDim.x) {
    uint4* dst = reinterpret_cast<uint4*>(out_rows[r]);
    if (!dst) continue;
    const uint4* src = z + r * vec_per_row;
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

extern "C" int fmoe_ep_expert_counts(const int32_t* topk_ids, int64_t numel, int total_experts, int32_t* counts,
                                     void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(total_experts >= 1 && total_experts <= kMaxExperts, "ep_expert_counts: need 1 <= experts <= %d", kMaxExperts);
  FMOE_REQUIRE(numel >= 0 && counts, "ep_expert_counts: bad arguments");
  auto st = (cudaStream_t)stream;
  FMOE_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * total_experts, st));
  if (numel == 0) return FMOE_OK;
  FMOE_REQUIRE(topk_ids, "ep_expert_counts: null pointer");
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(numel, 4096), 148);
  ep_expert_counts_kernel<<<grid, 1024, 0, st>>>(topk_ids, numel, total_experts, counts);
  return launch_status("ep_expert_counts_kernel");
}

namespace {
int check_layout_args(const char* who, int rank, int world, int total_experts, int experts_per_rank, int block) {
  using namespace fmoe;
  FMOE_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "%s: bad rank %d of %d", who, rank, world);
  FMOE_REQUIRE(experts_per_rank >= 1 && total_experts == experts_per_rank * world && total_experts <= kMaxExperts,
               "%s: need total_experts == experts_per_rank * world <= %d", who, kMaxExperts);
  FMOE_REQUIRE(block >= 1 && block <= 256, "%s: bad block %d", who, block);
  return FMOE_OK;
}
}  // namespace

extern "C" int fmoe_ep_dispatch_sorted(const void* rows, int64_t row_bytes, const float* row_scales, int scales_per_row,
                                       int64_t T, int top_k, const int32_t* topk_ids, const float* topk_weights,
                                       const int32_t* perm, const int32_t* matrix, int rank, int world,
                                       int total_experts, int experts_per_rank, int block, void* const* peer_rows,
                                       float* const* peer_scales, float* const* peer_weights, void* const* peer_src,
                                       int64_t capacity, void* own_z, int64_t z_row_bytes, void* stream) {
  using namespace fmoe;
  int rc = check_layout_args("ep_dispatch_sorted", rank, world, total_experts, experts_per_rank, block);
  if (rc) return rc;
  FMOE_REQUIRE(top_k >= 1 && capacity >= 0, "ep_dispatch_sorted: bad top_k / capacity");
  FMOE_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && z_row_bytes % 16 == 0, "ep_dispatch_sorted: rows must be multiples of 16 bytes");
  if (T <= 0) return FMOE_OK;
  FMOE_REQUIRE(rows && topk_ids && topk_weights && perm && matrix && peer_rows && peer_weights && peer_src,
               "ep_dispatch_sorted: null pointer");
  FMOE_REQUIRE(!row_scales || (peer_scales && scales_per_row > 0), "ep_dispatch_sorted: scales without a destination");
  FMOE_REQUIRE(aligned16(rows) && aligned16(own_z), "ep_dispatch_sorted: rows and z must be 16-byte aligned");
  const unsigned grid = (unsigned)std::min<int64_t>(T * top_k, 148 * 8);
  ep_dispatch_sorted_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)rows, row_bytes / 16, row_scales, scales_per_row, top_k, topk_ids, topk_weights, perm, T * top_k,
      matrix, rank, world, total_experts, experts_per_rank, block, (uint4* const*)peer_rows, peer_scales, peer_weights,
      (int2* const*)peer_src, capacity, (uint4*)own_z, z_row_bytes / 16);
  return launch_status("ep_dispatch_sorted_kernel");
}

extern "C" int fmoe_ep_recv_tables(const int32_t* matrix, int rank, int world, int total_experts, int experts_per_rank,
                                   int block, int64_t capacity, const void* recv_src, int64_t z_slots,
                                   void* const* peer_z, int64_t z_row_bytes, int32_t* sorted_token_ids,
                                   int32_t* expert_ids, int64_t expert_cap, int32_t* num_tokens_post_padded,
                                   void** out_rows, void* stream) {
  using namespace fmoe;
  int rc = check_layout_args("ep_recv_tables", rank, world, total_experts, experts_per_rank, block);
  if (rc) return rc;
  FMOE_REQUIRE(capacity >= 0 && capacity < (1ll << 31) && capacity % block == 0, "ep_recv_tables: capacity must be a multiple of the block below 2^31");
  FMOE_REQUIRE(matrix && sorted_token_ids && expert_ids && num_tokens_post_padded && expert_cap >= capacity / block,
               "ep_recv_tables: null pointer or expert_ids too short");
  if (out_rows)
    FMOE_REQUIRE(recv_src && peer_z && z_row_bytes > 0 && z_row_bytes % 16 == 0 && z_slots >= 0,
                 "ep_recv_tables: out_rows needs recv_src, peer_z and a row size that is a multiple of 16 bytes");
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div<int64_t>(capacity, 1024), 148 * 2));
  ep_recv_tables_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(matrix, rank, world, total_experts, experts_per_rank, block,
                                                              capacity, (const int2*)recv_src, z_slots,
                                                              (uint8_t* const*)peer_z, z_row_bytes, sorted_token_ids,
                                                              expert_ids, expert_cap, num_tokens_post_padded, out_rows);
  return launch_status("ep_recv_tables_kernel");
}

extern "C" int fmoe_ep_scatter_rows(const void* z_rows, int64_t row_bytes, void* const* out_rows,
                                    const int32_t* num_rows_dev, int64_t capacity, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "ep_scatter_rows: row size must be a multiple of 16 bytes");
  if (capacity <= 0) return FMOE_OK;
  FMOE_REQUIRE(z_rows && out_rows && num_rows_dev && aligned16(z_rows), "ep_scatter_rows: null or misaligned pointer");
  const unsigned grid = (unsigned)std::min<int64_t>(capacity, 148 * 8);
  ep_scatter_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)z_rows, row_bytes / 16, out_rows,
                                                                num_rows_dev, capacity);
  return launch_status("ep_scatter_rows_kernel");
}
