// moe_align_block_size: histogram -> scan -> stable scatter, one CTA.
//
// The slots [0, numel) are split into one contiguous chunk per warp.  Each warp
// counts its chunk per expert, a scan over (expert, warp) turns the counts into
// the first output position of every (warp, expert) pair, and a second pass over
// the chunk places each slot at base + (its rank among the equal ids seen so
// far), which keeps slots of an expert in ascending order.  The ranks inside a
// group of 32 slots come from __match_any_sync.
#include "common.cuh"

namespace fmoe {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;

__global__ void __launch_bounds__(kThreads)
moe_align_kernel(const int32_t* __restrict__ topk_ids, int numel, int E, int block,
                 int32_t* __restrict__ sorted_ids, int sorted_cap, int32_t* __restrict__ expert_ids,
                 int expert_cap, int32_t* __restrict__ num_post_pad) {
  pdl_entry();
  extern __shared__ int s_mem[];
  int* s_cnt = s_mem;                  // [kWarps][E] counts, then running output positions
  int* s_total = s_mem + kWarps * E;   // [E] per-expert count
  int* s_start = s_total + E;          // [E+1] padded start of each expert
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i < kWarps * E; i += kThreads) s_cnt[i] = 0;
  for (int i = tid; i < sorted_cap; i += kThreads) sorted_ids[i] = numel;
  __syncthreads();

  const int chunk = ceil_div(ceil_div(numel, kWarps), 32) * 32;  // multiple of 32 per warp
  const int lo = min(warp * chunk, numel), hi = min(lo + chunk, numel);

  // pass 1: per-warp histogram
  for (int base = lo; base < hi; base += 32) {
    int s = base + lane;
    int e = (s < hi) ? topk_ids[s] : -1;
    bool ok = (e >= 0 && e < E);
    unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok && (__ffs(peers) - 1) == lane) s_cnt[warp * E + e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();

  // scan over warps for each expert: s_cnt[w][e] <- number of slots of e in warps < w
  for (int e = tid; e < E; e += kThreads) {
    int run = 0;
    for (int w = 0; w < kWarps; ++w) {
      int c = s_cnt[w * E + e];
      s_cnt[w * E + e] = run;
      run += c;
    }
    s_total[e] = run;
  }
  __syncthreads();

  // padded exclusive scan over experts (E <= 1024: warp 0, 32 experts per step)
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < E; base += 32) {
      int e = base + lane;
      int padded = (e < E) ? ceil_div(s_total[e], block) * block : 0;
      int incl = padded;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      if (e < E) s_start[e] = carry + incl - padded;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      s_start[E] = carry;
      num_post_pad[0] = carry;
    }
  }
  __syncthreads();

  // block -> expert map (-1 after the used blocks)
  const int used_blocks = s_start[E] / block;
  for (int e = tid; e < E; e += kThreads) {
    int b0 = s_start[e] / block, b1 = s_start[e + 1] / block;
    for (int b = b0; b < b1 && b < expert_cap; ++b) expert_ids[b] = e;
  }
  for (int b = used_blocks + tid; b < expert_cap; b += kThreads) expert_ids[b] = -1;

  // pass 2: stable scatter
  for (int base = lo; base < hi; base += 32) {
    int s = base + lane;
    int e = (s < hi) ? topk_ids[s] : -1;
    bool ok = (e >= 0 && e < E);
    unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok) {
      int rank = __popc(peers & ((1u << lane) - 1u));
      int pos = s_start[e] + s_cnt[warp * E + e] + rank;
      if (pos < sorted_cap) sorted_ids[pos] = s;
    }
    __syncwarp();
    if (ok && (__ffs(peers) - 1) == lane) s_cnt[warp * E + e] += __popc(peers);
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------
// Multi-CTA variant for large inputs: the slots are cut into chunks of kChunk, one CTA per chunk.
//   count   : per-chunk histogram -> cnt[chunk][E]; sentinel fill of sorted_token_ids
//   scan    : one CTA: exclusive scan over chunks per expert, padded starts, expert_ids, total
//   scatter : every CTA redoes its chunk's per-warp histogram and places its slots (stable)
// cnt lives in caller scratch (chunks * E ints).
// ---------------------------------------------------------------------------------------------
constexpr int kChunk = 4096;

__global__ void __launch_bounds__(kThreads)
align_count_kernel(const int32_t* __restrict__ topk_ids, int numel, int E, int32_t* __restrict__ sorted_ids,
                   int sorted_cap, int32_t* __restrict__ cnt) {
  extern __shared__ int s_mem[];  // [E]
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += kThreads) s_mem[e] = 0;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + tid; i < sorted_cap; i += (int64_t)gridDim.x * kThreads)
    sorted_ids[i] = numel;
  __syncthreads();
  const int lo = blockIdx.x * kChunk, hi = min(lo + kChunk, numel);
  for (int s = lo + tid; s < hi; s += kThreads) {
    int e = topk_ids[s];
    if (e >= 0 && e < E) atomicAdd(&s_mem[e], 1);
  }
  __syncthreads();
  for (int e = tid; e < E; e += kThreads) cnt[blockIdx.x * E + e] = s_mem[e];
}

__global__ void __launch_bounds__(kThreads)
align_scan_kernel(int chunks, int E, int block, int32_t* __restrict__ cnt, int32_t* __restrict__ expert_ids,
                  int expert_cap, int32_t* __restrict__ num_post_pad) {
  extern __shared__ int s_mem[];
  int* s_total = s_mem;      // [E]
  int* s_start = s_mem + E;  // [E+1]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += kThreads) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      int v = cnt[c * E + e];
      cnt[c * E + e] = run;  // slots of e in earlier chunks
      run += v;
    }
    s_total[e] = run;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < E; base += 32) {
      int e = base + lane;
      int padded = (e < E) ? ceil_div(s_total[e], block) * block : 0;
      int incl = padded;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      if (e < E) s_start[e] = carry + incl - padded;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      s_start[E] = carry;
      num_post_pad[0] = carry;
    }
  }
  __syncthreads();
  const int used_blocks = s_start[E] / block;
  for (int e = tid; e < E; e += kThreads) {
    int b0 = s_start[e] / block, b1 = s_start[e + 1] / block;
    for (int b = b0; b < b1 && b < expert_cap; ++b) expert_ids[b] = e;
    for (int c = 0; c < chunks; ++c) cnt[c * E + e] += s_start[e];  // absolute first position per (chunk, expert)
  }
  for (int b = used_blocks + tid; b < expert_cap; b += kThreads) expert_ids[b] = -1;
}

__global__ void __launch_bounds__(kThreads)
align_scatter_kernel(const int32_t* __restrict__ topk_ids, int numel, int E, const int32_t* __restrict__ cnt,
                     int32_t* __restrict__ sorted_ids, int sorted_cap) {
  extern __shared__ int s_mem[];  // [kWarps][E] per-warp counts -> running positions
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kWarps * E; i += kThreads) s_mem[i] = 0;
  __syncthreads();
  constexpr int per_warp = kChunk / kWarps;  // 128 contiguous slots per warp
  const int lo = min(blockIdx.x * kChunk + warp * per_warp, numel), hi = min(lo + per_warp, numel);
  for (int base = lo; base < hi; base += 32) {
    int s = base + lane;
    int e = (s < hi) ? topk_ids[s] : -1;
    bool ok = (e >= 0 && e < E);
    unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok && (__ffs(peers) - 1) == lane) s_mem[warp * E + e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  for (int e = tid; e < E; e += kThreads) {
    int run = cnt[blockIdx.x * E + e];
    for (int w = 0; w < kWarps; ++w) {
      int c = s_mem[w * E + e];
      s_mem[w * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int base = lo; base < hi; base += 32) {
    int s = base + lane;
    int e = (s < hi) ? topk_ids[s] : -1;
    bool ok = (e >= 0 && e < E);
    unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok) {
      int pos = s_mem[warp * E + e] + __popc(peers & ((1u << lane) - 1u));
      if (pos < sorted_cap) sorted_ids[pos] = s;
    }
    __syncwarp();
    if (ok && (__ffs(peers) - 1) == lane) s_mem[warp * E + e] += __popc(peers);
    __syncwarp();
  }
}

}  // namespace
}  // namespace fmoe

extern "C" int64_t fmoe_moe_align_workspace_bytes(int64_t numel, int E) {
  return fmoe::ceil_div<int64_t>(numel > 0 ? numel : 1, fmoe::kChunk) * E * (int64_t)sizeof(int32_t);
}

extern "C" int fmoe_moe_align_block_size_ws(const int32_t* topk_ids, int64_t numel, int E, int block,
                                            int32_t* sorted_token_ids, int64_t sorted_cap, int32_t* expert_ids,
                                            int64_t expert_cap, int32_t* num_tokens_post_padded, void* workspace,
                                            int64_t workspace_bytes, void* stream) {
  using namespace fmoe;
  // small inputs, or no scratch: the single-CTA kernel
  if (numel < 2 * kChunk || !workspace)
    return fmoe_moe_align_block_size(topk_ids, numel, E, block, sorted_token_ids, sorted_cap, expert_ids, expert_cap,
                                     num_tokens_post_padded, stream);
  FMOE_REQUIRE(E >= 1 && E <= 1024, "moe_align_block_size: need 1 <= E <= 1024 (got %d)", E);
  FMOE_REQUIRE(block >= 1, "moe_align_block_size: block must be >= 1 (got %d)", block);
  FMOE_REQUIRE(numel < (1ll << 30), "moe_align_block_size: numel out of range");
  const int64_t need = numel + (numel < E ? numel : (int64_t)E) * (block - 1);
  FMOE_REQUIRE(sorted_cap >= need && sorted_cap < (1ll << 31), "moe_align_block_size: sorted_token_ids too small (%lld < %lld)",
               (long long)sorted_cap, (long long)need);
  FMOE_REQUIRE(expert_cap >= ceil_div<int64_t>(sorted_cap, block), "moe_align_block_size: expert_ids too small");
  FMOE_REQUIRE(sorted_token_ids && expert_ids && num_tokens_post_padded && topk_ids, "moe_align_block_size: null pointer");
  FMOE_REQUIRE(workspace_bytes >= fmoe_moe_align_workspace_bytes(numel, E), "moe_align_block_size: workspace too small");
  const int chunks = (int)ceil_div<int64_t>(numel, kChunk);
  auto st = (cudaStream_t)stream;
  int32_t* cnt = static_cast<int32_t*>(workspace);
  align_count_kernel<<<chunks, kThreads, E * sizeof(int), st>>>(topk_ids, (int)numel, E, sorted_token_ids, (int)sorted_cap, cnt);
  int rc = launch_status("align_count_kernel");
  if (rc) return rc;
  align_scan_kernel<<<1, kThreads, (2 * E + 1) * sizeof(int), st>>>(chunks, E, block, cnt, expert_ids, (int)expert_cap,
                                                                   num_tokens_post_padded);
  rc = launch_status("align_scan_kernel");
  if (rc) return rc;
  size_t smem = (size_t)kWarps * E * sizeof(int);
  if (smem > 48 * 1024)
    FMOE_CUDA_OK(cudaFuncSetAttribute(align_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  align_scatter_kernel<<<chunks, kThreads, smem, st>>>(topk_ids, (int)numel, E, cnt, sorted_token_ids, (int)sorted_cap);
  return launch_status("align_scatter_kernel");
}

extern "C" int fmoe_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int E, int block,
                                         int32_t* sorted_token_ids, int64_t sorted_cap,
                                         int32_t* expert_ids, int64_t expert_cap,
                                         int32_t* num_tokens_post_padded, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(E >= 1 && E <= 1024, "moe_align_block_size: need 1 <= E <= 1024 (got %d)", E);
  FMOE_REQUIRE(block >= 1, "moe_align_block_size: block must be >= 1 (got %d)", block);
  FMOE_REQUIRE(numel >= 0 && numel < (1ll << 30), "moe_align_block_size: numel out of range");
  // worst case: every non-empty expert wastes block-1 positions
  const int64_t need = numel + (numel < E ? numel : (int64_t)E) * (block - 1);
  FMOE_REQUIRE(sorted_cap >= need, "moe_align_block_size: sorted_token_ids too small (%lld < %lld)",
               (long long)sorted_cap, (long long)need);
  FMOE_REQUIRE(sorted_cap < (1ll << 31), "moe_align_block_size: sorted_cap out of range");
  FMOE_REQUIRE(expert_cap >= ceil_div<int64_t>(sorted_cap, block),
               "moe_align_block_size: expert_ids too small (%lld < %lld)", (long long)expert_cap,
               (long long)ceil_div<int64_t>(sorted_cap, block));
  FMOE_REQUIRE(sorted_token_ids && expert_ids && num_tokens_post_padded && (topk_ids || numel == 0),
               "moe_align_block_size: null pointer");
  size_t smem = ((size_t)kWarps * E + 2 * (size_t)E + 1) * sizeof(int);
  if (smem > 48 * 1024)
    FMOE_CUDA_OK(cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_pdl(moe_align_kernel, dim3(1), dim3(kThreads), smem, (cudaStream_t)stream, topk_ids, (int)numel, E, block,
             sorted_token_ids, (int)sorted_cap, expert_ids, (int)expert_cap, num_tokens_post_padded);
  return launch_status("moe_align_kernel");
}
