// Router kernels: one warp per token, shuffle reductions only.
//   fmoe_topk_softmax : softmax -> top-k -> renormalise
//   fmoe_topk_grouped : sigmoid + bias, group-limited top-k (DeepSeek-V3 style)
// Expert e of a token lives in lane e % 32, register e / 32 (coalesced loads).
// NaN contract: a NaN logit (or a NaN biased score) ranks as -inf, ties go to the lower index, and a softmax row
// without any logit above -inf is routed as if all its logits were equal; every id written is inside [0, E).
#include "common.cuh"

namespace fmoe {
namespace {

constexpr int kWarpsPerBlock = 4;
#define kNegInf (__int_as_float(0xff800000))

struct Best {
  float v;
  int idx;
};

// (value desc, index asc) ordering: the lower index wins a tie.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return (v > bv) || (v == bv && i < bi);
}

__device__ __forceinline__ Best warp_argmax(Best b) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, b.v, off);
    int oi = __shfl_xor_sync(0xffffffffu, b.idx, off);
    if (better(ov, oi, b.v, b.idx)) {
      b.v = ov;
      b.idx = oi;
    }
  }
  return b;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// k rounds of warp-wide argmax over the per-lane register file `key`; a taken
// entry is replaced by -inf with index INT_MAX so that it can never win again.
template <int VPT>
__device__ __forceinline__ void select_topk(float (&key)[VPT], int E, int k, int lane, int* sel_ids) {
  bool taken[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) taken[i] = (lane + 32 * i) >= E;
  for (int j = 0; j < k; ++j) {
    Best b{kNegInf, 0x7fffffff};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int e = lane + 32 * i;
      if (!taken[i] && better(key[i], e, b.v, b.idx)) {
        b.v = key[i];
        b.idx = e;
      }
    }
    b = warp_argmax(b);
    if (lane == 0) sel_ids[j] = b.idx;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (lane + 32 * i == b.idx) taken[i] = true;
  }
}

template <int VPT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
topk_softmax_kernel(const float* __restrict__ logits, int64_t T, int E, int k, int renorm,
                    float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
  pdl_entry();
  __shared__ int s_ids[kWarpsPerBlock][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  if (t >= T) return;
  const float* row = logits + t * E;
  float key[VPT];
  float mx = kNegInf;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int e = lane + 32 * i;
    const float v = (e < E) ? row[e] : kNegInf;
    key[i] = (v != v) ? kNegInf : v;  // NaN ranks as -inf
    mx = fmaxf(mx, key[i]);
  }
  mx = warp_max(mx);
  if (mx == kNegInf) {  // no logit above -inf: equal logits (uniform probabilities, experts 0..k-1)
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (lane + 32 * i < E) key[i] = 0.f;
  }
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (lane + 32 * i < E) denom += expf(key[i] - mx);
  denom = warp_sum(denom);

  select_topk<VPT>(key, E, k, lane, s_ids[warp]);
  __syncwarp();
  // lane j owns winner j
  int id = (lane < k) ? min(max(s_ids[warp][lane], 0), E - 1) : 0;
  // the winner's (sanitised) logit lives in lane id % 32, register id / 32
  float kv = kNegInf;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const float cand = __shfl_sync(0xffffffffu, key[i], id & 31);
    if (i == (id >> 5)) kv = cand;
  }
  float p = (lane < k) ? __fdiv_rn(expf(kv - mx), denom) : 0.f;
  if (renorm) {
    float s = 0.f;
    for (int j = 0; j < k; ++j) s += __shfl_sync(0xffffffffu, p, j);  // sequential, j ascending
    p = __fdiv_rn(p, s);
  }
  if (lane < k) {
    out_w[t * k + lane] = p;
    out_ids[t * k + lane] = id;
  }
}

// COOP (few tokens): one CTA per token; all its threads evaluate the fp64 sigmoids (one expert each instead of VPT in
// a row per lane), then warp 0 carries on alone.  Same arithmetic, shorter dependent chain.
template <int VPT, bool COOP>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
topk_grouped_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, int E,
                    int k, int n_group, int topk_group, int renorm, float scale,
                    float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
  pdl_entry();
  extern __shared__ float s_dyn[];  // per warp: score[E], choice[E]
  __shared__ int s_ids[kWarpsPerBlock][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = COOP ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  if (t >= T) return;
  float* s_score = s_dyn + (COOP ? (size_t)0 : (size_t)warp * 2 * E);
  float* s_choice = s_score + E;
  const float* row = logits + t * E;
  float key[VPT];
  auto scores = [&](int e, float* c_out) {
    // correctly rounded fp32 sigmoid: evaluate in fp64, round once
    const float lg = row[e];
    double z = (lg != lg) ? -INFINITY : (double)lg;  // NaN ranks as -inf (score 0)
    float s = (float)(1.0 / (1.0 + exp(-z)));
    float c = s + (bias ? bias[e] : 0.f);
    if (c != c) c = kNegInf;
    s_score[e] = s;
    s_choice[e] = c;
    *c_out = c;
  };
  if constexpr (COOP) {
    float unused;
    for (int e = threadIdx.x; e < E; e += blockDim.x) scores(e, &unused);
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int e = lane + 32 * i;
      key[i] = (e < E) ? s_choice[e] : kNegInf;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int e = lane + 32 * i;
      if (e < E) scores(e, &key[i]);
      else key[i] = kNegInf;
    }
  }
  __syncwarp();
  // group score: sum of the two largest choices of the group (lane g scans group g)
  const int gsz = E / n_group;
  float gscore = kNegInf;
  if (lane < n_group) {
    float m1 = kNegInf, m2 = kNegInf;
    for (int i = 0; i < gsz; ++i) {
      float c = s_choice[lane * gsz + ((i + lane) % gsz)];  // rotate start: spreads banks
      if (c > m1) {
        m2 = m1;
        m1 = c;
      } else if (c > m2) {
        m2 = c;
      }
    }
    gscore = (gsz >= 2) ? (m1 + m2) : m1;
    if (gscore != gscore) gscore = kNegInf;  // +inf + -inf
  }
  // keep the topk_group best groups (ties -> lower group index)
  uint32_t keep = 0;
  for (int j = 0; j < topk_group; ++j) {
    Best b{gscore, lane};
    if (lane >= n_group || ((keep >> lane) & 1u)) {
      b.v = kNegInf;
      b.idx = 0x7fffffff;
    }
    b = warp_argmax(b);
    if (b.idx < 32) keep |= 1u << b.idx;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int e = lane + 32 * i;
    if (e < E && !((keep >> (e / gsz)) & 1u)) key[i] = kNegInf;
  }
  select_topk<VPT>(key, E, k, lane, s_ids[warp]);
  __syncwarp();
  int id = (lane < k) ? min(max(s_ids[warp][lane], 0), E - 1) : 0;
  float w = (lane < k) ? s_score[id] : 0.f;
  if (renorm) {
    float s = 0.f;
    for (int j = 0; j < k; ++j) s += __shfl_sync(0xffffffffu, w, j);
    w = __fdiv_rn(w, s + 1e-20f);
  }
  w *= scale;
  if (lane < k) {
    out_w[t * k + lane] = w;
    out_ids[t * k + lane] = id;
  }
}

template <template <int> class Launcher, typename... Args>
int dispatch_vpt(int E, Args... args) {
  int vpt = ceil_div(E, 32);
  if (vpt <= 1) return Launcher<1>::run(args...);
  if (vpt <= 2) return Launcher<2>::run(args...);
  if (vpt <= 4) return Launcher<4>::run(args...);
  if (vpt <= 8) return Launcher<8>::run(args...);
  if (vpt <= 16) return Launcher<16>::run(args...);
  return Launcher<32>::run(args...);
}

template <int VPT>
struct SoftmaxLauncher {
  static int run(const float* logits, int64_t T, int E, int k, int renorm, float* w, int32_t* ids,
                 cudaStream_t st) {
    dim3 grid((unsigned)ceil_div<int64_t>(T, kWarpsPerBlock));
    launch_pdl(topk_softmax_kernel<VPT>, grid, dim3(kWarpsPerBlock * 32), 0, st, logits, T, E, k, renorm, w, ids);
    return launch_status("topk_softmax_kernel");
  }
};

template <int VPT>
struct GroupedLauncher {
  static int run(const float* logits, const float* bias, int64_t T, int E, int k, int n_group,
                 int topk_group, int renorm, float scale, float* w, int32_t* ids, cudaStream_t st) {
    size_t smem = (size_t)kWarpsPerBlock * 2 * E * sizeof(float);
    if (T <= 64) {  // decode-sized: a CTA per token shortens the chain of fp64 sigmoids (13.3 -> 8.7-9.9 us at T = 1, E = 256)
      launch_pdl(topk_grouped_kernel<VPT, true>, dim3((unsigned)T), dim3(kWarpsPerBlock * 32), smem, st, logits, bias, T, E,
                 k, n_group, topk_group, renorm, scale, w, ids);
      return launch_status("topk_grouped_kernel");
    }
    dim3 grid((unsigned)ceil_div<int64_t>(T, kWarpsPerBlock));
    launch_pdl(topk_grouped_kernel<VPT, false>, grid, dim3(kWarpsPerBlock * 32), smem, st, logits, bias, T, E, k, n_group,
               topk_group, renorm, scale, w, ids);
    return launch_status("topk_grouped_kernel");
  }
};

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_topk_softmax(const float* logits, int64_t T, int E, int k, int renormalize,
                                 float* topk_weights, int32_t* topk_ids, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(T >= 0 && E >= 1 && E <= 1024, "topk_softmax: need 1 <= E <= 1024 (got E=%d)", E);
  FMOE_REQUIRE(k >= 1 && k <= 32 && k <= E, "topk_softmax: need 1 <= k <= min(32,E) (got k=%d, E=%d)", k, E);
  if (T == 0) return FMOE_OK;
  FMOE_REQUIRE(logits && topk_weights && topk_ids, "topk_softmax: null pointer");
  return dispatch_vpt<SoftmaxLauncher>(E, logits, T, E, k, renormalize, topk_weights, topk_ids,
                                       (cudaStream_t)stream);
}

extern "C" int fmoe_topk_grouped(const float* logits, const float* bias, int64_t T, int E, int k,
                                 int n_group, int topk_group, int renormalize, float scale,
                                 float* topk_weights, int32_t* topk_ids, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(T >= 0 && E >= 1 && E <= 1024, "topk_grouped: need 1 <= E <= 1024 (got E=%d)", E);
  FMOE_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0,
               "topk_grouped: need 1 <= n_group <= 32 dividing E (got n_group=%d, E=%d)", n_group, E);
  FMOE_REQUIRE(topk_group >= 1 && topk_group <= n_group, "topk_grouped: bad topk_group=%d", topk_group);
  FMOE_REQUIRE(k >= 1 && k <= 32 && k <= topk_group * (E / n_group),
               "topk_grouped: k=%d exceeds the experts of the kept groups", k);
  if (T == 0) return FMOE_OK;
  FMOE_REQUIRE(logits && topk_weights && topk_ids, "topk_grouped: null pointer");
  return dispatch_vpt<GroupedLauncher>(E, logits, bias, T, E, k, n_group, topk_group, renormalize, scale,
                                       topk_weights, topk_ids, (cudaStream_t)stream);
}
