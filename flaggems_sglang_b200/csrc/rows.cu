// Row-wise helper kernels around the grouped GEMMs (all HBM-bound, 16-byte accesses):
//   fmoe_quant_fp8_group128 : per-row, per-128-channel e4m3 quantisation (+ optional row gather)
//   fmoe_gather_rows        : copy rows into the padded expert-sorted order
//   fmoe_moe_sum            : out[t] = sum_j z[t,j], optional post-scale
#include "common.cuh"

namespace fmoe {
namespace {

// Source row of output position p: p itself without a map; with a map, the map's entry divided by map_div,
// or p when map_div is 0 (the map then only marks padding).  -1 = padding position.
__device__ __forceinline__ int64_t mapped_row(const int32_t* row_map, int map_div, int64_t sentinel, int64_t p) {
  if (!row_map) return p;
  int32_t s = row_map[p];
  if (s < 0 || (int64_t)s >= sentinel) return -1;
  return map_div ? s / map_div : p;
}


// The work is the flat list of (output row, 128-channel group) items; 16 lanes own one item: each lane loads
// 8 consecutive channels (16 bytes of bf16, 32 of fp32) and writes 8 bytes.  A 16-lane team walks the list with
// the grid's team count as stride and loads kIlp items before it reduces any, so that short rows (few groups)
// keep as many loads in flight as long ones.  Row and group of an item advance by a fixed step: no division
// inside the loop.
template <typename InT>
__global__ void __launch_bounds__(256)
quant_group128_kernel(const InT* __restrict__ x, int64_t rows_out, int64_t K, const int32_t* __restrict__ row_map,
                      int map_div, int64_t sentinel, const int32_t* __restrict__ num_rows_dev,
                      uint8_t* __restrict__ q, float* __restrict__ scale) {
  pdl_entry();
  constexpr int kIlp = 4;
  const int sub = threadIdx.x & 15;  // lane inside the 16-lane team
  const unsigned hmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
  const int groups = (int)(K / 128);
  const int64_t limit = num_rows_dev ? min((int64_t)*num_rows_dev, rows_out) : rows_out;
  const int64_t teams = (int64_t)gridDim.x * 16;
  const int64_t team = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
  const int64_t step_p = teams / groups;
  const int step_g = (int)(teams % groups);
  int64_t p = team / groups;  // item of this team: (row p, group g); the next one is `teams` items further
  int g = (int)(team % groups);
  while (p < limit) {
    float v[kIlp][8];
    int64_t pu[kIlp];
    int gu[kIlp];
    bool real[kIlp];
#pragma unroll
    for (int u = 0; u < kIlp; ++u) {
      pu[u] = p;
      gu[u] = g;
      real[u] = false;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      if (p < limit) {
        const int64_t r = mapped_row(row_map, map_div, sentinel, p);
        real[u] = r >= 0;
        if (r >= 0) {
          const InT* src = x + r * K + g * 128 + sub * 8;
          if constexpr (sizeof(InT) == 4) {
            float4 f0 = __ldg(reinterpret_cast<const float4*>(src));
            float4 f1 = __ldg(reinterpret_cast<const float4*>(src) + 1);
            v[u][0] = f0.x; v[u][1] = f0.y; v[u][2] = f0.z; v[u][3] = f0.w;
            v[u][4] = f1.x; v[u][5] = f1.y; v[u][6] = f1.z; v[u][7] = f1.w;
          } else {
            uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[u][2 * i] = __low2float(h[i]);
              v[u][2 * i + 1] = __high2float(h[i]);
            }
          }
        }
      }
      p += step_p;
      g += step_g;
      if (g >= groups) {
        g -= groups;
        ++p;
      }
    }
#pragma unroll
    for (int u = 0; u < kIlp; ++u) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[u][i]));
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(hmask, amax, off));
      if (pu[u] >= limit) continue;  // uniform over the 16 lanes of the team
      uint2* dst = reinterpret_cast<uint2*>(q + pu[u] * K + (int64_t)gu[u] * 128 + sub * 8);
      if (!real[u]) {  // padding position: zeros with a unit scale
        *dst = make_uint2(0, 0);
        if (sub == 0) scale[pu[u] * groups + gu[u]] = 1.0f;
        continue;
      }
      const float s = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
      uint32_t lo = 0, hi = 0;
      if (amax <= 3.0e38f) {
        const float r = __frcp_rn(s);
        float qv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[i] = div_by_shared(v[u][i], s, r);
        // two values per conversion instruction (low byte = first value)
        auto pair = [](float a, float b) {
          return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        };
        lo = pair(qv[0], qv[1]) | (pair(qv[2], qv[3]) << 16);
        hi = pair(qv[4], qv[5]) | (pair(qv[6], qv[7]) << 16);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          lo |= (uint32_t)f32_to_e4m3_bits(__fdiv_rn(v[u][i], s)) << (8 * i);
          hi |= (uint32_t)f32_to_e4m3_bits(__fdiv_rn(v[u][4 + i], s)) << (8 * i);
        }
      }
      *dst = make_uint2(lo, hi);
      if (sub == 0) scale[pu[u] * groups + gu[u]] = s;
    }
  }
}

// Per-token dynamic quantisation to e4m3 with ONE scale per row (the activation side of per-channel w8a8).  A team of
// TEAM threads (a warp for rows up to 4096 channels, the whole CTA above) owns an output row and holds it in
// registers between the amax pass and the conversion: VECS 16-byte vectors per thread.  scale = max(amax / 448,
// 1 / (448 * 512)), q = rne(x / scale) saturated: the rule of vLLM's dynamic per-token quantiser.
template <int TEAM, int VECS>
__global__ void __launch_bounds__(256)
quant_row_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows_out, int64_t K, const int32_t* __restrict__ row_map,
                 int map_div, int64_t sentinel, const int32_t* __restrict__ num_rows_dev, uint8_t* __restrict__ q,
                 float* __restrict__ scale) {
  pdl_entry();
  __shared__ float s_max[8];
  constexpr int kTeams = 256 / TEAM;
  const int lane = threadIdx.x % TEAM;
  const int64_t limit = num_rows_dev ? min((int64_t)*num_rows_dev, rows_out) : rows_out;
  const int vecs = (int)(K / 8);  // 16-byte vectors per row
  // p is the same for all threads of a team (TEAM == 256: of the CTA, so the __syncthreads below are uniform)
  for (int64_t p = (int64_t)blockIdx.x * kTeams + threadIdx.x / TEAM; p < limit; p += (int64_t)gridDim.x * kTeams) {
    const int64_t r = mapped_row(row_map, map_div, sentinel, p);
    uint2* dst = reinterpret_cast<uint2*>(q + p * K);
    if (r < 0) {  // padding position: zeros with a unit scale
      for (int c = lane; c < vecs; c += TEAM) dst[c] = make_uint2(0, 0);
      if (lane == 0) scale[p] = 1.0f;
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + r * K);
    uint4 raw[VECS];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const int c = lane + i * TEAM;
      raw[i] = make_uint4(0, 0, 0, 0);
      if (c < vecs) {
        raw[i] = __ldg(src + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(__low2float(h[j])), fabsf(__high2float(h[j]))));
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if constexpr (TEAM == 256) {
      __syncthreads();  // s_max of the previous row has been read by everyone
      if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = s_max[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_max[w]);
    }
    const float s = fmaxf(__fdiv_rn(amax, 448.0f), 1.0f / (448.0f * 512.0f));
    const float rcp = __frcp_rn(s);
    const bool finite = amax <= 3.0e38f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const int c = lane + i * TEAM;
      if (c >= vecs) continue;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
      float v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __low2float(h[j]);
        v[2 * j + 1] = __high2float(h[j]);
      }
      uint32_t lo = 0, hi = 0;
      if (finite) {
        float qv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) qv[j] = div_by_shared(v[j], s, rcp);
        auto pair = [](float a, float b) {
          return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        };
        lo = pair(qv[0], qv[1]) | (pair(qv[2], qv[3]) << 16);
        hi = pair(qv[4], qv[5]) | (pair(qv[6], qv[7]) << 16);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo |= (uint32_t)f32_to_e4m3_bits(__fdiv_rn(v[j], s)) << (8 * j);
          hi |= (uint32_t)f32_to_e4m3_bits(__fdiv_rn(v[4 + j], s)) << (8 * j);
        }
      }
      dst[c] = make_uint2(lo, hi);
    }
    if (lane == 0) scale[p] = s;
  }
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, int64_t rows_out, int64_t vec_per_row,
                   const int32_t* __restrict__ row_map, int map_div, int64_t sentinel,
                   const int32_t* __restrict__ num_rows_dev, uint4* __restrict__ out) {
  pdl_entry();
  const int64_t limit = num_rows_dev ? min((int64_t)*num_rows_dev, rows_out) : rows_out;
  for (int64_t p = blockIdx.x; p < limit; p += gridDim.x) {
    const int64_t r = mapped_row(row_map, map_div, sentinel, p);
    for (int64_t c = threadIdx.x; c < vec_per_row; c += blockDim.x)
      out[p * vec_per_row + c] = (r >= 0) ? __ldg(x + r * vec_per_row + c) : make_uint4(0, 0, 0, 0);
  }
}

// each thread owns 8 bf16 (or 4 f32) columns of one token and adds the k slots in order
template <typename T>
__global__ void __launch_bounds__(256)
moe_sum_kernel(const T* __restrict__ z, int64_t Tn, int k, int64_t H, float scale, const T* __restrict__ addend,
               T* __restrict__ out) {
  pdl_entry();
  constexpr int V = 16 / sizeof(T);
  const int64_t vec_per_row = H / V;
  const int64_t total = Tn * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec_per_row, c = i % vec_per_row;
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    for (int j = 0; j < k; ++j) {
      uint4 raw = __ldg(reinterpret_cast<const uint4*>(z + ((t * k + j) * H)) + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] += to_f32(e[v]);
    }
    uint4 res;
    T* o = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      T r = from_f32<T>(acc[v]);
      if (scale != 1.0f) r = from_f32<T>(to_f32(r) * scale);
      o[v] = r;
    }
    if (addend) {  // e.g. the shared expert's output: one more rounded add, as the separate `+=` would do
      uint4 raw = __ldg(reinterpret_cast<const uint4*>(addend + t * H) + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int v = 0; v < V; ++v) o[v] = from_f32<T>(to_f32(o[v]) + to_f32(e[v]));
    }
    reinterpret_cast<uint4*>(out + t * H)[c] = res;
  }
}

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_quant_fp8_group128(const void* x, int in_dtype, int64_t rows_out, int64_t K,
                                       const int32_t* row_map, int map_div, int64_t map_sentinel,
                                       const int32_t* num_rows_dev, void* q, float* scale, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(K > 0 && K % 128 == 0, "quant_fp8_group128: K must be a positive multiple of 128 (got %lld)", (long long)K);
  FMOE_REQUIRE(in_dtype == FMOE_BF16 || in_dtype == FMOE_F32, "quant_fp8_group128: in_dtype must be bf16 or f32");
  FMOE_REQUIRE(!row_map || map_div >= 0, "quant_fp8_group128: map_div must be >= 0");
  if (rows_out <= 0) return FMOE_OK;
  FMOE_REQUIRE(x && q && scale, "quant_fp8_group128: null pointer");
  FMOE_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp8_group128: misaligned pointer");
  // 16 teams per CTA, 4 items per team and pass
  unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div<int64_t>(rows_out * (K / 128), 64), 148 * 8));
  auto st = (cudaStream_t)stream;
  if (in_dtype == FMOE_BF16)
    launch_pdl(quant_group128_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, rows_out, K,
               row_map, map_div, map_sentinel, num_rows_dev, (uint8_t*)q, scale);
  else
    launch_pdl(quant_group128_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)x, rows_out, K, row_map,
               map_div, map_sentinel, num_rows_dev, (uint8_t*)q, scale);
  return launch_status("quant_group128_kernel");
}

extern "C" int fmoe_quant_fp8_per_token(const void* x, int in_dtype, int64_t rows_out, int64_t K,
                                        const int32_t* row_map, int map_div, int64_t map_sentinel,
                                        const int32_t* num_rows_dev, void* q, float* scale, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(K > 0 && K % 8 == 0 && K <= 16384, "quant_fp8_per_token: K must be a multiple of 8 up to 16384 (got %lld)",
               (long long)K);
  FMOE_REQUIRE(in_dtype == FMOE_BF16, "quant_fp8_per_token: in_dtype must be bf16");
  FMOE_REQUIRE(!row_map || map_div >= 0, "quant_fp8_per_token: map_div must be >= 0");
  if (rows_out <= 0) return FMOE_OK;
  FMOE_REQUIRE(x && q && scale, "quant_fp8_per_token: null pointer");
  FMOE_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, "quant_fp8_per_token: misaligned pointer");
  auto go = [&](auto kernel, int teams) {
    unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(rows_out, teams), 148 * 8);
    launch_pdl(kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, rows_out, K, row_map,
               map_div, map_sentinel, num_rows_dev, (uint8_t*)q, scale);
  };
  if (K <= 2048) go(quant_row_kernel<32, 8>, 8);         // a warp per row, 8 rows per CTA
  else if (K <= 4096) go(quant_row_kernel<32, 16>, 8);
  else go(quant_row_kernel<256, 8>, 1);                  // a CTA per row
  return launch_status("quant_row_kernel");
}

extern "C" int fmoe_gather_rows(const void* x, int elem_bytes, int64_t rows_out, int64_t K,
                                const int32_t* row_map, int map_div, int64_t map_sentinel,
                                const int32_t* num_rows_dev, void* out, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 1, "gather_rows: elem_bytes must be 1, 2 or 4");
  FMOE_REQUIRE(K > 0 && (K * elem_bytes) % 16 == 0, "gather_rows: row size must be a multiple of 16 bytes");
  FMOE_REQUIRE(row_map && map_div >= 1, "gather_rows: row_map required");
  if (rows_out <= 0) return FMOE_OK;
  FMOE_REQUIRE(x && out && aligned16(x) && aligned16(out), "gather_rows: null or misaligned pointer");
  unsigned grid = (unsigned)std::min<int64_t>(rows_out, 148 * 8);
  launch_pdl(gather_rows_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const uint4*)x, rows_out,
             K * elem_bytes / 16, row_map, map_div, map_sentinel, num_rows_dev, (uint4*)out);
  return launch_status("gather_rows_kernel");
}

extern "C" int fmoe_moe_sum(const void* z, int dtype, int64_t T, int k, int64_t H, float scale, void* out,
                            void* stream) {
  return fmoe_moe_sum_add(z, dtype, T, k, H, scale, nullptr, out, stream);
}

extern "C" int fmoe_moe_sum_add(const void* z, int dtype, int64_t T, int k, int64_t H, float scale,
                                const void* addend, void* out, void* stream) {
  using namespace fmoe;
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "moe_sum: dtype must be bf16 or f32");
  const int eb = dtype == FMOE_BF16 ? 2 : 4;
  FMOE_REQUIRE(k >= 1 && H > 0 && (H * eb) % 16 == 0, "moe_sum: need k >= 1 and H*elem %% 16 == 0");
  if (T <= 0) return FMOE_OK;
  FMOE_REQUIRE(z && out && aligned16(z) && aligned16(out) && aligned16(addend), "moe_sum: null or misaligned pointer");
  int64_t total = T * (H * eb / 16);
  unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(total, 256), 148 * 16);
  auto st = (cudaStream_t)stream;
  if (dtype == FMOE_BF16)
    launch_pdl(moe_sum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)z, T, k, H, scale,
               (const __nv_bfloat16*)addend, (__nv_bfloat16*)out);
  else
    launch_pdl(moe_sum_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)z, T, k, H, scale,
               (const float*)addend, (float*)out);
  return launch_status("moe_sum_kernel");
}
