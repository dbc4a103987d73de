// Internal interface between the C-ABI entry points (api.cu) and the three
// grouped-GEMM kernel families.
#pragma once
#include "common.cuh"

namespace fmoe {

using GemmParams = fmoe_gemm_args;

// gated = true : gemm1, w has 2*n rows per expert (gate rows then up rows), output
//                silu(gate)*up of width n, written at the sorted position p.
// gated = false: gemm2, w has n rows per expert, output written at row slot(p).
int gemm_simt(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_stream(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_tcgen05(const GemmParams& p, bool gated, cudaStream_t st);
int gemm_tcgen05_fp8(const GemmParams& p, bool gated, cudaStream_t st);

// true when the variant can run these arguments (shape / alignment / dtype rules)
bool gemm_stream_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_supports(const GemmParams& p, bool gated);
bool gemm_tcgen05_fp8_supports(const GemmParams& p, bool gated);

// device status word written by bounded waits (gemm_tcgen05.cu)
int read_and_clear_device_status(cudaStream_t st, int* status_out);

}  // namespace fmoe
