// Host-callable launchers of the non-GEMM kernels (quantisers, paged KV, decoder glue).
// All of them only enqueue work on the given stream.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---- quant.cu
cudaError_t quantize_i8_per_row(const float* x, int64_t rows, int64_t cols, int8_t* q, float* scale, cudaStream_t s);
cudaError_t dequantize_i8_per_row(const int8_t* q, const float* scale, int64_t rows, int64_t cols, float* x,
                                  cudaStream_t s);
// `amax_scratch` is one uint32 of device memory owned by the context.
cudaError_t quantize_fp8_per_tensor(const float* x, int64_t n, uint8_t* q, float* scale, uint32_t* amax_scratch,
                                    cudaStream_t s);

}  // namespace b200
