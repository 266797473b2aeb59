// Quantisers of the quantized-linear path (no counterpart kernel in the reference;
// the API shape follows its proposed QuantOps, docs/backend-int8-quantization-decision.md:88-94).
//
//   int8, symmetric, one scale per row:   scale = amax(row) / 127,  q = rne(x / scale), |q| <= 127
//   FP8 E4M3, one scale per tensor:       scale = amax(x) / 448,    q = e4m3_rne_sat(x / scale)
//
// A row (or tensor) whose amax is 0 gets scale 0 and all-zero codes.  The division
// is the IEEE f32 division, so the CPU restatement produces the same bytes.
#include "kernels.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include <cuda_fp8.h>

namespace b200 {
namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Max over the CTA; every thread receives the result.
__device__ __forceinline__ float block_max(float v, float* scratch) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < (blockDim.x >> 5)) ? scratch[lane] : 0.0f;
    r = warp_max(r);
    return r;
}


__global__ void __launch_bounds__(kRowThreads)
quantize_i8_per_row_kernel(const float* __restrict__ x, int64_t cols, int8_t* __restrict__ q, float* __restrict__ scale) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const float* xr = x + row * cols;
    int8_t* qr = q + row * cols;
    float amax = 0.0f;
    const bool vec = (cols & 3) == 0;
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        for (int64_t i = threadIdx.x; i < cols / 4; i += kRowThreads) {
            const float4 v = x4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int64_t i = threadIdx.x; i < cols; i += kRowThreads) amax = fmaxf(amax, fabsf(xr[i]));
    }
    amax = block_max(amax, scratch);
    const float s = amax / 127.0f;
    if (threadIdx.x == 0) scale[row] = s;
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        uint32_t* q4 = reinterpret_cast<uint32_t*>(qr);
        for (int64_t i = threadIdx.x; i < cols / 4; i += kRowThreads) {
            const float4 v = x4[i];
            const uint32_t b0 = static_cast<uint32_t>(quant_i8(v.x, s)) & 0xFFu;
            const uint32_t b1 = static_cast<uint32_t>(quant_i8(v.y, s)) & 0xFFu;
            const uint32_t b2 = static_cast<uint32_t>(quant_i8(v.z, s)) & 0xFFu;
            const uint32_t b3 = static_cast<uint32_t>(quant_i8(v.w, s)) & 0xFFu;
            q4[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
    } else {
        for (int64_t i = threadIdx.x; i < cols; i += kRowThreads) qr[i] = static_cast<int8_t>(quant_i8(xr[i], s));
    }
}

__global__ void dequantize_i8_per_row_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale,
                                             int64_t rows, int64_t cols, float* __restrict__ x) {
    const int64_t n = rows * cols;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        x[i] = static_cast<float>(q[i]) * scale[i / cols];
    }
}

// amax over a tensor: max is order-independent, so an atomic on the bit pattern of a
// non-negative float is deterministic.
__global__ void amax_kernel(const float* __restrict__ x, int64_t n, uint32_t* __restrict__ amax_bits) {
    __shared__ float scratch[32];
    float m = 0.0f;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        m = fmaxf(m, fabsf(x[i]));
    m = block_max(m, scratch);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
}

__global__ void fp8_scale_kernel(const uint32_t* __restrict__ amax_bits, float* __restrict__ scale) {
    scale[0] = __uint_as_float(amax_bits[0]) / 448.0f;
}

__global__ void fp8_encode_kernel(const float* __restrict__ x, int64_t n, const float* __restrict__ scale,
                                  uint8_t* __restrict__ q) {
    const float s = scale[0];
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const float v = (s == 0.0f) ? 0.0f : x[i] / s;
        q[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
    }
}

int grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = int64_t(current_sm_count()) * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

}  // namespace

cudaError_t quantize_i8_per_row(const float* x, int64_t rows, int64_t cols, int8_t* q, float* scale, cudaStream_t s) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    quantize_i8_per_row_kernel<<<static_cast<unsigned>(rows), kRowThreads, 0, s>>>(x, cols, q, scale);
    return cudaGetLastError();
}

cudaError_t dequantize_i8_per_row(const int8_t* q, const float* scale, int64_t rows, int64_t cols, float* x,
                                  cudaStream_t s) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    dequantize_i8_per_row_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(q, scale, rows, cols, x);
    return cudaGetLastError();
}

cudaError_t quantize_fp8_per_tensor(const float* x, int64_t n, uint8_t* q, float* scale, uint32_t* amax_scratch,
                                    cudaStream_t s) {
    cudaError_t e = cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    if (n > 0) amax_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, n, amax_scratch);
    fp8_scale_kernel<<<1, 1, 0, s>>>(amax_scratch, scale);
    if (n > 0) fp8_encode_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, n, scale, q);
    return cudaGetLastError();
}

}  // namespace b200
