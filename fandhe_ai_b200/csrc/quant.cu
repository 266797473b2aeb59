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

// ---- block-scale contract (docs/int8-quant-grade-up-verification-plan.md:177-241 of the reference): blocks of 128
// values along a row, delta = pow2ceil(max(amax_block, 1e-4) / 127), q = rne(x / delta) (never clamps: |x / delta| <= 127).
constexpr int kQuantBlock = 128;

// smallest power of two >= x for a positive, finite, normal x
__device__ __forceinline__ float pow2ceil(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x7FFFFFu) == 0u ? x : __uint_as_float(((b >> 23) + 1u) << 23);
}

// One warp per (row, block): lane l holds values 4 l .. 4 l + 3 of the block.  `delta_rs` / `delta_bs` are the strides
// of the scale array per row and per block, so that it can be written as [rows, nb] or as [nb, rows].
__global__ void __launch_bounds__(256)
quantize_i8_block_pow2_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, int64_t nb, int8_t* __restrict__ q,
                              float* __restrict__ delta, int64_t delta_rs, int64_t delta_bs, uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t item = warp; item < rows * nb; item += warps) {
        const int64_t r = item / nb, b = item % nb;
        const int64_t c0 = b * kQuantBlock + 4 * lane;
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = c0 + t < cols ? x[r * cols + c0 + t] : 0.0f;
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        bool finite = isfinite(v[0]) && isfinite(v[1]) && isfinite(v[2]) && isfinite(v[3]);
        amax = warp_max(amax);
        finite = __all_sync(0xffffffffu, finite) != 0;
        float d = 1.0f;
        if (finite) d = pow2ceil(fmaxf(amax, 1e-4f) / 127.0f);
        else if (lane == 0) atomicOr(status, 1u);        // rejected input: codes of this block are zero
        if (lane == 0) delta[r * delta_rs + b * delta_bs] = d;
#pragma unroll
        for (int t = 0; t < 4; ++t)
            if (c0 + t < cols) q[r * cols + c0 + t] = finite ? static_cast<int8_t>(static_cast<int>(rintf(v[t] / d))) : int8_t(0);
    }
}

__global__ void dequantize_i8_block_kernel(const int8_t* __restrict__ q, const float* __restrict__ delta, int64_t rows,
                                           int64_t cols, int64_t delta_rs, int64_t delta_bs, float* __restrict__ x) {
    const int64_t n = rows * cols;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / cols, b = (i % cols) / kQuantBlock;
        x[i] = static_cast<float>(q[i]) * delta[r * delta_rs + b * delta_bs];
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

cudaError_t quantize_i8_block_pow2(const float* x, int64_t rows, int64_t cols, int8_t* q, float* delta, int transposed,
                                   uint32_t* status, cudaStream_t s) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    const int64_t nb = (cols + kQuantBlock - 1) / kQuantBlock;
    const int64_t rs = transposed ? 1 : nb, bs = transposed ? rows : 1;
    quantize_i8_block_pow2_kernel<<<grid_for(rows * nb * 32, 256), 256, 0, s>>>(x, rows, cols, nb, q, delta, rs, bs, status);
    return cudaGetLastError();
}

cudaError_t dequantize_i8_block(const int8_t* q, const float* delta, int64_t rows, int64_t cols, int transposed, float* x,
                                cudaStream_t s) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    const int64_t nb = (cols + kQuantBlock - 1) / kQuantBlock;
    dequantize_i8_block_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(q, delta, rows, cols, transposed ? 1 : nb,
                                                                         transposed ? rows : 1, x);
    return cudaGetLastError();
}

}  // namespace b200
