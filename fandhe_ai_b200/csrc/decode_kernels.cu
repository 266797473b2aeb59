// Row-wise kernels of the quantized decode step: the work between two GEMMs is done by one CTA
// per token row, which finishes the previous GEMM (sums its split-K planes, dequantises) and
// prepares the next one (residual, RMSNorm, per-token int8 quantisation), so activations make one
// trip through L2 between tensor-core kernels.
//
// Numeric contracts restated from the reference: RMSNorm accumulates the sum of squares in f64
// and downcasts once for rstd (crates/backend-cuda/src/kernels_rmsnorm.rs:194,
// crates/backend-cpu/src/rmsnorm.rs:203-228); SiLU is x * sigmoid_stable(x)
// (crates/tensor-core/src/scalar_op.rs:355,666-673); greedy sampling takes the first index of the
// maximum (crates/autodiff/src/generate/mod.rs:333-343); embedding lookup is a row gather
// (crates/backend-cuda/src/kernels_gather_scatter.rs:71-220).
#include "kernels.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// CTA-wide reductions; every thread receives the result.  `scratch` holds 32 doubles.
__device__ __forceinline__ float block_max_f(float v, double* scratch) {
    float* s = reinterpret_cast<float*>(scratch);
    v = warp_max_f(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) s[warp] = v;
    __syncthreads();
    float r = lane < (blockDim.x >> 5) ? s[lane] : 0.0f;
    return warp_max_f(r);
}
__device__ __forceinline__ double block_sum_d(double v, double* scratch) {
    v = warp_sum_d(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double r = lane < (blockDim.x >> 5) ? scratch[lane] : 0.0;
    return warp_sum_d(r);
}


// Sum of the split-K planes of element (m, n): integer addition, exact and order-free.
__device__ __forceinline__ int sum_planes(const int* raw, int splits, size_t plane, size_t idx) {
    int a = 0;
    for (int s = 0; s < splits; ++s) a += raw[s * plane + idx];
    return a;
}

// Quantises the row held in `row` (shared memory, n values) to int8 with scale amax / 127.
__device__ __forceinline__ void quant_row_from_smem(const float* row, int n, int8_t* q_row, float* scale_out,
                                                    double* scratch) {
    float amax = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_max_f(amax, scratch);
    const float s = amax / 127.0f;
    if (threadIdx.x == 0) *scale_out = s;
    // n % 4 == 0 is guaranteed by the host
    uint32_t* q4 = reinterpret_cast<uint32_t*>(q_row);
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
        const uint32_t b0 = static_cast<uint32_t>(quant_i8(row[4 * i + 0], s)) & 0xFFu;
        const uint32_t b1 = static_cast<uint32_t>(quant_i8(row[4 * i + 1], s)) & 0xFFu;
        const uint32_t b2 = static_cast<uint32_t>(quant_i8(row[4 * i + 2], s)) & 0xFFu;
        const uint32_t b3 = static_cast<uint32_t>(quant_i8(row[4 * i + 3], s)) & 0xFFu;
        q4[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
}

// RMSNorm of the row in `row` (in place): f64 sum of squares, rstd downcast once, (x * rstd) * w.
__device__ __forceinline__ void rmsnorm_row_in_smem(float* row, int n, const float* w, float eps, double* scratch) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const double v = static_cast<double>(row[i]);
        acc = fma(v, v, acc);
    }
    acc = block_sum_d(acc, scratch);
    const float inv_n = 1.0f / static_cast<float>(n);
    const float rstd = static_cast<float>(1.0 / sqrt(fma(acc, static_cast<double>(inv_n), static_cast<double>(eps))));
    for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = __fmul_rn(__fmul_rn(row[i], rstd), w[i]);
    __syncthreads();
}

// h[m, :] = table[ids[m], :]; then norm + quant for the first layer.
__global__ void __launch_bounds__(kRowThreads)
embed_norm_quant_kernel(const int* __restrict__ ids, const float* __restrict__ table, int vocab, int d,
                        const float* __restrict__ norm_w, float eps, float* __restrict__ h, int8_t* __restrict__ xq,
                        float* __restrict__ sx, uint32_t* err) {
    extern __shared__ double smem_d[];
    double* scratch = smem_d;
    float* row = reinterpret_cast<float*>(smem_d + 32);
    const int m = blockIdx.x;
    int id = ids[m];
    if (id < 0 || id >= vocab) {          // never read outside the table; flag it
        if (threadIdx.x == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrTokenId));
        id = 0;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = table[static_cast<size_t>(id) * d + i];
        row[i] = v;
        h[static_cast<size_t>(m) * d + i] = v;
    }
    __syncthreads();
    rmsnorm_row_in_smem(row, d, norm_w, eps, scratch);
    quant_row_from_smem(row, d, xq + static_cast<size_t>(m) * d, sx + m, scratch);
}

// Finishes a row-parallel-output GEMM (O or down projection):
//   h[m, n] += acc[m, n] * (sx_in[m] * sw[n]);  xn = rmsnorm(h[m, :]) * norm_w;  (xq, sx_out) = quant(xn)
__global__ void __launch_bounds__(kRowThreads)
resid_norm_quant_kernel(const int* __restrict__ raw, int splits, int M, int d, const float* __restrict__ sx_in,
                        const float* __restrict__ sw, const float* __restrict__ pre,
                        const float* __restrict__ norm_w, float eps,
                        float* __restrict__ h, int8_t* __restrict__ xq, float* __restrict__ sx_out) {
    extern __shared__ double smem_d[];
    double* scratch = smem_d;
    float* row = reinterpret_cast<float*>(smem_d + 32);
    const int m = blockIdx.x;
    const size_t plane = static_cast<size_t>(M) * d;
    const float sa = pre ? 0.0f : sx_in[m];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const size_t idx = static_cast<size_t>(m) * d + i;
        const float y = pre ? pre[idx]
                            : fmaf(static_cast<float>(sum_planes(raw, splits, plane, idx)), sa * sw[i], 0.0f);
        const float hv = y + h[idx];
        h[idx] = hv;
        row[i] = hv;
    }
    __syncthreads();
    rmsnorm_row_in_smem(row, d, norm_w, eps, scratch);
    quant_row_from_smem(row, d, xq + static_cast<size_t>(m) * d, sx_out + m, scratch);
}

// Finishes the gate/up GEMM: a = silu(g) * u over raw columns [0, F) (gate) and [F, 2F) (up); quantises a.
__global__ void __launch_bounds__(kRowThreads)
gate_quant_kernel(const int* __restrict__ raw, int splits, int M, int F, const float* __restrict__ sx_in,
                  const float* __restrict__ sw, int8_t* __restrict__ xq, float* __restrict__ sx_out) {
    extern __shared__ double smem_d[];
    double* scratch = smem_d;
    float* row = reinterpret_cast<float*>(smem_d + 32);
    const int m = blockIdx.x;
    const size_t plane = static_cast<size_t>(M) * 2 * F;
    const float sa = sx_in[m];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const size_t ig = static_cast<size_t>(m) * 2 * F + i;
        const float g = fmaf(static_cast<float>(sum_planes(raw, splits, plane, ig)), sa * sw[i], 0.0f);
        const float u = fmaf(static_cast<float>(sum_planes(raw, splits, plane, ig + F)), sa * sw[F + i], 0.0f);
        row[i] = __fmul_rn(silu(g), u);
    }
    __syncthreads();
    quant_row_from_smem(row, F, xq + static_cast<size_t>(m) * F, sx_out + m, scratch);
}

__global__ void dequant_planes_kernel(const int* __restrict__ raw, int splits, int M, int N,
                                      const float* __restrict__ sx, const float* __restrict__ sw, float* __restrict__ y) {
    const size_t plane = static_cast<size_t>(M) * N;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < plane; i += size_t(gridDim.x) * blockDim.x)
        y[i] = fmaf(static_cast<float>(sum_planes(raw, splits, plane, i)), sx[i / N] * sw[i % N], 0.0f);
}

// Start of a decode step: remember each row's position for the new token, then count it in.
// A row that takes part in the step appends at its current length.  A row that sits the step out (no request in
// its slot) rewrites its last position instead - position 0 of its first block when it is empty - so that every
// kernel of the step still sees a valid one-token-or-longer sequence and its real contents stay untouched.
__global__ void begin_step_kernel(uint32_t* seq_lens, uint32_t* positions, const uint32_t* active, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const uint32_t len = seq_lens[i];
        if (active[i]) {
            positions[i] = len;
            seq_lens[i] = len + 1;
        } else {
            const uint32_t l = len > 0 ? len : 1u;
            positions[i] = l - 1;
            seq_lens[i] = l;
        }
    }
}

// Prefill of l_new tokens per sequence: token row m = b * l_new + i sits at position seq_lens[b] + i.
__global__ void prefill_positions_kernel(const uint32_t* seq_lens, uint32_t* positions, int count, int l_new) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m < count * l_new) positions[m] = seq_lens[m / l_new] + static_cast<uint32_t>(m % l_new);
}
__global__ void prefill_advance_kernel(uint32_t* seq_lens, int count, int l_new) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < count) seq_lens[b] += static_cast<uint32_t>(l_new);
}

// First index of the maximum of each row (strict '>' keeps the earliest index on ties).
__global__ void __launch_bounds__(kRowThreads)
argmax_rows_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out_ids) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const int m = blockIdx.x;
    const float* row = logits + static_cast<size_t>(m) * vocab;
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best) { best = v; bi = i; }            // ascending i per thread: first max kept
    }
    auto better = [](float v, int i, float bv, int bidx) { return v > bv || (v == bv && i < bidx); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out_ids[m] = bi == 0x7FFFFFFF ? 0 : bi;
    }
}

// Synthetic weights: element i of tensor `stream` is std * N(0,1) drawn from a counter-based hash
// (splitmix64 of (seed, stream, i)) and Box-Muller, so any shard can be generated independently.
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void fill_normal_kernel(float* out, int64_t n, uint64_t seed, uint64_t stream, float std) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const uint64_t r = splitmix64(splitmix64(seed ^ (stream * 0xD1B54A32D192ED03ull)) + static_cast<uint64_t>(i));
        const float u1 = (static_cast<float>(r >> 40) + 1.0f) * (1.0f / 16777217.0f);        // (0, 1)
        const float u2 = static_cast<float>((r >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);   // [0, 1)
        out[i] = std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    }
}
__global__ void fill_normal_bf16_kernel(uint16_t* out, int64_t n, uint64_t seed, uint64_t stream, float std) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const uint64_t r = splitmix64(splitmix64(seed ^ (stream * 0xD1B54A32D192ED03ull)) + static_cast<uint64_t>(i));
        const float u1 = (static_cast<float>(r >> 40) + 1.0f) * (1.0f / 16777217.0f);
        const float u2 = static_cast<float>((r >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        out[i] = static_cast<uint16_t>(f32_to_bf16_bits(std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2)));
    }
}
// Copies columns [c0, c0 + cols) of a row-major int8 matrix [rows, ld] into a dense [rows, cols] matrix.
__global__ void slice_cols_i8_kernel(const int8_t* __restrict__ src, int64_t rows, int64_t ld, int64_t c0, int64_t cols,
                                     int8_t* __restrict__ dst) {
    const int64_t n = rows * cols;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        dst[i] = src[(i / cols) * ld + c0 + (i % cols)];
}

int grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = int64_t(current_sm_count()) * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}
size_t row_smem(int n) { return 32 * sizeof(double) + static_cast<size_t>(n) * sizeof(float); }

template <typename K>
cudaError_t ensure_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

}  // namespace

cudaError_t embed_norm_quant(const int* ids, const float* table, int vocab, int M, int d, const float* norm_w, float eps,
                             float* h, int8_t* xq, float* sx, uint32_t* err, cudaStream_t s) {
    cudaError_t e = ensure_smem(embed_norm_quant_kernel, row_smem(d));
    if (e != cudaSuccess) return e;
    embed_norm_quant_kernel<<<M, kRowThreads, row_smem(d), s>>>(ids, table, vocab, d, norm_w, eps, h, xq, sx, err);
    return cudaGetLastError();
}
cudaError_t resid_norm_quant(const int* raw, int splits, int M, int d, const float* sx_in, const float* sw,
                             const float* pre, const float* norm_w, float eps, float* h, int8_t* xq, float* sx_out,
                             cudaStream_t s) {
    cudaError_t e = ensure_smem(resid_norm_quant_kernel, row_smem(d));
    if (e != cudaSuccess) return e;
    resid_norm_quant_kernel<<<M, kRowThreads, row_smem(d), s>>>(raw, splits, M, d, sx_in, sw, pre, norm_w, eps, h, xq,
                                                               sx_out);
    return cudaGetLastError();
}
cudaError_t dequant_planes(const int* raw, int splits, int M, int N, const float* sx, const float* sw, float* y,
                           cudaStream_t s) {
    dequant_planes_kernel<<<grid_for(int64_t(M) * N, 256), 256, 0, s>>>(raw, splits, M, N, sx, sw, y);
    return cudaGetLastError();
}
cudaError_t gate_quant(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, int8_t* xq,
                       float* sx_out, cudaStream_t s) {
    cudaError_t e = ensure_smem(gate_quant_kernel, row_smem(F));
    if (e != cudaSuccess) return e;
    gate_quant_kernel<<<M, kRowThreads, row_smem(F), s>>>(raw, splits, M, F, sx_in, sw, xq, sx_out);
    return cudaGetLastError();
}
cudaError_t begin_step(uint32_t* seq_lens, uint32_t* positions, const uint32_t* active, int n, cudaStream_t s) {
    begin_step_kernel<<<(n + 127) / 128, 128, 0, s>>>(seq_lens, positions, active, n);
    return cudaGetLastError();
}
cudaError_t prefill_positions(const uint32_t* seq_lens, uint32_t* positions, int count, int l_new, cudaStream_t s) {
    const int n = count * l_new;
    prefill_positions_kernel<<<(n + 255) / 256, 256, 0, s>>>(seq_lens, positions, count, l_new);
    return cudaGetLastError();
}
cudaError_t prefill_advance(uint32_t* seq_lens, int count, int l_new, cudaStream_t s) {
    prefill_advance_kernel<<<(count + 127) / 128, 128, 0, s>>>(seq_lens, count, l_new);
    return cudaGetLastError();
}
cudaError_t argmax_rows(const float* logits, int M, int vocab, int* out_ids, cudaStream_t s) {
    argmax_rows_kernel<<<M, kRowThreads, 0, s>>>(logits, vocab, out_ids);
    return cudaGetLastError();
}
cudaError_t fill_normal(float* out, int64_t n, uint64_t seed, uint64_t stream_id, float std, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    fill_normal_kernel<<<grid_for(n, 256), 256, 0, s>>>(out, n, seed, stream_id, std);
    return cudaGetLastError();
}
cudaError_t fill_normal_bf16(uint16_t* out, int64_t n, uint64_t seed, uint64_t stream_id, float std, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    fill_normal_bf16_kernel<<<grid_for(n, 256), 256, 0, s>>>(out, n, seed, stream_id, std);
    return cudaGetLastError();
}
cudaError_t slice_cols_i8(const int8_t* src, int64_t rows, int64_t ld, int64_t c0, int64_t cols, int8_t* dst,
                          cudaStream_t s) {
    if (rows * cols == 0) return cudaSuccess;
    slice_cols_i8_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(src, rows, ld, c0, cols, dst);
    return cudaGetLastError();
}

}  // namespace b200
