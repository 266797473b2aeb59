// Row-wise kernels of the decode step.
//
// Between two GEMMs a token row is owned by one CTA of up to 1024 threads that keeps the row in registers
// (1, 2 or 4 groups of four columns per thread) and does the two row-wide reductions (f64 sum of squares
// for RMSNorm, |max| for the per-token int8 scale) as block reductions summed in warp order, so the result
// does not depend on scheduling.  The two kernels that run once per step (embedding gather + first norm,
// greedy argmax over the vocabulary) cut a row into column chunks, one CTA each, launched as one
// thread-block cluster per row with the partial results exchanged through distributed shared memory in
// cluster-rank order.  Rows wider than 16384 columns use the one-CTA kernels of decode_kernels.cu.
//
// The per-element arithmetic is the same everywhere (and in the CPU restatement):
// y = fma(float(sum of planes), sx * sw, 0); h += y; xn = (h * rstd) * w; q = rne(xn / (amax / 127)).
#include <cooperative_groups.h>

#include "kernels.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxChunk = 2048;   // columns a CTA may hold (shared-memory row chunk)

struct RowShared {
    double part_sum;      // this CTA's sum of squares
    float part_max;       // this CTA's |max|
    double warp_d[8];
    float warp_f[8];
    int warp_i[8];
    float chunk[kMaxChunk];
};

__device__ __forceinline__ double block_sum(double v, RowShared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh.warp_d[warp] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) r += sh.warp_d[w];
    return r;
}
__device__ __forceinline__ float block_max(float v, RowShared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh.warp_f[warp] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, sh.warp_f[w]);
    return r;
}


// Row-wide sum over the cluster in rank order.
__device__ __forceinline__ double cluster_sum(cg::cluster_group& cl, RowShared& sh, double mine) {
    if (threadIdx.x == 0) sh.part_sum = mine;
    cl.sync();
    double total = 0.0;
    const unsigned n = cl.num_blocks();
    for (unsigned r = 0; r < n; ++r) total += *cl.map_shared_rank(&sh.part_sum, r);
    return total;
}
__device__ __forceinline__ float cluster_max(cg::cluster_group& cl, RowShared& sh, float mine) {
    if (threadIdx.x == 0) sh.part_max = mine;
    cl.sync();
    float total = 0.0f;
    const unsigned n = cl.num_blocks();
    for (unsigned r = 0; r < n; ++r) total = fmaxf(total, *cl.map_shared_rank(&sh.part_max, r));
    return total;
}

// RMSNorm + per-token int8 quantisation of the row whose chunk [c0, c0 + nc) sits in sh.chunk.
// `n` is the full row width.  Ends with a cluster barrier so that no CTA leaves while a peer still reads it.
__device__ __forceinline__ void norm_quant_chunk(cg::cluster_group& cl, RowShared& sh, int n, int c0, int nc,
                                                 const float* __restrict__ norm_w, float eps, int8_t* __restrict__ q_row,
                                                 float* __restrict__ scale_out, int fp8 = 0) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < nc; i += kThreads) {
        const double v = static_cast<double>(sh.chunk[i]);
        acc = fma(v, v, acc);
    }
    acc = cluster_sum(cl, sh, block_sum(acc, sh));
    const float inv_n = 1.0f / static_cast<float>(n);
    const float rstd = static_cast<float>(1.0 / sqrt(fma(acc, static_cast<double>(inv_n), static_cast<double>(eps))));
    float amax = 0.0f;
    for (int i = threadIdx.x; i < nc; i += kThreads) {
        const float v = __fmul_rn(__fmul_rn(sh.chunk[i], rstd), norm_w[c0 + i]);
        sh.chunk[i] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = cluster_max(cl, sh, block_max(amax, sh));
    const float s = fp8 ? amax / kE4m3Max : amax / 127.0f;
    if (cl.block_rank() == 0 && threadIdx.x == 0) *scale_out = s;
    uint32_t* q4 = reinterpret_cast<uint32_t*>(q_row + c0);
    for (int i = threadIdx.x; i < nc / 4; i += kThreads) {
        if (fp8) {
            q4[i] = quant4_e4m3(sh.chunk[4 * i + 0], sh.chunk[4 * i + 1], sh.chunk[4 * i + 2], sh.chunk[4 * i + 3], s);
            continue;
        }
        const uint32_t b0 = static_cast<uint32_t>(quant_i8(sh.chunk[4 * i + 0], s)) & 0xFFu;
        const uint32_t b1 = static_cast<uint32_t>(quant_i8(sh.chunk[4 * i + 1], s)) & 0xFFu;
        const uint32_t b2 = static_cast<uint32_t>(quant_i8(sh.chunk[4 * i + 2], s)) & 0xFFu;
        const uint32_t b3 = static_cast<uint32_t>(quant_i8(sh.chunk[4 * i + 3], s)) & 0xFFu;
        q4[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
    cl.sync();
}

// Sum of the split-K planes of four consecutive elements (16-byte loads): int32 sums, or (fp8) f32 sums in plane
// order whose bits are returned; acc_word_f32 turns either into the f32 value.
__device__ __forceinline__ int4 sum_planes4(const int* __restrict__ raw, int splits, size_t plane, size_t idx, int fp8 = 0) {
    if (fp8) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(raw + s * plane + idx);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        return make_int4(__float_as_int(a.x), __float_as_int(a.y), __float_as_int(a.z), __float_as_int(a.w));
    }
    int4 a = make_int4(0, 0, 0, 0);
    for (int s = 0; s < splits; ++s) {
        const int4 v = *reinterpret_cast<const int4*>(raw + s * plane + idx);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    return a;
}

// grid = (CL, M), cluster = (CL, 1, 1): blockIdx.x = column chunk (= cluster rank), blockIdx.y = row.

__global__ void __launch_bounds__(kThreads)
embed_norm_quant_cl_kernel(const int* __restrict__ ids, const float* __restrict__ table, int vocab, int d, int nc,
                           const float* __restrict__ norm_w, float eps, float* __restrict__ h, int8_t* __restrict__ xq,
                           float* __restrict__ sx, uint32_t* err, int fp8) {
    __shared__ RowShared sh;
    cg::cluster_group cl = cg::this_cluster();
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.y, c0 = blockIdx.x * nc;
    int id = ids[m];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrTokenId));
        id = 0;
    }
    const float* src = table + static_cast<size_t>(id) * d + c0;
    float* hdst = h + static_cast<size_t>(m) * d + c0;
    for (int g = threadIdx.x; g < nc / 4; g += kThreads) {
        const float4 v = *reinterpret_cast<const float4*>(src + 4 * g);
        *reinterpret_cast<float4*>(hdst + 4 * g) = v;
        *reinterpret_cast<float4*>(&sh.chunk[4 * g]) = v;
    }
    __syncthreads();
    norm_quant_chunk(cl, sh, d, c0, nc, norm_w, eps, xq + static_cast<size_t>(m) * d, sx + m, fp8);
}

// First index of the row maximum; chunk = columns per CTA (a multiple of 4).
__global__ void __launch_bounds__(kThreads)
argmax_cl_kernel(const float* __restrict__ logits, int vocab, int chunk, int* __restrict__ out_ids) {
    __shared__ RowShared sh;
    __shared__ float part_v;
    __shared__ int part_i;
    cg::cluster_group cl = cg::this_cluster();
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.y;
    const int c0 = blockIdx.x * chunk;
    int c1 = c0 + chunk;
    if (c1 > vocab) c1 = vocab;
    const float* row = logits + static_cast<size_t>(m) * vocab;
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    auto better = [](float v, int i, float bv, int bidx) { return v > bv || (v == bv && i < bidx); };
    for (int i = c0 + 4 * threadIdx.x; i < c1; i += 4 * kThreads) {     // vocab % 4 == 0 (checked on the host)
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        if (v.x > best) { best = v.x; bi = i; }
        if (v.y > best) { best = v.y; bi = i + 1; }
        if (v.z > best) { best = v.z; bi = i + 2; }
        if (v.w > best) { best = v.w; bi = i + 3; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sh.warp_f[warp] = best; sh.warp_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kThreads / 32; ++w)
            if (better(sh.warp_f[w], sh.warp_i[w], best, bi)) { best = sh.warp_f[w]; bi = sh.warp_i[w]; }
        part_v = best;
        part_i = bi;
    }
    cl.sync();
    if (cl.block_rank() == 0 && threadIdx.x == 0) {
        best = part_v; bi = part_i;
        for (unsigned r = 1; r < cl.num_blocks(); ++r) {
            const float ov = *cl.map_shared_rank(&part_v, r);
            const int oi = *cl.map_shared_rank(&part_i, r);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        out_ids[m] = bi == 0x7FFFFFFF ? 0 : bi;
    }
    cl.sync();
}

// Finishes the QKV GEMM: one CTA per (row, group of heads); no row-wide reduction is needed.
// q and k heads are rotated (rotate-half pairs (i, i + dh/2)), v heads are only dequantised.
__global__ void __launch_bounds__(kThreads)
qkv_rope_append_par_kernel(const int* __restrict__ raw, int splits, int M, int rows_per_seq, int hq, int hkv, int dh, int heads_per_cta,
                           const float* __restrict__ sx_in, const float* __restrict__ sw,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                           const uint32_t* __restrict__ positions, const uint32_t* __restrict__ active,
                           const uint32_t* __restrict__ block_tables,
                           int max_blocks_per_seq, int block_size, int num_blocks, float* __restrict__ q_out,
                           uint16_t* __restrict__ k_pool, uint16_t* __restrict__ v_pool, uint32_t* err, int fp8) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.y;
    const bool keep_kv = active == nullptr || active[m] != 0u;     // a row that sits the step out keeps its cache
    const int n = (hq + 2 * hkv) * dh;
    const int half = dh / 2;
    const size_t plane = static_cast<size_t>(M) * n;
    const float sa = sx_in[m];
    const int pos = static_cast<int>(positions[m]);
    bool ok = pos < max_pos;
    uint32_t blk = 0;
    if (ok) {
        blk = block_tables[static_cast<size_t>(m / rows_per_seq) * max_blocks_per_seq + pos / block_size];
        ok = blk < static_cast<uint32_t>(num_blocks);
    }
    if (!ok) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAppendSlot));
        return;
    }
    const float* cr = cos_t + static_cast<size_t>(pos) * half;
    const float* sr = sin_t + static_cast<size_t>(pos) * half;
    const size_t slot = static_cast<size_t>(blk) * block_size + pos % block_size;
    const int ekv = hkv * dh;
    const int head0 = blockIdx.x * heads_per_cta;
    for (int t = threadIdx.x; t < heads_per_cta * half; t += kThreads) {
        const int head = head0 + t / half, i = t % half;
        if (head >= hq + 2 * hkv) break;
        const size_t idx = static_cast<size_t>(m) * n + head * dh + i;
        int a1 = 0, a2 = 0;
        float f1 = 0.0f, f2 = 0.0f;
        for (int s = 0; s < splits; ++s) {
            if (fp8) {
                f1 += __int_as_float(raw[s * plane + idx]);
                f2 += __int_as_float(raw[s * plane + idx + half]);
            } else {
                a1 += raw[s * plane + idx];
                a2 += raw[s * plane + idx + half];
            }
        }
        const float x1 = fmaf(fp8 ? f1 : static_cast<float>(a1), sa * sw[head * dh + i], 0.0f);
        const float x2 = fmaf(fp8 ? f2 : static_cast<float>(a2), sa * sw[head * dh + i + half], 0.0f);
        if (head < hq + hkv) {
            const float c = cr[i], s = sr[i];
            const float o1 = fmaf(x1, c, -__fmul_rn(x2, s));
            const float o2 = fmaf(x2, c, __fmul_rn(x1, s));
            if (head < hq) {
                q_out[(static_cast<size_t>(m) * hq + head) * dh + i] = o1;
                q_out[(static_cast<size_t>(m) * hq + head) * dh + i + half] = o2;
            } else if (keep_kv) {
                const int kh = head - hq;
                k_pool[slot * ekv + kh * dh + i] = static_cast<uint16_t>(f32_to_bf16_bits(o1));
                k_pool[slot * ekv + kh * dh + i + half] = static_cast<uint16_t>(f32_to_bf16_bits(o2));
            }
        } else if (keep_kv) {
            const int vh = head - hq - hkv;
            v_pool[slot * ekv + vh * dh + i] = static_cast<uint16_t>(f32_to_bf16_bits(x1));
            v_pool[slot * ekv + vh * dh + i + half] = static_cast<uint16_t>(f32_to_bf16_bits(x2));
        }
    }
}

// ------------------------------------------------------------------------------------ one wide CTA per row
// Rows of up to 16384 columns: one CTA of up to 1024 threads owns a token row, every thread keeps VPT groups
// of four columns in registers, and the two row-wide reductions are plain block reductions (warp shuffles, one
// shared-memory exchange summed in warp order).  All rows of a decode batch run in one wave with no cluster
// barriers in the dependency chain; the arithmetic per element is the same as in the cluster kernels.
constexpr int kWideThreads = 1024;
constexpr int kWideMaxVpt = 4;

struct WideShared {
    double wd[32];
    float wf[32];
};

__device__ __forceinline__ double wide_sum(double v, WideShared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh.wd[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; ++w) r += sh.wd[w];
    return r;
}
__device__ __forceinline__ float wide_max(float v, WideShared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh.wf[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; ++w) r = fmaxf(r, sh.wf[w]);
    return r;
}
__device__ __forceinline__ uint32_t quant4(const float4& v, float s) {
    const uint32_t b0 = static_cast<uint32_t>(quant_i8(v.x, s)) & 0xFFu;
    const uint32_t b1 = static_cast<uint32_t>(quant_i8(v.y, s)) & 0xFFu;
    const uint32_t b2 = static_cast<uint32_t>(quant_i8(v.z, s)) & 0xFFu;
    const uint32_t b3 = static_cast<uint32_t>(quant_i8(v.w, s)) & 0xFFu;
    return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}
// four codes of the row's activation format: int8 (scale amax / 127) or e4m3 (scale amax / 448)
__device__ __forceinline__ uint32_t pack4(const float4& v, float s, int fp8) {
    return fp8 ? quant4_e4m3(v.x, v.y, v.z, v.w, s) : quant4(v, s);
}
__device__ __forceinline__ float row_scale(float amax, int fp8) { return fp8 ? amax / kE4m3Max : amax / 127.0f; }
__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

// |max| of the row, scale = amax / 127 (int8) or amax / 448 (e4m3), code store.  v[k] holds group
// threadIdx.x + k * blockDim.x.
template <int VPT>
__device__ __forceinline__ void wide_quant(const float4 (&v)[VPT], int groups, WideShared& sh, int8_t* __restrict__ q_row,
                                           float* __restrict__ scale_out, int fp8 = 0) {
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
        if (int(threadIdx.x + k * blockDim.x) < groups) amax = fmaxf(amax, amax4(v[k]));
    amax = wide_max(amax, sh);
    const float s = row_scale(amax, fp8);
    if (threadIdx.x == 0) *scale_out = s;
    uint32_t* q4 = reinterpret_cast<uint32_t*>(q_row);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) q4[g] = pack4(v[k], s, fp8);
    }
}

template <int VPT>
__device__ __forceinline__ void wide_norm_quant(float4 (&v)[VPT], int groups, int n, WideShared& sh,
                                                const float* __restrict__ norm_w, float eps, int8_t* __restrict__ q_row,
                                                float* __restrict__ scale_out, int fp8 = 0) {
    double acc = 0.0;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
        if (int(threadIdx.x + k * blockDim.x) < groups) {
            const double a = v[k].x, b = v[k].y, c = v[k].z, e = v[k].w;
            acc = fma(a, a, acc); acc = fma(b, b, acc); acc = fma(c, c, acc); acc = fma(e, e, acc);
        }
    acc = wide_sum(acc, sh);
    const float inv_n = 1.0f / static_cast<float>(n);
    const float rstd = static_cast<float>(1.0 / sqrt(fma(acc, static_cast<double>(inv_n), static_cast<double>(eps))));
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) {
            const float4 w4 = *reinterpret_cast<const float4*>(norm_w + 4 * g);
            v[k].x = __fmul_rn(__fmul_rn(v[k].x, rstd), w4.x);
            v[k].y = __fmul_rn(__fmul_rn(v[k].y, rstd), w4.y);
            v[k].z = __fmul_rn(__fmul_rn(v[k].z, rstd), w4.z);
            v[k].w = __fmul_rn(__fmul_rn(v[k].w, rstd), w4.w);
        }
    }
    wide_quant<VPT>(v, groups, sh, q_row, scale_out, fp8);
}

template <int VPT, bool kF8>
__global__ void __launch_bounds__(kWideThreads)
resid_norm_quant_wide_kernel(const int* __restrict__ raw, int splits, int M, int d, const float* __restrict__ sx_in,
                             const float* __restrict__ sw, const float* __restrict__ pre, const float* __restrict__ norm_w,
                             float eps, float* __restrict__ h, int8_t* __restrict__ xq, float* __restrict__ sx_out) {
    constexpr int fp8 = kF8 ? 1 : 0;
    __shared__ WideShared sh;
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = d / 4;
    const size_t plane = static_cast<size_t>(M) * d;
    const size_t base = static_cast<size_t>(m) * d;
    const float sa = pre ? 0.0f : sx_in[m];
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) {
            float4 y;
            if (pre) {
                y = *reinterpret_cast<const float4*>(pre + base + 4 * g);
            } else {
                const int4 a = sum_planes4(raw, splits, plane, base + 4 * g, fp8);
                const float4 w4 = *reinterpret_cast<const float4*>(sw + 4 * g);
                y.x = fmaf(acc_word_f32(a.x, fp8), sa * w4.x, 0.0f);
                y.y = fmaf(acc_word_f32(a.y, fp8), sa * w4.y, 0.0f);
                y.z = fmaf(acc_word_f32(a.z, fp8), sa * w4.z, 0.0f);
                y.w = fmaf(acc_word_f32(a.w, fp8), sa * w4.w, 0.0f);
            }
            float4 hv = *reinterpret_cast<const float4*>(h + base + 4 * g);
            hv.x = y.x + hv.x; hv.y = y.y + hv.y; hv.z = y.z + hv.z; hv.w = y.w + hv.w;
            *reinterpret_cast<float4*>(h + base + 4 * g) = hv;
            v[k] = hv;
        }
    }
    wide_norm_quant<VPT>(v, groups, d, sh, norm_w, eps, xq + base, sx_out + m, fp8);
}

// kF8: the FP8 form (f32 accumulator words in, E4M3 codes out); a template parameter because the extra paths cost the
// int8 instantiation registers it does not have (1024 threads: 64 per thread)
template <int VPT, bool kF8>
__global__ void __launch_bounds__(kWideThreads)
gate_quant_wide_kernel(const int* __restrict__ raw, int splits, int M, int F, const float* __restrict__ sx_in,
                       const float* __restrict__ sw, int8_t* __restrict__ xq, float* __restrict__ sx_out) {
    constexpr int fp8 = kF8 ? 1 : 0;
    __shared__ WideShared sh;
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = F / 4;
    const size_t plane = static_cast<size_t>(M) * 2 * F;
    const size_t base = static_cast<size_t>(m) * 2 * F;
    const float sa = sx_in[m];
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) {
            const int4 ag = sum_planes4(raw, splits, plane, base + 4 * g, fp8);
            const int4 au = sum_planes4(raw, splits, plane, base + F + 4 * g, fp8);
            const float4 wg = *reinterpret_cast<const float4*>(sw + 4 * g);
            const float4 wu = *reinterpret_cast<const float4*>(sw + F + 4 * g);
            v[k].x = __fmul_rn(silu(fmaf(acc_word_f32(ag.x, fp8), sa * wg.x, 0.0f)), fmaf(acc_word_f32(au.x, fp8), sa * wu.x, 0.0f));
            v[k].y = __fmul_rn(silu(fmaf(acc_word_f32(ag.y, fp8), sa * wg.y, 0.0f)), fmaf(acc_word_f32(au.y, fp8), sa * wu.y, 0.0f));
            v[k].z = __fmul_rn(silu(fmaf(acc_word_f32(ag.z, fp8), sa * wg.z, 0.0f)), fmaf(acc_word_f32(au.z, fp8), sa * wu.z, 0.0f));
            v[k].w = __fmul_rn(silu(fmaf(acc_word_f32(ag.w, fp8), sa * wg.w, 0.0f)), fmaf(acc_word_f32(au.w, fp8), sa * wu.w, 0.0f));
        }
    }
    wide_quant<VPT>(v, groups, sh, xq + static_cast<size_t>(m) * F, sx_out + m, fp8);
}

template <int VPT>
__global__ void __launch_bounds__(kWideThreads)
quant_rows_wide_kernel(const float* __restrict__ x, int n, int8_t* __restrict__ xq, float* __restrict__ sx_out, int fp8) {
    __shared__ WideShared sh;
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = n / 4;
    const float* src = x + static_cast<size_t>(m) * n;
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) v[k] = *reinterpret_cast<const float4*>(src + 4 * g);
    }
    wide_quant<VPT>(v, groups, sh, xq + static_cast<size_t>(m) * n, sx_out + m, fp8);
}

// ------------------------------------------------------------------------------------ rows under a global scale
// Tensor parallelism with exact integer sums: the per-token scale of a row that is split over the ranks comes from
// the maximum over ALL ranks' columns, so the row maximum is taken first (and merged across the ranks by the
// caller), and the quantiser then uses the merged maximum instead of the local one.
template <int VPT>
__global__ void __launch_bounds__(kWideThreads)
rows_amax_wide_kernel(const float* __restrict__ x, int n, float* __restrict__ amax_out) {
    __shared__ WideShared sh;
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = n / 4;
    const float* src = x + static_cast<size_t>(m) * n;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) amax = fmaxf(amax, amax4(*reinterpret_cast<const float4*>(src + 4 * g)));
    }
    amax = wide_max(amax, sh);
    if (threadIdx.x == 0) amax_out[m] = amax;
}

template <int VPT>
__global__ void __launch_bounds__(kWideThreads)
quant_rows_scaled_wide_kernel(const float* __restrict__ x, int n, const float* __restrict__ amax_in, int8_t* __restrict__ xq,
                              float* __restrict__ sx_out) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = n / 4;
    const float* src = x + static_cast<size_t>(m) * n;
    const float s = amax_in[m] / 127.0f;
    if (threadIdx.x == 0) sx_out[m] = s;
    uint32_t* q4 = reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m) * n);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) q4[g] = quant4(*reinterpret_cast<const float4*>(src + 4 * g), s);
    }
}

// a = silu(gate) * up of this rank's columns as f32 (the arithmetic of gate_quant_wide) and the row maximum of |a|
template <int VPT>
__global__ void __launch_bounds__(kWideThreads)
gate_f32_wide_kernel(const int* __restrict__ raw, int splits, int M, int F, const float* __restrict__ sx_in,
                     const float* __restrict__ sw, float* __restrict__ out, float* __restrict__ amax_out) {
    __shared__ WideShared sh;
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, groups = F / 4;
    const size_t plane = static_cast<size_t>(M) * 2 * F;
    const size_t base = static_cast<size_t>(m) * 2 * F;
    const float sa = sx_in[m];
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) {
            const int4 ag = sum_planes4(raw, splits, plane, base + 4 * g);
            const int4 au = sum_planes4(raw, splits, plane, base + F + 4 * g);
            const float4 wg = *reinterpret_cast<const float4*>(sw + 4 * g);
            const float4 wu = *reinterpret_cast<const float4*>(sw + F + 4 * g);
            float4 v;
            v.x = __fmul_rn(silu(fmaf(static_cast<float>(ag.x), sa * wg.x, 0.0f)), fmaf(static_cast<float>(au.x), sa * wu.x, 0.0f));
            v.y = __fmul_rn(silu(fmaf(static_cast<float>(ag.y), sa * wg.y, 0.0f)), fmaf(static_cast<float>(au.y), sa * wu.y, 0.0f));
            v.z = __fmul_rn(silu(fmaf(static_cast<float>(ag.z), sa * wg.z, 0.0f)), fmaf(static_cast<float>(au.z), sa * wu.z, 0.0f));
            v.w = __fmul_rn(silu(fmaf(static_cast<float>(ag.w), sa * wg.w, 0.0f)), fmaf(static_cast<float>(au.w), sa * wu.w, 0.0f));
            *reinterpret_cast<float4*>(out + static_cast<size_t>(m) * F + 4 * g) = v;
            amax = fmaxf(amax, amax4(v));
        }
    }
    amax = wide_max(amax, sh);
    if (threadIdx.x == 0) amax_out[m] = amax;
}

// ------------------------------------------------------------------------------------ cross-GPU finish
// Tensor parallel, after a row-parallel GEMM: every rank holds an f32 partial [M, d] of the layer output in its
// exchange block.  Rank r owns the token rows [r * rows, (r + 1) * rows): it adds the partials of its rows over
// all ranks (peer loads, rank order), adds the residual stream (which therefore lives only on the owner), applies
// RMSNorm and the per-token int8 quantisation, and stores the finished int8 row and its scale into the exchange
// block of every rank - the A operand of the next GEMM.
//
// Flags are epoch counters that a rank writes into the other ranks' blocks (layout of a block: ready[tp] at +0,
// delivered[tp] at +256, then sx, xq and part at the given offsets):
//   ready[s]      rank s has finished the partial of this epoch           (waited for here, before the loads)
//   delivered[s]  rank s has stored its finished rows of this epoch here  (waited for by the consumer of xq: the
//                 next GEMM polls them right before it loads its A operand, so the wait overlaps its weight prefetch)
// This kernel does not wait for the other ranks' rows.  What keeps a fast rank from overwriting data a slow one
// still reads: a rank rewrites `part` only after a GEMM that waited for every delivered flag of the previous epoch
// (a rank delivers after its peer loads), and peers store into xq / sx only after this rank raised its next ready
// flag, which it does after its own readers of xq / sx have finished.  Every wait is bounded by time and a rank
// that gives up poisons the flags it owns (see wait_peer_flag).  One CTA per owned row.
struct TpFinishArgs {
    uint8_t* const* peers;     // [tp] base of every rank's exchange block (this rank's own included)
    size_t o_sx, o_xq, o_part; // byte offsets inside a block
    int tp, rank;
    int rows;                  // rows per rank
    int d;                     // row width
    const float* norm_w;
    float eps;
    float* h;                  // [M, d] residual stream (only the owned rows are kept current)
    uint32_t* epoch;           // this rank's call counter
    unsigned int* arrived;     // CTAs of this launch that have delivered their row
    uint32_t* err;
    uint64_t timeout_ns;       // bound of every flag wait
    // Scattered form: the GEMMs of all ranks have stored the partials of this rank's rows into the planes
    // [tp][rows][d] of this rank's block (GemmPush) and count their launches in count[tp] at o_count; this kernel then
    // sends no ready flag and loads nothing from a peer.  push_tiles = counts per GEMM launch (0: the pulled form),
    // *push_target = counts consumed by the earlier calls.
    size_t o_count;
    uint32_t push_tiles;
    uint32_t* push_target;
    int fp8;                   // the delivered rows are e4m3 codes under the scale amax / 448
};

// kScattered / kF8 are template parameters for the registers' sake (1024 threads: 64 per thread).
template <int VPT, bool kScattered, bool kF8>
__global__ void __launch_bounds__(kWideThreads)
tp_finish_kernel(TpFinishArgs a) {
    __shared__ WideShared sh;
    __shared__ int s_ok, s_last;
    __shared__ uint8_t* s_peer[16];
    // the table of block bases is read once, before anything waits: a pointer fetched from memory between two
    // remote loads would put one memory round trip in front of each of them
    if (threadIdx.x < a.tp) s_peer[threadIdx.x] = a.peers[threadIdx.x];
    if (threadIdx.x == 0) s_ok = 1;
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t epoch = *a.epoch + 1;
    constexpr bool scattered = kScattered;
    constexpr int fp8 = kF8 ? 1 : 0;
    const uint32_t target = scattered ? *a.push_target + a.push_tiles : 0u;
    __syncthreads();
    uint8_t* mine = s_peer[a.rank];
    const uint32_t* ready = reinterpret_cast<const uint32_t*>(mine);
    // 1. this rank's partial is complete (the GEMM before this kernel has finished): tell every rank
    if (!scattered && blockIdx.x == 0 && threadIdx.x < a.tp) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(s_peer[threadIdx.x]) + a.rank, epoch);
    }
    // 2. wait for every rank's partial (scattered form: for every tile of every rank's GEMM; the ready word of a rank
    //    then only carries its poison)
    if (threadIdx.x < a.tp) {
        const bool got = scattered ? wait_peer_count(reinterpret_cast<const uint32_t*>(mine + a.o_count) + threadIdx.x, target,
                                                     ready + threadIdx.x, a.err, a.timeout_ns)
                                   : wait_peer_flag(ready + threadIdx.x, epoch, a.err, a.timeout_ns);
        if (!got) s_ok = 0;
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    const int row = a.rank * a.rows + blockIdx.x;
    const int groups = a.d / 4;
    const size_t base = static_cast<size_t>(row) * a.d;
    float4 v[VPT];
    if (ok) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int g = threadIdx.x + k * blockDim.x;
            if (g < groups) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                // eight ranks at a time: all their loads are in flight before the first addition (one NVLink round
                // trip instead of one per rank); the additions stay in rank order
                for (int p0 = 0; p0 < a.tp; p0 += 8) {
                    float4 x[8];
                    const float* src[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int p = p0 + i < a.tp ? p0 + i : 0;
                        src[i] = scattered ? reinterpret_cast<const float*>(mine + a.o_part) +
                                                 (static_cast<size_t>(p) * a.rows + blockIdx.x) * a.d + 4 * g
                                           : reinterpret_cast<const float*>(s_peer[p] + a.o_part) + base + 4 * g;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (p0 + i < a.tp) x[i] = ld_relaxed_sys_f4(src[i]);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (p0 + i < a.tp) {
                            y.x = __fadd_rn(y.x, x[i].x); y.y = __fadd_rn(y.y, x[i].y);
                            y.z = __fadd_rn(y.z, x[i].z); y.w = __fadd_rn(y.w, x[i].w);
                        }
                }
                float4 hv = *reinterpret_cast<const float4*>(a.h + base + 4 * g);
                hv.x = y.x + hv.x; hv.y = y.y + hv.y; hv.z = y.z + hv.z; hv.w = y.w + hv.w;
                *reinterpret_cast<float4*>(a.h + base + 4 * g) = hv;
                v[k] = hv;
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k) v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // RMSNorm and the per-token scale (same arithmetic as wide_norm_quant)
    double acc = 0.0;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
        if (int(threadIdx.x + k * blockDim.x) < groups) {
            const double x0 = v[k].x, x1 = v[k].y, x2 = v[k].z, x3 = v[k].w;
            acc = fma(x0, x0, acc); acc = fma(x1, x1, acc); acc = fma(x2, x2, acc); acc = fma(x3, x3, acc);
        }
    acc = wide_sum(acc, sh);
    const float inv_n = 1.0f / static_cast<float>(a.d);
    const float rstd = static_cast<float>(1.0 / sqrt(fma(acc, static_cast<double>(inv_n), static_cast<double>(a.eps))));
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int g = threadIdx.x + k * blockDim.x;
        if (g < groups) {
            const float4 w4 = *reinterpret_cast<const float4*>(a.norm_w + 4 * g);
            v[k].x = __fmul_rn(__fmul_rn(v[k].x, rstd), w4.x);
            v[k].y = __fmul_rn(__fmul_rn(v[k].y, rstd), w4.y);
            v[k].z = __fmul_rn(__fmul_rn(v[k].z, rstd), w4.z);
            v[k].w = __fmul_rn(__fmul_rn(v[k].w, rstd), w4.w);
            amax = fmaxf(amax, amax4(v[k]));
        }
    }
    amax = wide_max(amax, sh);
    const float s = row_scale(amax, fp8);
    // 3. deliver the row to every rank
    if (ok) {
        for (int p = 0; p < a.tp; ++p) {
            uint32_t* q4 = reinterpret_cast<uint32_t*>(s_peer[p] + a.o_xq + base);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int g = threadIdx.x + k * blockDim.x;
                if (g < groups) q4[g] = pack4(v[k], s, fp8);
            }
            if (threadIdx.x == 0) reinterpret_cast<float*>(s_peer[p] + a.o_sx)[row] = s;
        }
    }
    // The row stores above become visible to the other GPUs through one chain: a device-scope fence by every storing
    // thread, the CTA barrier, the count of this CTA in this GPU's memory (device-scope fences around it), and the
    // system-scope fence and release of the CTA that completes the launch.  Only that last CTA waits for the peers'
    // acknowledgements.
    __threadfence();
    __syncthreads();
    // 4. the last CTA of this launch tells every rank that this rank's rows are delivered (or, after a failed wait,
    //    that they never will be) and advances the call counter
    if (threadIdx.x == 0) {
        const unsigned int seen = atomicAdd(a.arrived, 1u);
        __threadfence();
        s_last = seen == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        // a failure in any CTA of this launch has set the error word by now
        const bool failed = !ok || *reinterpret_cast<volatile uint32_t*>(a.err) != 0u;
        if (threadIdx.x < a.tp) {
            __threadfence_system();
            uint32_t* peer = reinterpret_cast<uint32_t*>(s_peer[threadIdx.x]);
            if (failed) st_release_sys(peer + a.rank, kPeerPoison);
            st_release_sys(peer + 64 + a.rank, failed ? kPeerPoison : epoch);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            *a.arrived = 0u;
            *a.epoch = epoch;
            if (scattered) *a.push_target = target;
        }
    }
}

// Groups of four columns per thread (1, 2 or 4) and the block size for a row of n columns; vpt = 0 when the
// row is too wide (or not a multiple of 4) for the one-CTA kernels.
void wide_shape(int n, int* vpt, int* threads, int rows = 1) {
    *vpt = 0;
    *threads = 0;
    if (n <= 0 || n % 4 != 0) return;
    const int groups = n / 4;
    int v = (groups + kWideThreads - 1) / kWideThreads;
    if (v > kWideMaxVpt) return;
    if (v == 3) v = 4;
    // more rows than SMs: smaller CTAs (more groups per thread) so that several rows share an SM and the batch
    // still runs as one wave
    while (rows > current_sm_count() && v < kWideMaxVpt && groups / (2 * v) >= 256) v *= 2;
    *vpt = v;
    *threads = ((groups + v - 1) / v + 31) / 32 * 32;
}

// Largest power-of-two cluster size <= 8 whose chunks are multiples of 4 columns, fit the shared chunk and
// keep every thread busy; 0 when the row cannot be chunked that way.
int pick_cluster(int n) {
    for (int cl = 8; cl >= 1; cl >>= 1) {
        if (n % (cl * 4) != 0) continue;
        const int nc = n / cl;
        if (nc > kMaxChunk) continue;
        if (cl > 1 && nc < kThreads * 2) continue;   // too little work per CTA: use fewer, larger chunks
        return cl;
    }
    return 0;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_cluster(void (*kernel)(KArgs...), int cl, int rows, cudaStream_t s, Args... args) {
    return launch_ex(kernel, dim3(cl, rows, 1), dim3(kThreads, 1, 1), 0, s, cl, true, args...);
}

}  // namespace

// Dispatchers: the wide (or cluster) kernel when the row width allows it, else the one-CTA-per-row kernel.
cudaError_t embed_norm_quant_auto(const int* ids, const float* table, int vocab, int M, int d, const float* norm_w,
                                  float eps, float* h, int8_t* xq, float* sx, uint32_t* err, cudaStream_t s, int fp8) {
    const int cl = pick_cluster(d);
    if (cl == 0) return fp8 ? cudaErrorInvalidValue : embed_norm_quant(ids, table, vocab, M, d, norm_w, eps, h, xq, sx, err, s);
    return launch_cluster(embed_norm_quant_cl_kernel, cl, M, s, ids, table, vocab, d, d / cl, norm_w, eps, h, xq, sx, err, fp8);
}

cudaError_t resid_norm_quant_auto(const int* raw, int splits, int M, int d, const float* sx_in, const float* sw,
                                  const float* pre, const float* norm_w, float eps, float* h, int8_t* xq, float* sx_out,
                                  cudaStream_t s, int fp8) {
    int vpt, threads;
    wide_shape(d, &vpt, &threads, M);
#define B200_WIDE_RESID(V)                                                                                                     \
    return fp8 ? launch_ex(resid_norm_quant_wide_kernel<V, true>, dim3(M), dim3(threads), 0, s, 1, true, raw, splits, M, d,   \
                           sx_in, sw, pre, norm_w, eps, h, xq, sx_out)                                                          \
               : launch_ex(resid_norm_quant_wide_kernel<V, false>, dim3(M), dim3(threads), 0, s, 1, true, raw, splits, M, d,  \
                           sx_in, sw, pre, norm_w, eps, h, xq, sx_out)
    if (vpt == 1) B200_WIDE_RESID(1);
    if (vpt == 2) B200_WIDE_RESID(2);
    if (vpt == 4) B200_WIDE_RESID(4);
#undef B200_WIDE_RESID
    if (fp8) return cudaErrorInvalidValue;      // the FP8 format exists in the wide kernels only
    return resid_norm_quant(raw, splits, M, d, sx_in, sw, pre, norm_w, eps, h, xq, sx_out, s);
}

cudaError_t gate_quant_auto(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, int8_t* xq,
                            float* sx_out, cudaStream_t s, int fp8) {
    int vpt, threads;
    wide_shape(F, &vpt, &threads, M);
#define B200_WIDE_GATE(V)                                                                                                 \
    return fp8 ? launch_ex(gate_quant_wide_kernel<V, true>, dim3(M), dim3(threads), 0, s, 1, true, raw, splits, M, F, sx_in, \
                           sw, xq, sx_out)                                                                                 \
               : launch_ex(gate_quant_wide_kernel<V, false>, dim3(M), dim3(threads), 0, s, 1, true, raw, splits, M, F, sx_in, \
                           sw, xq, sx_out)
    if (vpt == 1) B200_WIDE_GATE(1);
    if (vpt == 2) B200_WIDE_GATE(2);
    if (vpt == 4) B200_WIDE_GATE(4);
#undef B200_WIDE_GATE
    if (fp8) return cudaErrorInvalidValue;
    return gate_quant(raw, splits, M, F, sx_in, sw, xq, sx_out, s);
}

cudaError_t quantize_rows_auto(const float* x, int M, int n, int8_t* xq, float* sx_out, cudaStream_t s, int fp8) {
    int vpt, threads;
    wide_shape(n, &vpt, &threads, M);
    if (vpt == 1) return launch_ex(quant_rows_wide_kernel<1>, dim3(M), dim3(threads), 0, s, 1, true, x, n, xq, sx_out, fp8);
    if (vpt == 2) return launch_ex(quant_rows_wide_kernel<2>, dim3(M), dim3(threads), 0, s, 1, true, x, n, xq, sx_out, fp8);
    if (vpt == 4) return launch_ex(quant_rows_wide_kernel<4>, dim3(M), dim3(threads), 0, s, 1, true, x, n, xq, sx_out, fp8);
    if (fp8) return cudaErrorInvalidValue;
    return quantize_i8_per_row(x, M, n, xq, sx_out, s);
}

cudaError_t argmax_rows_auto(const float* logits, int M, int vocab, int* out_ids, cudaStream_t s) {
    if (vocab % 4 != 0 || vocab < 8 * 4 * kThreads) return argmax_rows(logits, M, vocab, out_ids, s);
    const int cl = 8;
    int chunk = (vocab + cl - 1) / cl;
    chunk = (chunk + 3) / 4 * 4;
    return launch_cluster(argmax_cl_kernel, cl, M, s, logits, vocab, chunk, out_ids);
}

cudaError_t qkv_rope_append_auto(const int* raw, int splits, int M, int hq, int hkv, int dh, const float* sx_in,
                                 const float* sw, const float* cos_t, const float* sin_t, int max_pos,
                                 const uint32_t* positions, const uint32_t* active, const uint32_t* block_tables,
                                 int max_blocks_per_seq, int block_size, int num_blocks, float* q_out, uint16_t* k_pool,
                                 uint16_t* v_pool, uint32_t* err, cudaStream_t s, int rows_per_seq, int fp8) {
    const int heads = hq + 2 * hkv;
    int hpc = (2 * kThreads) / (dh / 2);      // two rotary pairs per thread
    if (hpc < 1) hpc = 1;
    dim3 grid((heads + hpc - 1) / hpc, M);
    return launch_ex(qkv_rope_append_par_kernel, grid, dim3(kThreads), 0, s, 1, true, raw, splits, M, rows_per_seq, hq, hkv, dh, hpc, sx_in,
                     sw, cos_t, sin_t, max_pos, positions, active, block_tables, max_blocks_per_seq, block_size, num_blocks,
                     q_out, k_pool, v_pool, err, fp8);
}

cudaError_t rows_amax(const float* x, int M, int n, float* amax_out, cudaStream_t s) {
    int vpt, threads;
    wide_shape(n, &vpt, &threads, M);
    if (vpt == 1) return launch_ex(rows_amax_wide_kernel<1>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax_out);
    if (vpt == 2) return launch_ex(rows_amax_wide_kernel<2>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax_out);
    if (vpt == 4) return launch_ex(rows_amax_wide_kernel<4>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax_out);
    return cudaErrorInvalidValue;
}

cudaError_t quantize_rows_with_amax(const float* x, int M, int n, const float* amax, int8_t* xq, float* sx_out, cudaStream_t s) {
    int vpt, threads;
    wide_shape(n, &vpt, &threads, M);
    if (vpt == 1) return launch_ex(quant_rows_scaled_wide_kernel<1>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax, xq, sx_out);
    if (vpt == 2) return launch_ex(quant_rows_scaled_wide_kernel<2>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax, xq, sx_out);
    if (vpt == 4) return launch_ex(quant_rows_scaled_wide_kernel<4>, dim3(M), dim3(threads), 0, s, 1, true, x, n, amax, xq, sx_out);
    return cudaErrorInvalidValue;
}

cudaError_t gate_rows_f32(const int* raw, int splits, int M, int F, const float* sx_in, const float* sw, float* out,
                          float* amax_out, cudaStream_t s) {
    int vpt, threads;
    wide_shape(F, &vpt, &threads, M);
#define B200_GATE_F32(V)                                                                                           \
    return launch_ex(gate_f32_wide_kernel<V>, dim3(M), dim3(threads), 0, s, 1, true, raw, splits, M, F, sx_in, sw, \
                     out, amax_out)
    if (vpt == 1) B200_GATE_F32(1);
    if (vpt == 2) B200_GATE_F32(2);
    if (vpt == 4) B200_GATE_F32(4);
#undef B200_GATE_F32
    return cudaErrorInvalidValue;
}

bool rows_scaled_supported(int n) {
    int vpt, threads;
    wide_shape(n, &vpt, &threads);
    return vpt != 0;
}

bool tp_finish_supported(int d) {
    int vpt, threads;
    wide_shape(d, &vpt, &threads);
    return vpt != 0;
}

cudaError_t tp_finish(uint8_t* const* peers, size_t o_sx, size_t o_xq, size_t o_part, int tp, int rank, int rows, int d,
                      const float* norm_w, float eps, float* h, uint32_t* epoch, unsigned int* arrived, uint32_t* err,
                      cudaStream_t s, uint64_t timeout_ns, size_t o_count, uint32_t push_tiles, uint32_t* push_target, int fp8) {
    int vpt, threads;
    wide_shape(d, &vpt, &threads);
    if (push_tiles != 0u && push_target == nullptr) return cudaErrorInvalidValue;
    TpFinishArgs a{peers, o_sx, o_xq, o_part, tp, rank, rows, d, norm_w, eps, h, epoch, arrived, err,
                   timeout_ns ? timeout_ns : kPeerWaitNs, o_count, push_tiles, push_target, fp8};
#define B200_TP_FINISH(V)                                                                                             \
    do {                                                                                                              \
        if (push_tiles != 0u)                                                                                         \
            return fp8 ? launch_ex(tp_finish_kernel<V, true, true>, dim3(rows), dim3(threads), 0, s, 1, true, a)      \
                       : launch_ex(tp_finish_kernel<V, true, false>, dim3(rows), dim3(threads), 0, s, 1, true, a);    \
        return fp8 ? launch_ex(tp_finish_kernel<V, false, true>, dim3(rows), dim3(threads), 0, s, 1, true, a)         \
                   : launch_ex(tp_finish_kernel<V, false, false>, dim3(rows), dim3(threads), 0, s, 1, true, a);       \
    } while (0)
    if (vpt == 1) B200_TP_FINISH(1);
    if (vpt == 2) B200_TP_FINISH(2);
    if (vpt == 4) B200_TP_FINISH(4);
#undef B200_TP_FINISH
    return cudaErrorInvalidValue;
}

}  // namespace b200
