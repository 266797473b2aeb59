// Paged KV cache kernels: append and decode attention.
//
// Pool layout (unchanged from the reference, crates/tensor-core/src/paged_kv.rs:17-21):
// K and V pools are [num_blocks, block_size, E_kv] row-major; the token at logical position
// pos of a sequence lives in pool row  block_table[pos / block_size] * block_size + pos % block_size.
// Here E_kv = num_kv_heads * head_dim and the element type is bf16 (or f32, the reference's type).
//
// Replaces paged_kv_append_f32 and paged_attention_f32
// (crates/backend-cuda/src/kernels_paged_kv.rs:55-83, 86-228).  The reference kernel walks the
// keys with one CTA per query row and lets thread 0 do max and sum alone; here the key range of
// a query row is cut into chunks (flash-decoding split-K), each chunk is one CTA fed by a TMA
// ring of 4 KB tiles gathered through the block table, and a second kernel merges the chunks.
#include <mutex>

#include "kernels.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

// ------------------------------------------------------------------------------------ append
template <typename KvT>
__device__ __forceinline__ KvT to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ uint16_t to_kv<uint16_t>(float v) { return static_cast<uint16_t>(f32_to_bf16_bits(v)); }

template <typename KvT>
__global__ void paged_kv_append_kernel(const float* __restrict__ k_new, const float* __restrict__ v_new,
                                       KvT* __restrict__ k_pool, KvT* __restrict__ v_pool,
                                       const uint32_t* __restrict__ slots, int64_t rows, int64_t e, int64_t pool_rows,
                                       uint32_t* err) {
    // one thread per 4 consecutive elements of a row (e % 4 == 0 is checked on the host)
    const int64_t groups_per_row = e / 4;
    const int64_t total = rows * groups_per_row;
    for (int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; g < total; g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = g / groups_per_row;
        const int64_t c = (g % groups_per_row) * 4;
        const int64_t slot = slots[r];
        if (slot >= pool_rows) {   // never write out of range; flag it instead
            atomicCAS(err, 0u, static_cast<uint32_t>(kErrAppendSlot));
            continue;
        }
        const float4 kv = *reinterpret_cast<const float4*>(k_new + r * e + c);
        const float4 vv = *reinterpret_cast<const float4*>(v_new + r * e + c);
        KvT* kd = k_pool + slot * e + c;
        KvT* vd = v_pool + slot * e + c;
        if constexpr (sizeof(KvT) == 4) {
            *reinterpret_cast<float4*>(kd) = kv;
            *reinterpret_cast<float4*>(vd) = vv;
        } else {
            uint2 ko, vo;
            ko.x = f32_to_bf16_bits(kv.x) | (f32_to_bf16_bits(kv.y) << 16);
            ko.y = f32_to_bf16_bits(kv.z) | (f32_to_bf16_bits(kv.w) << 16);
            vo.x = f32_to_bf16_bits(vv.x) | (f32_to_bf16_bits(vv.y) << 16);
            vo.y = f32_to_bf16_bits(vv.z) | (f32_to_bf16_bits(vv.w) << 16);
            *reinterpret_cast<uint2*>(kd) = ko;
            *reinterpret_cast<uint2*>(vd) = vo;
        }
    }
}

// scalar variant for e % 4 != 0
template <typename KvT>
__global__ void paged_kv_append_scalar_kernel(const float* __restrict__ k_new, const float* __restrict__ v_new,
                                              KvT* __restrict__ k_pool, KvT* __restrict__ v_pool,
                                              const uint32_t* __restrict__ slots, int64_t rows, int64_t e,
                                              int64_t pool_rows, uint32_t* err) {
    const int64_t total = rows * e;
    for (int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; g < total; g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = g / e, c = g % e;
        const int64_t slot = slots[r];
        if (slot >= pool_rows) {
            atomicCAS(err, 0u, static_cast<uint32_t>(kErrAppendSlot));
            continue;
        }
        k_pool[slot * e + c] = to_kv<KvT>(k_new[g]);
        v_pool[slot * e + c] = to_kv<KvT>(v_new[g]);
    }
}

// ------------------------------------------------------------------------------------ attention, generic
template <typename KvT>
__device__ __forceinline__ float kv_to_f32(KvT v);
template <>
__device__ __forceinline__ float kv_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float kv_to_f32<uint16_t>(uint16_t v) { return bf16_bits_to_f32(v); }

constexpr int kGenThreads = 128;
constexpr int kGenMaxDimsPerLane = 8;   // head_dim <= 256

// Any head_dim <= 256, any block size, any q:kv head ratio, f32 or bf16 pools.  One CTA per
// (query row, q head); each warp walks tokens warp, warp + 4, ... with an online softmax, lanes
// stride the head dimension; the four warps are merged at the end.  Writes NaN when it meets an
// out-of-range block id (the reference kernel's reaction, kernels_paged_kv.rs:86-228).
//
// Every floating-point step is written as an explicitly rounded operation in a fixed order (no
// compiler contraction, butterfly reductions whose result is the same in every lane, exp_det), so a
// CPU restatement of this order reproduces the output bit for bit:
//   s_j = butterfly_sum over lanes of fma-chain over t of (q[d] * scale) * k_j[d],  d = lane + 32 t
//   m' = max(m, s_j); c = exp(m - m'); p = exp(s_j - m'); l = fma(l, c, p); o[d] = fma(p, v_j[d], o[d] * c)
//   merge of warps w = 0..3 in order: g_w = exp(m_w - max_w m_w); L = fma(l_w, g_w, L); O[d] = fma(o_w[d], g_w, O[d])
//   out[d] = O[d] / L
// A sequence length above max_blocks_per_seq * block_size is clamped and flagged (kErrAttnSeqLen).
template <typename KvT>
__global__ void __launch_bounds__(kGenThreads)
paged_attention_generic_kernel(const float* __restrict__ q, const KvT* __restrict__ k_pool, const KvT* __restrict__ v_pool,
                               const uint32_t* __restrict__ block_tables, const uint32_t* __restrict__ seq_lens,
                               PagedAttnShape sh, float* __restrict__ out, uint32_t* err) {
    __shared__ float red_m[4], red_l[4];
    __shared__ float red_o[4][256];
    const int row = blockIdx.x;              // b * l_new + i
    const int h = blockIdx.y;
    const int b = row / sh.l_new, i = row % sh.l_new;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dh = sh.head_dim;
    const int kvh = h / (sh.num_q_heads / sh.num_kv_heads);
    const int64_t ekv = int64_t(sh.num_kv_heads) * dh;
    int64_t len = seq_lens[b];
    const int64_t cap = int64_t(sh.max_blocks_per_seq) * sh.block_size;
    if (len > cap) {
        if (threadIdx.x == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnSeqLen));
        len = cap;
    }
    const int limit = int(len) - sh.l_new + i + 1;
    const float* q_row = q + (int64_t(row) * sh.num_q_heads + h) * dh;
    float qs[kGenMaxDimsPerLane];
#pragma unroll
    for (int t = 0; t < kGenMaxDimsPerLane; ++t) {
        const int d = lane + 32 * t;
        qs[t] = d < dh ? __fmul_rn(q_row[d], sh.scale) : 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    float acc[kGenMaxDimsPerLane];
#pragma unroll
    for (int t = 0; t < kGenMaxDimsPerLane; ++t) acc[t] = 0.0f;
    bool bad = false;
    for (int j = warp; j < limit; j += 4) {
        const uint32_t blk = block_tables[int64_t(b) * sh.max_blocks_per_seq + j / sh.block_size];
        if (blk >= uint32_t(sh.num_blocks)) { bad = true; break; }
        const int64_t off = (int64_t(blk) * sh.block_size + j % sh.block_size) * ekv + int64_t(kvh) * dh;
        float s = 0.0f;
#pragma unroll
        for (int t = 0; t < kGenMaxDimsPerLane; ++t) {
            const int d = lane + 32 * t;
            if (d < dh) s = __fmaf_rn(qs[t], kv_to_f32<KvT>(k_pool[off + d]), s);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
        const float m_new = fmaxf(m, s);
        const float corr = exp_det(__fsub_rn(m, m_new));      // exp(-inf) = 0 on the first token
        const float p = exp_det(__fsub_rn(s, m_new));
        l = __fmaf_rn(l, corr, p);
#pragma unroll
        for (int t = 0; t < kGenMaxDimsPerLane; ++t) {
            const int d = lane + 32 * t;
            if (d < dh) acc[t] = __fmaf_rn(p, kv_to_f32<KvT>(v_pool[off + d]), __fmul_rn(acc[t], corr));
        }
        m = m_new;
    }
    if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
#pragma unroll
    for (int t = 0; t < kGenMaxDimsPerLane; ++t) {
        const int d = lane + 32 * t;
        if (d < dh) red_o[warp][d] = acc[t];
    }
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    float* o_row = out + (int64_t(row) * sh.num_q_heads + h) * dh;
    if (any_bad) {
        if (threadIdx.x == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnBlockId));
        for (int d = threadIdx.x; d < dh; d += kGenThreads) o_row[d] = __int_as_float(0x7FC00000);
        return;
    }
    float mm = fmaxf(fmaxf(red_m[0], red_m[1]), fmaxf(red_m[2], red_m[3]));
    float w[4], ll = 0.0f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        w[t] = red_m[t] == -INFINITY ? 0.0f : exp_det(__fsub_rn(red_m[t], mm));
        ll = __fmaf_rn(red_l[t], w[t], ll);
    }
    for (int d = threadIdx.x; d < dh; d += kGenThreads) {
        float o = 0.0f;
#pragma unroll
        for (int t = 0; t < 4; ++t) o = __fmaf_rn(red_o[t][d], w[t], o);
        o_row[d] = limit > 0 ? __fdiv_rn(o, ll) : 0.0f;
    }
}

// ------------------------------------------------------------------------------------ attention, fast path
// head_dim 128, bf16 pools, block_size 16, G = q heads per kv head in {1, 2, 4}.
constexpr int kD = 128;
constexpr int kBS = 16;                 // tokens per block = tokens per tile
constexpr int kTileBytes = kBS * kD * 2;  // 4096
constexpr int kConsumerWarps = 4;
constexpr int kStagesPerWarp = 3;       // K and V of one and a half of a warp's blocks in flight
constexpr int kStages = kConsumerWarps * kStagesPerWarp;
constexpr int kFastThreads = 32 * (kConsumerWarps + 1);
constexpr int kMaxChunkBlocks = 256;    // upper bound of blocks per split (tuning range)
constexpr int kDefaultChunkBlocks = 32;
constexpr int kCtasPerSm = 3;           // resident CTAs of the persistent attention kernel per SM

#include "paged_attn_persistent.cuh"

// Merges the chunk partials of one (query row, q head): one warp each, lanes own 4 dims.
__global__ void __launch_bounds__(128)
paged_attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               const uint32_t* __restrict__ seq_lens, PagedAttnShape sh, int chunk_tokens, int max_chunks,
                               float* __restrict__ out, unsigned int* __restrict__ work_counter, uint32_t* err) {
    pdl_wait();
    pdl_launch_dependents();
    // every attention CTA has finished: leave the work counter at zero for the next attention launch
    if (blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t pair = int64_t(blockIdx.x) * 4 + warp;          // row * Hq + h
    const int64_t pairs = int64_t(sh.batch) * sh.l_new * sh.num_q_heads;
    if (pair >= pairs) return;
    const int row = int(pair / sh.num_q_heads);
    const int b = row / sh.l_new, i = row % sh.l_new;
    const int limit = int(seq_lens[b]) - sh.l_new + i + 1;
    int nchunks = limit > 0 ? (limit + chunk_tokens - 1) / chunk_tokens : 0;
    if (nchunks > max_chunks) {       // a length above the planned maximum: never read past the row's partials
        if (lane == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnSeqLen));
        nchunks = max_chunks;
    }
    const float* ml = part_ml + pair * max_chunks * 2;
    float m = -INFINITY;
    for (int c = 0; c < nchunks; ++c) m = fmaxf(m, ml[2 * c]);
    float l = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < nchunks; ++c) {
        const float w = exp2f(ml[2 * c] - m);       // the partial maxima are in log2 units
        l = fmaf(ml[2 * c + 1], w, l);
        const float4 po = *reinterpret_cast<const float4*>(part_o + (pair * max_chunks + c) * kD + lane * 4);
        o.x = fmaf(po.x, w, o.x); o.y = fmaf(po.y, w, o.y); o.z = fmaf(po.z, w, o.z); o.w = fmaf(po.w, w, o.w);
    }
    if (nchunks == 0) l = 1.0f;
    *reinterpret_cast<float4*>(out + pair * kD + lane * 4) = make_float4(o.x / l, o.y / l, o.z / l, o.w / l);
}

// The same merge for a whole query row at once (one warp per q head, at most 32 heads), followed by the
// per-token int8 quantisation of the row [Hq * 128] that the output projection reads: scale = |max| / 127.
// `out` (f32) is written too when it is not null.
__global__ void __launch_bounds__(1024)
paged_attention_combine_quant_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     const uint32_t* __restrict__ seq_lens, PagedAttnShape sh, int chunk_tokens,
                                     int max_chunks, float* __restrict__ out, int8_t* __restrict__ xq,
                                     float* __restrict__ sx, unsigned int* __restrict__ work_counter, uint32_t* err, int fp8) {
    __shared__ float warp_max[32];
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int64_t pair = int64_t(row) * sh.num_q_heads + warp;
    const int b = row / sh.l_new, i = row % sh.l_new;
    const int limit = int(seq_lens[b]) - sh.l_new + i + 1;
    int nchunks = limit > 0 ? (limit + chunk_tokens - 1) / chunk_tokens : 0;
    if (nchunks > max_chunks) {       // a length above the planned maximum: never read past the row's partials
        if (lane == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnSeqLen));
        nchunks = max_chunks;
    }
    const float* ml = part_ml + pair * max_chunks * 2;
    float m = -INFINITY;
    for (int c = 0; c < nchunks; ++c) m = fmaxf(m, ml[2 * c]);
    float l = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < nchunks; ++c) {
        const float w = exp2f(ml[2 * c] - m);
        l = fmaf(ml[2 * c + 1], w, l);
        const float4 po = *reinterpret_cast<const float4*>(part_o + (pair * max_chunks + c) * kD + lane * 4);
        o.x = fmaf(po.x, w, o.x); o.y = fmaf(po.y, w, o.y); o.z = fmaf(po.z, w, o.z); o.w = fmaf(po.w, w, o.w);
    }
    if (nchunks == 0) l = 1.0f;
    const float4 v = make_float4(o.x / l, o.y / l, o.z / l, o.w / l);
    if (out) *reinterpret_cast<float4*>(out + pair * kD + lane * 4) = v;
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < sh.num_q_heads; ++w) amax = fmaxf(amax, warp_max[w]);
    const float scale = fp8 ? amax / kE4m3Max : amax / 127.0f;
    if (threadIdx.x == 0) sx[row] = scale;
    const uint32_t b0 = static_cast<uint32_t>(quant_i8(v.x, scale)) & 0xFFu;
    const uint32_t b1 = static_cast<uint32_t>(quant_i8(v.y, scale)) & 0xFFu;
    const uint32_t b2 = static_cast<uint32_t>(quant_i8(v.z, scale)) & 0xFFu;
    const uint32_t b3 = static_cast<uint32_t>(quant_i8(v.w, scale)) & 0xFFu;
    reinterpret_cast<uint32_t*>(xq + pair * kD)[lane] =
        fp8 ? quant4_e4m3(v.x, v.y, v.z, v.w, scale) : (b0 | (b1 << 8) | (b2 << 16) | (b3 << 24));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// The pool is [pool_rows, E_kv] bf16.  One copy brings a whole [16 tokens x 128 dims] tile of one kv head: the
// map sees the two 64-element halves of a head as a third dimension (stride 128 bytes), so the box
// [64, 16, 2] lands as two [16 x 128-byte] sub-tiles, each written with the 128-byte swizzle.
bool make_pool_map(CUtensorMap* map, const void* pool, int64_t pool_rows, int64_t ekv) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(ekv - kD / 2), static_cast<cuuint64_t>(pool_rows), 2};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ekv) * 2, kD};
    cuuint32_t box[3] = {kD / 2, kBS, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int G>
cudaError_t launch_fast(const PagedAttnPlan& plan, const float* q, const uint32_t* tables, const uint32_t* seq_lens,
                        float* part_o, float* part_ml, unsigned int* work_counter, int sm_count, uint32_t* err,
                        cudaStream_t stream) {
    const int smem = attn_smem_bytes();    // the kernel lays out four head rows whatever G is
    static int configured[64] = {};
    if (cudaError_t e = ensure_dynamic_smem(paged_attention_decode_kernel<G>, smem, configured)) return e;
    const PagedAttnShape& sh = plan.shape;
    const int group = sh.num_q_heads / sh.num_kv_heads;
    const int64_t items = int64_t(sh.num_kv_heads) * (group / G) * plan.max_chunks * sh.batch * sh.l_new;
    const int64_t resident = int64_t(sm_count > 0 ? sm_count : current_sm_count()) * kCtasPerSm;
    dim3 grid(static_cast<unsigned>(items < resident ? items : resident));
    return launch_ex(paged_attention_decode_kernel<G>, grid, dim3(kFastThreads), smem, stream, 1, true, plan.tma_k,
                     plan.tma_v, q, tables, seq_lens, sh, plan.chunk_blocks, plan.max_chunks, part_o, part_ml,
                     work_counter, err);
}

int grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = int64_t(current_sm_count()) * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

}  // namespace

cudaError_t paged_kv_append(const float* k_new, const float* v_new, void* k_pool, void* v_pool, const uint32_t* slots_dev,
                            int64_t rows, int64_t e, int64_t pool_rows, int kv_bf16, uint32_t* err, cudaStream_t s) {
    if (rows == 0 || e == 0) return cudaSuccess;
    const bool vec = (e % 4) == 0;
    const int grid = grid_for(vec ? rows * (e / 4) : rows * e, 256);
    if (kv_bf16) {
        if (vec)
            paged_kv_append_kernel<uint16_t><<<grid, 256, 0, s>>>(k_new, v_new, static_cast<uint16_t*>(k_pool),
                                                                 static_cast<uint16_t*>(v_pool), slots_dev, rows, e, pool_rows, err);
        else
            paged_kv_append_scalar_kernel<uint16_t><<<grid, 256, 0, s>>>(k_new, v_new, static_cast<uint16_t*>(k_pool),
                                                                        static_cast<uint16_t*>(v_pool), slots_dev, rows, e, pool_rows, err);
    } else {
        if (vec)
            paged_kv_append_kernel<float><<<grid, 256, 0, s>>>(k_new, v_new, static_cast<float*>(k_pool),
                                                              static_cast<float*>(v_pool), slots_dev, rows, e, pool_rows, err);
        else
            paged_kv_append_scalar_kernel<float><<<grid, 256, 0, s>>>(k_new, v_new, static_cast<float*>(k_pool),
                                                                     static_cast<float*>(v_pool), slots_dev, rows, e, pool_rows, err);
    }
    return cudaGetLastError();
}

bool paged_attention_fast_path(const PagedAttnShape& sh, int kv_bf16) {
    if (!kv_bf16 || sh.head_dim != kD || sh.block_size != kBS) return false;
    if (sh.num_kv_heads <= 0 || sh.num_q_heads % sh.num_kv_heads != 0) return false;
    const int group = sh.num_q_heads / sh.num_kv_heads;
    return group == 1 || group == 2 || group == 4 || group == 8;
}

cudaError_t paged_attention_make_plan(PagedAttnPlan* plan, const PagedAttnShape& sh, int kv_bf16, const void* k_pool,
                                      const void* v_pool, int max_seq_len, int want_chunk_blocks) {
    plan->shape = sh;
    plan->kv_bf16 = kv_bf16;
    plan->fast = paged_attention_fast_path(sh, kv_bf16) && ((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0) &&
                 ((reinterpret_cast<uintptr_t>(v_pool) & 15) == 0);
    plan->chunk_blocks = 0;
    plan->max_chunks = 0;
    if (!plan->fast) return cudaSuccess;
    // 32 blocks per work item also for small launches: fewer, larger items beat more, smaller ones even when
    // there are fewer items than resident CTAs (measured at 128 rows x 1 KV head: 8 / 16 / 32 blocks ->
    // 0.40 / 0.44 / 0.50 of the HBM peak)
    int cb = want_chunk_blocks > 0 ? want_chunk_blocks : kDefaultChunkBlocks;
    if (cb > kMaxChunkBlocks) cb = kMaxChunkBlocks;
    plan->chunk_blocks = cb;
    const int chunk_tokens = cb * kBS;
    plan->max_chunks = max_seq_len > 0 ? (max_seq_len + chunk_tokens - 1) / chunk_tokens : 1;
    const int64_t pool_rows = int64_t(sh.num_blocks) * sh.block_size;
    const int64_t ekv = int64_t(sh.num_kv_heads) * sh.head_dim;
    if (!make_pool_map(&plan->tma_k, k_pool, pool_rows, ekv) || !make_pool_map(&plan->tma_v, v_pool, pool_rows, ekv))
        return cudaErrorInvalidValue;
    return cudaSuccess;
}

bool paged_attention_can_quantize(const PagedAttnPlan& plan) { return plan.fast && plan.shape.num_q_heads <= 32; }

size_t paged_attention_scratch_bytes(const PagedAttnPlan& plan) {
    if (!plan.fast) return 0;
    const size_t pairs = size_t(plan.shape.batch) * plan.shape.l_new * plan.shape.num_q_heads;
    return pairs * plan.max_chunks * (kD + 2) * sizeof(float);
}

// ------------------------------------------------------------------------------------ static scratch
// Scratch for callers that must not allocate: the split partials of the decode-attention kernel live
// in this file-scope array instead of a cudaMalloc'ed buffer.  Every GPU that loads the library holds
// these 32 MiB until the process exits.  In host code the symbol below is only a stand-in: the device
// address has to be asked for with cudaGetSymbolAddress, once per device, with that device current.
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_attention_static_scratch[kStaticScratchBytes];

size_t paged_attention_static_scratch_capacity() { return kStaticScratchBytes; }

cudaError_t paged_attention_static_scratch(int device, void** out) {
    constexpr int kMaxDevices = 64;
    static void* ptrs[kMaxDevices] = {};
    static std::mutex mu;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[device]) {
        int current = -1;
        cudaError_t e = cudaGetDevice(&current);
        if (e != cudaSuccess) return e;
        if (current != device) return cudaErrorInvalidDevice;   // the caller makes `device` current first
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attention_static_scratch);
        if (e != cudaSuccess) return e;
        ptrs[device] = p;
    }
    *out = ptrs[device];
    return cudaSuccess;
}

cudaError_t paged_attention_launch(const PagedAttnPlan& plan, const float* q, const void* k_pool, const void* v_pool,
                                   const uint32_t* tables_dev, const uint32_t* seq_lens_dev, float* out, void* scratch,
                                   unsigned int* work_counter, int sm_count, uint32_t* err, cudaStream_t stream,
                                   int8_t* xq_out, float* sx_out, int fp8) {
    const PagedAttnShape& sh = plan.shape;
    const int64_t rows = int64_t(sh.batch) * sh.l_new;
    if (rows == 0) return cudaSuccess;
    if (!plan.fast || (reinterpret_cast<uintptr_t>(q) & 15) != 0) {   // the fast kernel bulk-copies 16-byte aligned q rows
        if (xq_out || !out) return cudaErrorInvalidValue;             // only the fast path quantises its output
        dim3 grid(static_cast<unsigned>(rows), sh.num_q_heads);
        if (plan.kv_bf16)
            paged_attention_generic_kernel<uint16_t><<<grid, kGenThreads, 0, stream>>>(
                q, static_cast<const uint16_t*>(k_pool), static_cast<const uint16_t*>(v_pool), tables_dev, seq_lens_dev, sh, out, err);
        else
            paged_attention_generic_kernel<float><<<grid, kGenThreads, 0, stream>>>(
                q, static_cast<const float*>(k_pool), static_cast<const float*>(v_pool), tables_dev, seq_lens_dev, sh, out, err);
        return cudaGetLastError();
    }
    const size_t pairs = size_t(rows) * sh.num_q_heads;
    float* part_o = static_cast<float*>(scratch);
    float* part_ml = part_o + pairs * plan.max_chunks * kD;
    const int group = sh.num_q_heads / sh.num_kv_heads;
    cudaError_t e;
    if (group == 1) e = launch_fast<1>(plan, q, tables_dev, seq_lens_dev, part_o, part_ml, work_counter, sm_count, err, stream);
    else if (group == 2) e = launch_fast<2>(plan, q, tables_dev, seq_lens_dev, part_o, part_ml, work_counter, sm_count, err, stream);
    else e = launch_fast<4>(plan, q, tables_dev, seq_lens_dev, part_o, part_ml, work_counter, sm_count, err, stream);
    if (e != cudaSuccess) return e;
    if (xq_out)
        return launch_ex(paged_attention_combine_quant_kernel, dim3(static_cast<unsigned>(rows)), dim3(32 * sh.num_q_heads),
                         0, stream, 1, true, part_o, part_ml, seq_lens_dev, sh, plan.chunk_blocks * kBS, plan.max_chunks,
                         out, xq_out, sx_out, work_counter, err, fp8);
    const int blocks = static_cast<int>((pairs + 3) / 4);
    return launch_ex(paged_attention_combine_kernel, dim3(blocks), dim3(128), 0, stream, 1, true, part_o, part_ml,
                     seq_lens_dev, sh, plan.chunk_blocks * kBS, plan.max_chunks, out, work_counter, err);
}

}  // namespace b200
