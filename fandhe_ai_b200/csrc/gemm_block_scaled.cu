// INT8 GEMM under the block-scale contract the reference proposes for its quantisation backend
// (docs/int8-quant-grade-up-verification-plan.md:177-241; QuantOps::gemm_i8_s32_scaled,
// docs/backend-int8-quantization-decision.md:88-94):
//
//   out[m, n] = narrow_f32( sum over blocks b ascending, in f64, of widen( f32(s32 partial of block b) * (da[m, b] * db[b, n]) ) )
//
// with blocks of 128 values along K, power-of-two scales da / db, so every step up to the widening is exact and the
// result is a pure function of the inputs: a CPU restatement of the same order matches bit for bit.
//
// One CTA computes a 128 x 64 output tile.  The 128-byte operand stage of the tcgen05 pipeline is exactly one block of
// K, so each stage is multiplied into a FRESH accumulator (two TMEM buffers of 64 columns alternate); the four
// epilogue warps pull every block's s32 partial out of TMEM, scale it and add it to f64 accumulators held in
// registers (64 per thread: thread = output row), while the MMA warp already fills the other buffer.
#include "gemm_tc5.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 64;
constexpr int kBK = 128;        // bytes of K per stage = values per scale block
constexpr int kUmmaK = 32;
constexpr int kThreads = 192;
constexpr int kABytes = kBM * kBK;
constexpr int kBBytes = kBN * kBK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStages = 6;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 8 * (2 * kStages + 4) + 16;

struct BlockScaledArgs {
    int M, N, K;
    int nb;                   // blocks along K
    const float* a_delta;     // [M, nb]
    const float* b_delta;     // [nb, N]
    float* out;               // [M, N]
    uint32_t* status;         // bit 1: a result was not finite
    uint32_t* err;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_block_scaled_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                            BlockScaledArgs p) {
    constexpr uint32_t kIdesc = umma_idesc(1, 2, kBM, kBN);
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + kStages * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tmem_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_dyn + (tmem_slot - smem_u32(smem_dyn)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full(b), 1);
            mbar_init(tmem_empty(b), 128);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * kBN);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM;

    if (warp == 0) {
        if (elect_one()) {
            for (int i = 0; i < p.nb; ++i) {
                const int s = i % kStages;
                if (i >= kStages && !mbar_wait(empty_bar(s), ((i / kStages) & 1) ^ 1u, p.err, kErrProducerWait)) break;
                mbar_arrive_expect_tx(full_bar(s), kStageBytes);
                tma_load_2d(smem_base + s * kStageBytes, &tma_a, full_bar(s), i * kBK, m0);
                tma_load_2d(smem_base + s * kStageBytes + kABytes, &tma_b, full_bar(s), i * kBK, n0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            for (int i = 0; i < p.nb; ++i) {
                const int s = i % kStages, buf = i & 1;
                if (!mbar_wait(tmem_empty(buf), (((i >> 1) & 1) ^ 1u), p.err, kErrMmaWait)) break;
                if (!mbar_wait(full_bar(s), (i / kStages) & 1, p.err, kErrMmaWait)) break;
                tc5_fence_after();
                const uint32_t a_src = smem_base + s * kStageBytes;
                const uint64_t adesc = umma_desc_k128(a_src);
                const uint64_t bdesc = umma_desc_k128(a_src + kABytes);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k)      // a fresh accumulator for every block of K
                    umma_ss<true>(tmem_base + static_cast<uint32_t>(buf * kBN), adesc + 2u * k, bdesc + 2u * k, kIdesc, k != 0 ? 1u : 0u);
                tc5_commit(empty_bar(s));
                tc5_commit(tmem_full(buf));
            }
        }
    } else {
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        const bool row_ok = row < p.M;
        const float* da_row = p.a_delta + static_cast<size_t>(row_ok ? row : 0) * p.nb;
        double acc[kBN];
#pragma unroll
        for (int j = 0; j < kBN; ++j) acc[j] = 0.0;
        bool ok = true;
        for (int i = 0; i < p.nb; ++i) {
            const int buf = i & 1;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(tmem_full(buf), (i >> 1) & 1, p.err, kErrEpilogueWait)) != 0;
            tc5_fence_after();
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(buf * kBN) + (static_cast<uint32_t>(q * 32) << 16);
            uint32_t v0[32], v1[32];
            tmem_ld_32x32(t_row, v0);
            tmem_ld_32x32(t_row + 32, v1);
            const float da = da_row[i];
            const float* db = p.b_delta + static_cast<size_t>(i) * p.N + n0;
            tmem_ld_wait();
            tc5_fence_before();
            mbar_arrive(tmem_empty(buf));          // the values are in registers: the MMA warp may refill the buffer
            if (!ok) continue;
#pragma unroll
            for (int j = 0; j < kBN; ++j) {
                if (n0 + j < p.N) {
                    // composed scale first (exact: both are powers of two), one multiplication, widen, add
                    const float dout = __fmul_rn(da, __ldg(db + j));
                    const int part = static_cast<int>(j < 32 ? v0[j & 31] : v1[j & 31]);
                    const float val = __fmul_rn(__int2float_rn(part), dout);
                    acc[j] = __dadd_rn(acc[j], static_cast<double>(val));
                }
            }
        }
        if (row_ok && ok) {
            bool finite = true;
            float* dst = p.out + static_cast<size_t>(row) * p.N + n0;
#pragma unroll
            for (int j = 0; j < kBN; j += 4) {
                if (n0 + j < p.N) {       // N is a multiple of 16: groups of four are whole
                    const float4 y = make_float4(__double2float_rn(acc[j]), __double2float_rn(acc[j + 1]),
                                                 __double2float_rn(acc[j + 2]), __double2float_rn(acc[j + 3]));
                    finite = finite && isfinite(y.x) && isfinite(y.y) && isfinite(y.z) && isfinite(y.w);
                    *reinterpret_cast<float4*>(dst + j) = y;
                }
            }
            if (!finite) atomicOr(p.status, 2u);
        }
    }
    tc5_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc5_fence_after();
        tmem_dealloc(tmem_base, 2 * kBN);
    }
}

}  // namespace

cudaError_t gemm_i8_block_scaled(const void* a, const float* a_delta, const void* b, const float* b_delta, int M, int N, int K,
                                 float* out, uint32_t* status, uint32_t* err, cudaStream_t stream, const char** why) {
    static const char* kNone = "";
    if (why) *why = kNone;
    auto fail = [&](const char* msg) {
        if (why) *why = msg;
        return cudaErrorInvalidValue;
    };
    if (M <= 0 || N <= 0 || K <= 0) return fail("gemm_i8_block_scaled: m, n, k must be positive");
    if (K % 16 != 0 || N % 16 != 0) return fail("gemm_i8_block_scaled: n and k must be multiples of 16");
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail("gemm_i8_block_scaled: operand and output addresses must be 16-byte aligned");
    CUtensorMap tma_a, tma_b;
    if (!gemm_make_operand_map(&tma_a, a, M, K, kBM)) return fail("gemm_i8_block_scaled: cuTensorMapEncodeTiled failed for A");
    if (!gemm_make_operand_map(&tma_b, b, N, K, kBN)) return fail("gemm_i8_block_scaled: cuTensorMapEncodeTiled failed for B");
    static int configured[64] = {};
    if (cudaError_t e = ensure_dynamic_smem(gemm_i8_block_scaled_kernel, kSmemBytes, configured)) return e;
    BlockScaledArgs args{M, N, K, (K + kBK - 1) / kBK, a_delta, b_delta, out, status, err};
    dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
    return launch_ex(gemm_i8_block_scaled_kernel, grid, dim3(kThreads), kSmemBytes, stream, 1, false, tma_a, tma_b, args);
}

}  // namespace b200
