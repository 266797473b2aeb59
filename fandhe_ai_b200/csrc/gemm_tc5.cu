// tcgen05 / TMEM quantized GEMM for sm_100a.
//
// One CTA computes a 128 x BN accumulator tile (optionally over a slice of K).
// Warp roles: warp 0 = TMA producer (one elected lane), warp 1 = TMEM owner and
// MMA issuer (one elected lane), warps 2..5 = epilogue (each reads the 32 TMEM
// lanes of its quarter).  Operand tiles are K-major with 128-byte rows, written
// by TMA with the 128-byte swizzle and consumed by tcgen05.mma through
// shared-memory descriptors; a ring of `stages` buffers is handed back and forth
// with full/empty mbarriers; the accumulator lives in TMEM until the epilogue
// pulls it out with tcgen05.ld.
//
// Replaces, for the quantized path, the reference's fused GEMM kernels
// gemm_tiled_bias_act_f32 (crates/backend-cuda/src/kernels.rs:368-477) and
// gemm_mma_f16 (crates/backend-cuda/src/kernels_mma.rs:227-375).
#include <cooperative_groups.h>

#include <cstdlib>

#include "gemm_tc5.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kBM = 128;      // accumulator rows per CTA = TMEM lanes
constexpr int kBK = 128;       // operand bytes along K per stage (one swizzle row)
constexpr int kUmmaK = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int kThreads = 192;
constexpr int kABytes = kBM * kBK;

struct KernelArgs {
    int M, N, K;
    int stages;
    int kb_total;        // ceil(K / kBK)
    int kb_per_split;
    int gate;            // B tile = bn/2 gate rows + bn/2 up rows
    int n_half;          // N / 2 in the gate form
    int cluster_reduce;  // the splits of a tile form a cluster and reduce through distributed shared memory
    GemmEpilogue ep;
    uint32_t* err;
};

template <bool kInt8>
__device__ __forceinline__ float acc_to_f32(uint32_t v) {
    if constexpr (kInt8) return static_cast<float>(static_cast<int32_t>(v));
    return __uint_as_float(v);
}

__device__ __forceinline__ void store_out4(const GemmEpilogue& ep, size_t idx, float y0, float y1, float y2, float y3) {
    if (ep.residual) {
        const float4 r = *reinterpret_cast<const float4*>(ep.residual + idx);
        y0 += r.x; y1 += r.y; y2 += r.z; y3 += r.w;
    }
    if (ep.out_bf16) {
        uint2 o;
        o.x = f32_to_bf16_bits(y0) | (f32_to_bf16_bits(y1) << 16);
        o.y = f32_to_bf16_bits(y2) | (f32_to_bf16_bits(y3) << 16);
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(ep.out) + idx) = o;
    } else {
        *reinterpret_cast<float4*>(static_cast<float*>(ep.out) + idx) = make_float4(y0, y1, y2, y3);
    }
}

// Four finished accumulators of (row, columns n .. n + 3): raw store into the single output plane, or the
// fused epilogue (not the gate form).
// First element of output row `row` when the rows are scattered over the ranks' exchange blocks (GemmPush).
__device__ __forceinline__ float* push_row(const GemmPush& ps, int row, int N) {
    const int owner = row / ps.rows;
    return reinterpret_cast<float*>(ps.peers[owner] + ps.o_part) +
           (static_cast<size_t>(ps.rank) * ps.rows + (row - owner * ps.rows)) * N;
}

// Called by one warp of a tile's first CTA after a CTA or cluster barrier that follows the tile's stores (see
// GemmPush): counts the tile; the warp that completes the launch tells every rank.  The barrier, the device-scope
// fences around the local counter and the system-scope fence and release of the last warp order every store of the
// launch before the count that the owners acquire.
__device__ __forceinline__ void push_signal(const GemmPush& ps, int lane, unsigned int tiles) {
    unsigned int last = 0;
    if (lane == 0) {
        __threadfence();
        last = atomicAdd(ps.arrived, 1u) == tiles - 1u ? 1u : 0u;
        if (last) {
            __threadfence();
            *ps.arrived = 0u;
        }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last && lane < ps.tp) {
        __threadfence_system();
        red_release_sys_add(reinterpret_cast<uint32_t*>(ps.peers[lane] + ps.o_count) + ps.rank, 1u);
    }
}

template <bool kInt8>
__device__ __forceinline__ void emit4(const KernelArgs& p, int row, int n, const uint32_t (&v)[4], float* pushed = nullptr) {
    const GemmEpilogue& ep = p.ep;
    if (!ep.fused) {
        *reinterpret_cast<uint4*>(static_cast<uint32_t*>(ep.raw) + static_cast<size_t>(row) * p.N + n) =
            make_uint4(v[0], v[1], v[2], v[3]);
        return;
    }
    const float sa = ep.a_scale[ep.a_per_row ? row : 0];
    float y[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const float sb = ep.b_scale[ep.b_per_col ? n + t : 0];
        const float b = ep.bias ? ep.bias[n + t] : 0.0f;
        float x = fmaf(acc_to_f32<kInt8>(v[t]), sa * sb, b);
        if (ep.act == kActSilu) x = silu(x);
        else if (ep.act == kActRelu) x = fmaxf(x, 0.0f);
        y[t] = x;
    }
    if (pushed) {
        *reinterpret_cast<float4*>(pushed + n) = make_float4(y[0], y[1], y[2], y[3]);
        return;
    }
    store_out4(ep, static_cast<size_t>(row) * p.N + n, y[0], y[1], y[2], y[3]);
}

// kAux selects one of three instantiations: 0 the plain kernel; 1 the rows are scattered over the GPUs (GemmPush);
// 2 the first CTA stamps %globaltimer (GemmEpilogue::stamps).  Template parameters, not run-time flags: the mere
// presence of either path cost the plain decode GEMMs 0.09 + 0.04 ms per 8B-shape step (measured on one GPU).
constexpr int kAuxNone = 0, kAuxPush = 1, kAuxStamps = 2;

template <int BN, bool kInt8, int kAux>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, KernelArgs p) {
    constexpr int kBBytes = BN * kBK;
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr uint32_t kTmemCols = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;     // a power of two
    constexpr uint32_t kIdesc = kInt8 ? umma_idesc(1, 2, kBM, BN) : umma_idesc(0, 1, kBM, BN);
    constexpr int kPartPitch = BN + 4;          // words per row of a partial tile parked for the cluster reduction

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + p.stages * kStageBytes;   // full[s], empty[s], tmem_full, tmem slot
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (p.stages + s); };
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * p.stages);
    const uint32_t tmem_slot = tmem_full_bar + 8u;
    // generic pointer to the TMEM-address slot
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_dyn + (tmem_slot - smem_u32(smem_dyn)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool stamping = kAux == kAuxStamps && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    constexpr bool pushing = kAux == kAuxPush;     // the rows go to their owner ranks (GemmPush)
    auto stamp = [&](int i) {
        if constexpr (kAux == kAuxStamps) {
            if (stamping) p.ep.stamps[i] = global_timer_ns();
        }
    };
    if (threadIdx.x == 0) stamp(kGemmStampEntry);

    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    if (threadIdx.x == 0) stamp(kGemmStampSetup);

    const int out_cols = p.gate ? BN / 2 : BN;          // output columns per CTA
    const int n0 = blockIdx.x * out_cols;               // first output column
    const int m0 = blockIdx.y * kBM;
    const int split = blockIdx.z;
    const int kb_begin = split * p.kb_per_split;
    int kb_end = kb_begin + p.kb_per_split;
    if (kb_end > p.kb_total) kb_end = p.kb_total;
    const int num_kb = kb_end > kb_begin ? kb_end - kb_begin : 0;

    if (warp == 0) {
        const bool leader = elect_one();
        if (p.ep.wait.flags != nullptr) {
            // The A operand comes from other GPUs: the leader puts the weight tiles of the first ring pass in flight,
            // then the lanes wait for the peers' flags (one flag per lane) and only then the A tiles are loaded.
            if (leader) {
                const int pre = num_kb < p.stages ? num_kb : p.stages;
                for (int i = 0; i < pre; ++i) {
                    mbar_arrive_expect_tx(full_bar(i), kStageBytes);
                    const uint32_t b_dst = smem_base + i * kStageBytes + kABytes;
                    const int kx = (kb_begin + i) * kBK;
                    tma_load_2d(b_dst, &tma_b, full_bar(i), kx, n0);
                    if (p.gate) tma_load_2d(b_dst + (BN / 2) * kBK, &tma_b, full_bar(i), kx, p.n_half + n0);
                }
            }
            __syncwarp();
            pdl_wait();
            if (lane < p.ep.wait.n) wait_peer_flag(p.ep.wait.flags + lane, *p.ep.wait.epoch, p.err, p.ep.wait.timeout_ns);
            __syncwarp();
        }
        if (leader) {
            const bool b_in_flight = p.ep.wait.flags != nullptr;
            if (b_in_flight) fence_proxy_async_all();
            auto load_b = [&](int i, int s) {
                const uint32_t b_dst = smem_base + s * kStageBytes + kABytes;
                const int kx = (kb_begin + i) * kBK;
                tma_load_2d(b_dst, &tma_b, full_bar(s), kx, n0);
                if (p.gate) tma_load_2d(b_dst + (BN / 2) * kBK, &tma_b, full_bar(s), kx, p.n_half + n0);
            };
            auto load_a = [&](int i, int s) {
                tma_load_2d(smem_base + s * kStageBytes, &tma_a, full_bar(s), (kb_begin + i) * kBK, m0);
            };
            // The B operand (weights) does not depend on the kernel that runs before this one: fill the first
            // pass over the ring with B tiles while that kernel still drains, then wait for it and add the A tiles.
            const int pre = num_kb < p.stages ? num_kb : p.stages;
            if (!b_in_flight) {
                for (int i = 0; i < pre; ++i) {
                    mbar_arrive_expect_tx(full_bar(i), kStageBytes);
                    load_b(i, i);
                }
                pdl_wait();
            }
            stamp(kGemmStampDepWait);
            pdl_launch_dependents();
            for (int i = 0; i < pre; ++i) load_a(i, i);
            stamp(kGemmStampLoadsIssued);
            for (int i = pre; i < num_kb; ++i) {
                const int s = i % p.stages;
                const uint32_t ph = (i / p.stages) & 1;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, p.err, kErrProducerWait)) break;
                mbar_arrive_expect_tx(full_bar(s), kStageBytes);
                load_a(i, s);
                load_b(i, s);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            bool ok = true;
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % p.stages;
                const uint32_t ph = (i / p.stages) & 1;
                ok = mbar_wait(full_bar(s), ph, p.err, kErrMmaWait);
                if (!ok) break;
                if (i == 0) stamp(kGemmStampFirstTile);
                tc5_fence_after();
                const uint32_t a_src = smem_base + s * kStageBytes;
                const uint64_t adesc = umma_desc_k128(a_src);
                const uint64_t bdesc = umma_desc_k128(a_src + kABytes);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k) {
                    // advance both descriptors by 32 bytes along K inside the swizzle row
                    umma_ss<kInt8>(tmem_base, adesc + 2u * k, bdesc + 2u * k, kIdesc, (i | k) != 0 ? 1u : 0u);
                }
                tc5_commit(empty_bar(s));
            }
            tc5_commit(tmem_full_bar);
            stamp(kGemmStampMmaIssued);
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        const bool row_ok = row < p.M;
        pdl_wait();      // scales, bias, residual and the output buffers belong to the surrounding kernels
        bool ready = num_kb > 0 && mbar_wait(tmem_full_bar, 0, p.err, kErrEpilogueWait);
        tc5_fence_after();
        if (warp == 2 && lane == 0) stamp(kGemmStampAccReady);
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        const GemmEpilogue& ep = p.ep;
        if (ready && p.cluster_reduce) {
            // park this CTA's partial tile in its own shared memory, column-major ([col][row]): the operand ring
            // is idle by now (every MMA has completed), consecutive threads hold consecutive rows
            uint32_t* part = reinterpret_cast<uint32_t*>(smem_dyn + (smem_base - smem_u32(smem_dyn)));
            const int rl = q * 32 + lane;
            if (!pushing) {
                // column-major ([col][row]): consecutive threads hold consecutive rows, 4-byte accesses without bank conflicts
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) part[(c0 + j) * kBM + rl] = v[j];
                }
            } else {
                // the rows will be scattered over the GPUs: row-major with a pitch of BN + 4 words (the 16-byte stores of
                // eight neighbouring rows fall into different banks), so that the reduction below reads and then stores
                // whole row segments
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4*>(part + rl * kPartPitch + c0 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        } else if (ready) {
            if (!ep.fused) {
                uint32_t* raw = static_cast<uint32_t*>(ep.raw) +
                                (static_cast<size_t>(split) * p.M + (row_ok ? row : 0)) * p.N;
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const int n = n0 + c0 + j;
                            if (n < p.N) *reinterpret_cast<uint4*>(raw + n) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        }
                    }
                }
            } else if (!p.gate) {
                const float sa = ep.a_scale[ep.a_per_row ? (row_ok ? row : 0) : 0];
                const size_t row_off = static_cast<size_t>(row_ok ? row : 0) * p.N;
                float* pushed = pushing && row_ok ? push_row(ep.push, row, p.N) : nullptr;
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const int n = n0 + c0 + j;
                            if (n >= p.N) break;
                            float y[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float sb = ep.b_scale[ep.b_per_col ? n + t : 0];
                                const float b = ep.bias ? ep.bias[n + t] : 0.0f;
                                float x = fmaf(acc_to_f32<kInt8>(v[j + t]), sa * sb, b);
                                if (ep.act == kActSilu) x = silu(x);
                                else if (ep.act == kActRelu) x = fmaxf(x, 0.0f);
                                y[t] = x;
                            }
                            if (pushed) *reinterpret_cast<float4*>(pushed + n) = make_float4(y[0], y[1], y[2], y[3]);
                            else store_out4(ep, row_off + n, y[0], y[1], y[2], y[3]);
                        }
                    }
                }
            } else {
                // gate form: columns [0, BN/2) hold gate, [BN/2, BN) hold up, for outputs n0 .. n0 + BN/2
                const float sa = ep.a_scale[ep.a_per_row ? (row_ok ? row : 0) : 0];
                const size_t row_off = static_cast<size_t>(row_ok ? row : 0) * p.n_half;
                constexpr int kHalf = BN / 2;
                constexpr int kStep = kHalf < 32 ? kHalf : 32;
                for (int c0 = 0; c0 < kHalf; c0 += 32) {
                    if (n0 + c0 >= p.n_half) break;
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_row + c0, g);
                    tmem_ld_32x32(t_row + kHalf + c0, u);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < kStep; j += 4) {
                            const int n = n0 + c0 + j;
                            if (n >= p.n_half) break;
                            float y[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float sg = ep.b_scale[ep.b_per_col ? n + t : 0];
                                const float su = ep.b_scale[ep.b_per_col ? p.n_half + n + t : 0];
                                const float bg = ep.bias ? ep.bias[n + t] : 0.0f;
                                const float bu = ep.bias ? ep.bias[p.n_half + n + t] : 0.0f;
                                const float gv = fmaf(acc_to_f32<kInt8>(g[j + t]), sa * sg, bg);
                                const float uv = fmaf(acc_to_f32<kInt8>(u[j + t]), sa * su, bu);
                                y[t] = silu(gv) * uv;
                            }
                            store_out4(ep, row_off + n, y[0], y[1], y[2], y[3]);
                        }
                    }
                }
            }
        }
    }

    if (p.cluster_reduce) {
        // Split-K inside a cluster: the `splits` CTAs of one output tile exchange their partial tiles through
        // distributed shared memory; CTA `rank` sums a slice of BN / splits columns over all peers in rank
        // order (exact for int32, fixed order for f32) and writes the finished values, so only one plane
        // leaves the kernel.  Both barriers are reached by every thread on every path.
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();
        if (warp >= 2) {
            const int nsplit = static_cast<int>(cl.num_blocks());
            const int rank = static_cast<int>(cl.block_rank());
            const int cpr = BN / nsplit;                   // columns per rank, a multiple of 4
            const int rl = (warp & 3) * 32 + lane;
            const int row = m0 + rl;
            uint32_t* part = reinterpret_cast<uint32_t*>(smem_dyn + (smem_base - smem_u32(smem_dyn)));
            if (p.ep.rope.enabled) {
                // One tile = one head.  This rank finishes the dims [rank * cpr / 2, (rank + 1) * cpr / 2) and their
                // rotation partners 64 further on: sum over the peers, dequantise, rotate (q and k heads), store.
                const GemmRope& rp = p.ep.rope;
                const int half_cpr = cpr / 2;
                const int head = n0 / BN;
                bool ok = row < p.M;
                int pos = 0;
                uint32_t blk = 0;
                if (ok) {
                    pos = static_cast<int>(rp.positions[row]);
                    bool valid = pos < rp.max_pos;
                    if (valid) {
                        blk = rp.block_tables[static_cast<size_t>(row) * rp.max_blocks_per_seq + pos / rp.block_size];
                        valid = blk < static_cast<uint32_t>(rp.num_blocks);
                    }
                    if (!valid) {
                        atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrAppendSlot));
                        ok = false;
                    }
                }
                const float sa = ok ? p.ep.a_scale[row] : 0.0f;
                const bool keep_kv = ok && (rp.active == nullptr || rp.active[row] != 0u);   // a row that sits the step out
                const float* cr = rp.cos_t + static_cast<size_t>(pos) * 64;
                const float* sr = rp.sin_t + static_cast<size_t>(pos) * 64;
                const size_t slot = static_cast<size_t>(blk) * rp.block_size + pos % rp.block_size;
                for (int cc = 0; cc < half_cpr; cc += 4) {
                    const int i0 = rank * half_cpr + cc;
                    // partial sums over the K slices in rank order: int32 (exact), or f32 for FP8 operands
                    uint32_t lo[4] = {0u, 0u, 0u, 0u}, hi[4] = {0u, 0u, 0u, 0u};
                    for (int peer = 0; peer < nsplit; ++peer) {
                        const uint32_t* pp = cl.map_shared_rank(part, peer);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint32_t a = pp[(i0 + t) * kBM + rl], b = pp[(64 + i0 + t) * kBM + rl];
                            if constexpr (kInt8) {
                                lo[t] += a;
                                hi[t] += b;
                            } else {
                                lo[t] = __float_as_uint(__uint_as_float(lo[t]) + __uint_as_float(a));
                                hi[t] = __float_as_uint(__uint_as_float(hi[t]) + __uint_as_float(b));
                            }
                        }
                    }
                    if (!ok) continue;
                    float o1[4], o2[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float x1 = fmaf(acc_to_f32<kInt8>(lo[t]), sa * p.ep.b_scale[head * BN + i0 + t], 0.0f);
                        const float x2 = fmaf(acc_to_f32<kInt8>(hi[t]), sa * p.ep.b_scale[head * BN + 64 + i0 + t], 0.0f);
                        if (head < rp.hq + rp.hkv) {
                            const float c = cr[i0 + t], sn = sr[i0 + t];
                            o1[t] = fmaf(x1, c, -__fmul_rn(x2, sn));
                            o2[t] = fmaf(x2, c, __fmul_rn(x1, sn));
                        } else {
                            o1[t] = x1;
                            o2[t] = x2;
                        }
                    }
                    if (head < rp.hq) {
                        float* dst = rp.q_out + (static_cast<size_t>(row) * rp.hq + head) * BN + i0;
                        *reinterpret_cast<float4*>(dst) = make_float4(o1[0], o1[1], o1[2], o1[3]);
                        *reinterpret_cast<float4*>(dst + 64) = make_float4(o2[0], o2[1], o2[2], o2[3]);
                    } else if (keep_kv) {
                        const bool is_k = head < rp.hq + rp.hkv;
                        const int kh = is_k ? head - rp.hq : head - rp.hq - rp.hkv;
                        uint16_t* dst = (is_k ? rp.k_pool : rp.v_pool) + (slot * rp.hkv + kh) * BN + i0;
                        uint2 a, b;
                        a.x = f32_to_bf16_bits(o1[0]) | (f32_to_bf16_bits(o1[1]) << 16);
                        a.y = f32_to_bf16_bits(o1[2]) | (f32_to_bf16_bits(o1[3]) << 16);
                        b.x = f32_to_bf16_bits(o2[0]) | (f32_to_bf16_bits(o2[1]) << 16);
                        b.y = f32_to_bf16_bits(o2[2]) | (f32_to_bf16_bits(o2[3]) << 16);
                        *reinterpret_cast<uint2*>(dst) = a;
                        *reinterpret_cast<uint2*>(dst + 64) = b;
                    }
                }
            } else if (!pushing) {
                // CTA `rank` finishes a slice of BN / nsplit columns of all rows
                for (int cc = 0; cc < cpr; cc += 4) {
                    const int col = rank * cpr + cc;
                    uint32_t v[4] = {0u, 0u, 0u, 0u};
                    for (int peer = 0; peer < nsplit; ++peer) {
                        const uint32_t* pp = cl.map_shared_rank(part, peer);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint32_t x = pp[(col + t) * kBM + rl];
                            if constexpr (kInt8) v[t] += x;    // two's complement wrap = int32 addition
                            else v[t] = __float_as_uint(__uint_as_float(v[t]) + __uint_as_float(x));
                        }
                    }
                    const int n = n0 + col;
                    if (row < p.M && n < p.N) emit4<kInt8>(p, row, n, v);
                }
            } else {
                // Scattered output: CTA `rank` finishes the rows [rank * kBM / nsplit, (rank + 1) * kBM / nsplit) of the tile,
                // all BN columns, sixteen bytes per thread and consecutive threads along a row, so that the owner's memory
                // receives whole row segments (16-byte stores into 32 different rows per instruction cost 1.1 ms per
                // 8B-shape decode step on two GPUs)
                const int rows_per = kBM / nsplit;
                constexpr int kGroups = BN / 4;
                const int total = rows_per * kGroups;
                for (int idx = (warp - 2) * 32 + lane; idx < total; idx += 128) {
                    const int r_tile = rank * rows_per + idx / kGroups;     // row inside the tile
                    const int col = 4 * (idx % kGroups);
                    uint32_t v[4] = {0u, 0u, 0u, 0u};
                    for (int peer = 0; peer < nsplit; ++peer) {
                        const uint4 x = *reinterpret_cast<const uint4*>(cl.map_shared_rank(part, peer) + r_tile * kPartPitch + col);
                        if constexpr (kInt8) {       // two's complement wrap = int32 addition
                            v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
                        } else {
                            v[0] = __float_as_uint(__uint_as_float(v[0]) + __uint_as_float(x.x));
                            v[1] = __float_as_uint(__uint_as_float(v[1]) + __uint_as_float(x.y));
                            v[2] = __float_as_uint(__uint_as_float(v[2]) + __uint_as_float(x.z));
                            v[3] = __float_as_uint(__uint_as_float(v[3]) + __uint_as_float(x.w));
                        }
                    }
                    const int out_row = m0 + r_tile;
                    const int n = n0 + col;
                    if (out_row < p.M && n < p.N) emit4<kInt8>(p, out_row, n, v, push_row(p.ep.push, out_row, p.N));
                }
            }
        }
        cl.sync();
        // every CTA of the cluster has stored its rows of the tile: the first one counts the tile
        if (pushing && warp == 2 && cl.block_rank() == 0) push_signal(p.ep.push, lane, gridDim.x * gridDim.y);
    }

    if (warp == 2 && lane == 0) stamp(kGemmStampStored);      // this warp's part of the tile is stored
    tc5_fence_before();
    __syncthreads();
    if (pushing && !p.cluster_reduce && warp == 2) push_signal(p.ep.push, lane, gridDim.x * gridDim.y);
    if (warp == 1) {
        __syncwarp();
        tc5_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
        if (lane == 0) stamp(kGemmStampExit);
    }
}

#include "gemm_tc5_persist.cuh"

// Sums the split-K partial planes in plane order and applies the same epilogue as the
// fused path.  One thread per four output columns.
template <bool kInt8>
__global__ void splitk_epilogue_kernel(const uint32_t* __restrict__ raw, int splits, int M, int N, int gate,
                                       GemmEpilogue ep) {
    const int n_out = gate ? N / 2 : N;
    const int64_t groups = static_cast<int64_t>(M) * (n_out / 4);
    const size_t plane = static_cast<size_t>(M) * N;
    for (int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; g < groups; g += int64_t(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(g / (n_out / 4));
        const int n = static_cast<int>(g % (n_out / 4)) * 4;
        const float sa = ep.a_scale[ep.a_per_row ? m : 0];
        float y[4];
        auto total = [&](int col, float* out4) {
            const uint32_t* src = raw + static_cast<size_t>(m) * N + col;
            if constexpr (kInt8) {
                int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
                for (int s = 0; s < splits; ++s) {
                    const uint4 v = *reinterpret_cast<const uint4*>(src + s * plane);
                    a0 += static_cast<int>(v.x); a1 += static_cast<int>(v.y);
                    a2 += static_cast<int>(v.z); a3 += static_cast<int>(v.w);
                }
                out4[0] = static_cast<float>(a0); out4[1] = static_cast<float>(a1);
                out4[2] = static_cast<float>(a2); out4[3] = static_cast<float>(a3);
            } else {
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                for (int s = 0; s < splits; ++s) {
                    const uint4 v = *reinterpret_cast<const uint4*>(src + s * plane);
                    a0 += __uint_as_float(v.x); a1 += __uint_as_float(v.y);
                    a2 += __uint_as_float(v.z); a3 += __uint_as_float(v.w);
                }
                out4[0] = a0; out4[1] = a1; out4[2] = a2; out4[3] = a3;
            }
        };
        if (!gate) {
            float t[4];
            total(n, t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float sb = ep.b_scale[ep.b_per_col ? n + i : 0];
                const float b = ep.bias ? ep.bias[n + i] : 0.0f;
                float x = fmaf(t[i], sa * sb, b);
                if (ep.act == kActSilu) x = silu(x);
                else if (ep.act == kActRelu) x = fmaxf(x, 0.0f);
                y[i] = x;
            }
        } else {
            float tg[4], tu[4];
            total(n, tg);
            total(n_out + n, tu);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float sg = ep.b_scale[ep.b_per_col ? n + i : 0];
                const float su = ep.b_scale[ep.b_per_col ? n_out + n + i : 0];
                const float bg = ep.bias ? ep.bias[n + i] : 0.0f;
                const float bu = ep.bias ? ep.bias[n_out + n + i] : 0.0f;
                y[i] = silu(fmaf(tg[i], sa * sg, bg)) * fmaf(tu[i], sa * su, bu);
            }
        }
        store_out4(ep, static_cast<size_t>(m) * n_out + n, y[0], y[1], y[2], y[3]);
    }
}

// Sums int32 partial planes in plane order (integer addition: exact, order-free).
__global__ void sum_planes_i32_kernel(const int* __restrict__ raw, int splits, int64_t elems, int* __restrict__ out) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < elems; i += int64_t(gridDim.x) * blockDim.x) {
        int a = 0;
        for (int s = 0; s < splits; ++s) a += raw[s * elems + i];
        out[i] = a;
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess) {
            sym = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// 2-D map over a row-major [rows, cols] matrix of bytes, box = [box_rows, 128 bytes], 128-byte swizzle.
bool make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tensor map of an output plane [rows, cols] of 4-byte (f32 / raw accumulators) or 2-byte (bf16) elements for TMA
// stores of 32 x 32 boxes whose shared-memory rows (128 or 64 bytes) are swizzled over their own width.
bool make_out_map(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, int elem_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, elem_bytes == 4 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int BN, bool kInt8, int kAux>
cudaError_t launch_aux_t(const GemmPlan& plan, const KernelArgs& args, cudaStream_t stream) {
    const int stage_bytes = kABytes + BN * kBK;
    const int smem = plan.stages * stage_bytes + 1024 + 8 * (2 * plan.stages + 2);
    static int configured[64] = {};
    if (cudaError_t e = ensure_dynamic_smem(gemm_tc5_kernel<BN, kInt8, kAux>, smem, configured)) return e;
    const int out_cols = plan.gate ? BN / 2 : BN;
    const int n_out = plan.gate ? plan.N / 2 : plan.N;
    dim3 grid((n_out + out_cols - 1) / out_cols, (plan.M + kBM - 1) / kBM, plan.splits);
    return launch_ex_z(gemm_tc5_kernel<BN, kInt8, kAux>, grid, dim3(kThreads), smem, stream, plan.cluster ? plan.splits : 1, true,
                       plan.tma_a, plan.tma_b, args);
}

template <int BN, bool kInt8>
cudaError_t launch_t(const GemmPlan& plan, const KernelArgs& args, cudaStream_t stream) {
    if (args.ep.push.peers != nullptr) {
        if (args.ep.stamps != nullptr) return cudaErrorInvalidValue;
        return launch_aux_t<BN, kInt8, kAuxPush>(plan, args, stream);
    }
    if (args.ep.stamps != nullptr) {
        if constexpr (kInt8) return launch_aux_t<BN, true, kAuxStamps>(plan, args, stream);
        else return cudaErrorInvalidValue;          // the stamping instantiation exists for int8 operands
    }
    return launch_aux_t<BN, kInt8, kAuxNone>(plan, args, stream);
}

constexpr int kMaxSmem = 232448;   // dynamic shared memory a CTA may ask for on sm_100

template <int BN, bool kInt8, bool kPair>
cudaError_t launch_persist_t(const GemmPlan& plan, PersistArgs args, cudaStream_t stream) {
    const int stage_bytes = kABytes + (kPair ? BN / 2 : BN) * kBK;
    // Output through shared memory and TMA stores when the plane allows it (16-byte aligned base and row pitch); the
    // staging buffers may cost the operand ring a stage.
    CUtensorMap tma_out = plan.tma_a;      // placeholder when the stores stay per thread
    const GemmEpilogue& ep = args.ep;
    void* out = ep.fused ? ep.out : ep.raw;
    const int elem = ep.fused && ep.out_bf16 ? 2 : 4;
    const int n_out = plan.gate ? plan.N / 2 : plan.N;
    static const bool tma_store_allowed = [] {
        const char* e = std::getenv("B200_GEMM_TMA_STORE");      // 0 keeps the per-thread stores, for measurements
        return !(e && e[0] == '0');
    }();
    args.tma_store = 0;
    if (tma_store_allowed && out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (static_cast<size_t>(n_out) * elem) % 16 == 0 &&
        make_out_map(&tma_out, out, plan.M, n_out, elem)) {
        args.tma_store = 1;
        const int fit = (kMaxSmem - 1024 - 256 - kOutStageTotal) / stage_bytes;
        if (args.stages > fit) args.stages = fit;
        if (args.stages < 2) return cudaErrorInvalidValue;
    }
    const int smem = args.stages * stage_bytes + 1024 + 8 * (2 * args.stages + 5) + 16 + (args.tma_store ? kOutStageTotal : 0);
    static int configured[64] = {};
    if (cudaError_t e = ensure_dynamic_smem(gemm_tc5_persist_kernel<BN, kInt8, kPair>, smem, configured)) return e;
    return launch_ex(gemm_tc5_persist_kernel<BN, kInt8, kPair>, dim3(plan.grid), dim3(kPersistThreads), smem, stream, kPair ? 2 : 1,
                     true, plan.tma_a, plan.tma_b, tma_out, args);
}

}  // namespace

bool gemm_make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    return make_operand_map(map, base, rows, cols, box_rows);
}

bool gemm_plan_can_rope(const GemmPlan& plan, int hq, int hkv) {
    return !plan.persist && plan.cluster && plan.bn == 128 && !plan.gate && plan.splits >= 2 &&
           plan.splits <= 16 && (128 / plan.splits) % 8 == 0 && plan.N == (hq + 2 * hkv) * 128;
}

void gemm_plan_make_persistent(GemmPlan* plan, int sm_count, bool fused_epilogue) {
    if (sm_count <= 0) return;
    const int bn = plan->bn;
    if (bn != 128 && bn != 256) return;
    const int out_cols = plan->gate ? bn / 2 : bn;
    const int n_out = plan->gate ? plan->N / 2 : plan->N;
    const long long tiles = static_cast<long long>((plan->M + kBM - 1) / kBM) * ((n_out + out_cols - 1) / out_cols);
    // The fused epilogues are what the one-tile kernel is slow at (four epilogue warps, nothing to overlap them
    // with), so they switch at half a wave of tiles; raw accumulator output switches at two waves.
    const long long min_tiles = fused_epilogue ? (sm_count + 1) / 2 : 2LL * sm_count;
    if (tiles > 0x3FFFFFFF || tiles < min_tiles) return;
    // CTA pairs for 256-wide tiles of problems with at least two tile rows: each CTA moves a third less through its
    // shared memory per MMA (B200_GEMM_PAIR=0 in the environment keeps the one-CTA form, for measurements)
    static const bool pair_allowed = [] {
        const char* e = std::getenv("B200_GEMM_PAIR");
        return !(e && e[0] == '0');
    }();
    // (with at most one 128 x 256 tile per SM the one-CTA form has as many rounds and more streams in flight: measured)
    const bool pair = pair_allowed && bn == 256 && plan->M > kBM && sm_count >= 2 && tiles > sm_count;
    // (256 x 128 tiles on pairs were tried for grids whose last round is half empty, 4096^3 = 3.46 rounds of 256 x 256
    // tiles: 1944 TOPS against 2565, the narrower MMA does not keep the tensor pipe fed.)
    const int stage_bytes = kABytes + (pair ? bn / 2 : bn) * kBK;
    int stages = (kMaxSmem - 1024 - 256) / stage_bytes;
    if (stages > 8) stages = 8;
    if (pair) {
        // B is fetched in boxes of bn / 2 rows (the gated layout already is)
        if (!plan->gate && plan->b_ptr != nullptr && !make_operand_map(&plan->tma_b, plan->b_ptr, plan->N, plan->K, bn / 2)) return;
        const long long pair_tiles = static_cast<long long>((plan->M + 2 * kBM - 1) / (2 * kBM)) * ((n_out + out_cols - 1) / out_cols);
        const long long pairs = pair_tiles < sm_count / 2 ? pair_tiles : sm_count / 2;
        plan->grid = static_cast<int>(2 * pairs);
    } else {
        plan->grid = tiles < sm_count ? static_cast<int>(tiles) : sm_count;
    }
    plan->pair = pair ? 1 : 0;
    plan->persist = 1;
    plan->stages = stages;
    plan->splits = 1;
    plan->cluster = 0;
    plan->out_planes = 1;
}

cudaError_t gemm_make_plan(GemmPlan* plan, int kind, const void* a, const void* b, int M, int N, int K, int gate,
                           int want_splits, int want_bn, const char** why, bool encode_maps) {
    static const char* kNone = "";
    if (why) *why = kNone;
    auto fail = [&](const char* msg) {
        if (why) *why = msg;
        return cudaErrorInvalidValue;
    };
    if (M <= 0 || N <= 0 || K <= 0) return fail("gemm: m, n, k must be positive");
    if (K % 16 != 0) return fail("gemm: k must be a multiple of 16 (TMA row stride)");
    if (N % 16 != 0) return fail("gemm: n must be a multiple of 16");
    if (gate && (N % 32 != 0)) return fail("gemm: gated n must be a multiple of 32");
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
        return fail("gemm: operand base addresses must be 16-byte aligned");
    plan->kind = kind;
    plan->M = M; plan->N = N; plan->K = K; plan->gate = gate;
    plan->b_ptr = encode_maps ? b : nullptr;
    const int m_tiles = (M + kBM - 1) / kBM;
    const int kb_total = (K + kBK - 1) / kBK;
    int bn = want_bn;
    if (bn <= 0) {
        bn = (M >= 512) ? 256 : 128;
        const int sms = current_sm_count();
        const int tiles128 = (N + 127) / 128;
        if (m_tiles == 1 && !gate) {
            // One row of tiles (decode shapes): what counts is how evenly the weight stream spreads over the SMs.
            // 224-wide tiles when they turn a grid of more than one CTA per SM into a single even wave ...
            if (tiles128 > sms && N % 224 == 0 && N / 224 <= sms) bn = 224;
            // ... and 64-wide tiles for narrow outputs, so that K is cut into fewer, longer slices per tile
            else if (tiles128 >= 16 && 4 * tiles128 <= sms && N % 64 == 0) bn = 64;
        }
    }
    if (bn != 64 && bn != 128 && bn != 224 && bn != 256) return fail("gemm: tile width must be 64, 128, 224 or 256");
    if (gate && bn == 224) return fail("gemm: the gated layout takes tile widths 64, 128 or 256");
    const int n_out = gate ? N / 2 : N;
    const int out_cols = gate ? bn / 2 : bn;
    const int tiles = m_tiles * ((n_out + out_cols - 1) / out_cols);
    // A power-of-two split count up to 8 whose slices tile K exactly can be reduced inside a cluster.
    auto exact_pow2 = [&](int s) {
        if (s < 2 || s > 8 || (s & (s - 1)) != 0) return false;
        const int per = (kb_total + s - 1) / s;
        return (kb_total + per - 1) / per == s;
    };
    int splits = want_splits;
    if (splits <= 0) {
        splits = 1;
        const int sms = current_sm_count();
        if (2 * tiles <= sms) {      // splitting pays only when it at least doubles the number of busy SMs
            int cap = 2 * sms / tiles;
            if (cap > kb_total / 2) cap = kb_total / 2;
            if (cap > 8) cap = 8;
            for (int s = 2; s <= cap; s *= 2)
                if (exact_pow2(s)) splits = s;
        }
    }
    if (splits > kb_total) splits = kb_total;
    {   // every split must own at least one K block
        const int per = (kb_total + splits - 1) / splits;
        splits = (kb_total + per - 1) / per;
    }
    plan->bn = bn;
    plan->splits = splits;
    const int stage_bytes = kABytes + bn * kBK;
    // Small grids keep two CTAs per SM resident (about 100 KB each); big ones take the whole SM.
    int stages = (m_tiles * 1 >= 4 || bn >= 224) ? (200 * 1024) / stage_bytes : (100 * 1024) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    plan->stages = stages;
    // the parked partial tile (bn x 128 accumulators) reuses the operand ring
    plan->cluster = (!gate && exact_pow2(splits) && stages * stage_bytes >= (bn + 4) * kBM * 4) ? 1 : 0;
    plan->out_planes = plan->cluster ? 1 : splits;
    if (!encode_maps) return cudaSuccess;      // shape decisions only (plan queries)
    if (!make_operand_map(&plan->tma_a, a, M, K, kBM)) return fail("gemm: cuTensorMapEncodeTiled failed for A");
    if (!make_operand_map(&plan->tma_b, b, N, K, gate ? bn / 2 : bn)) return fail("gemm: cuTensorMapEncodeTiled failed for B");
    return cudaSuccess;
}

cudaError_t gemm_launch(const GemmPlan& plan, const GemmEpilogue& ep, uint32_t* err, cudaStream_t stream) {
    if (plan.persist) {
        if (!ep.fused && plan.gate) return cudaErrorInvalidValue;   // raw output always uses the plain column layout
        if (ep.rope.enabled) return cudaErrorInvalidValue;
        PersistArgs pa;
        pa.M = plan.M; pa.N = plan.N; pa.K = plan.K;
        pa.stages = plan.stages;
        pa.kb_total = (plan.K + kBK - 1) / kBK;
        const int out_cols = plan.gate ? plan.bn / 2 : plan.bn;
        const int n_out = plan.gate ? plan.N / 2 : plan.N;
        pa.tiles_m = plan.pair ? (plan.M + 2 * kBM - 1) / (2 * kBM) : (plan.M + kBM - 1) / kBM;
        pa.tiles_n = (n_out + out_cols - 1) / out_cols;
        pa.group_m = plan.pair ? 8 : 16;
        pa.gate = plan.gate;
        pa.n_half = plan.N / 2;
        pa.vec16 = ((reinterpret_cast<uintptr_t>(ep.b_scale) | reinterpret_cast<uintptr_t>(ep.bias)) & 15) == 0 ? 1 : 0;
        pa.ep = ep;
        pa.err = err;
        if (ep.push.peers != nullptr) return cudaErrorInvalidValue;    // the scatter exists in the one-tile kernel only
        const bool i8p = plan.kind == kGemmI8;
        if (plan.pair) {
            if (plan.bn != 256 || ep.wait.flags != nullptr) return cudaErrorInvalidValue;
            return i8p ? launch_persist_t<256, true, true>(plan, pa, stream) : launch_persist_t<256, false, true>(plan, pa, stream);
        }
        if (plan.bn == 128) return i8p ? launch_persist_t<128, true, false>(plan, pa, stream) : launch_persist_t<128, false, false>(plan, pa, stream);
        return i8p ? launch_persist_t<256, true, false>(plan, pa, stream) : launch_persist_t<256, false, false>(plan, pa, stream);
    }
    KernelArgs args;
    args.M = plan.M; args.N = plan.N; args.K = plan.K;
    args.stages = plan.stages;
    args.kb_total = (plan.K + kBK - 1) / kBK;
    args.kb_per_split = (args.kb_total + plan.splits - 1) / plan.splits;
    args.gate = plan.gate;
    args.n_half = plan.N / 2;
    args.ep = ep;
    args.err = err;
    args.cluster_reduce = plan.cluster;
    if (ep.fused && plan.splits != 1 && !plan.cluster) return cudaErrorInvalidValue;
    if (ep.rope.enabled && !gemm_plan_can_rope(plan, ep.rope.hq, ep.rope.hkv)) return cudaErrorInvalidValue;
    if (!ep.fused && plan.gate) return cudaErrorInvalidValue;   // raw planes always use the plain column layout
    if (ep.push.peers != nullptr &&
        (!ep.fused || plan.gate || ep.rope.enabled || ep.residual != nullptr || ep.out_bf16 || ep.push.rows <= 0 ||
         ep.push.tp <= 0 || ep.push.tp > 32 || ep.push.arrived == nullptr || plan.M != ep.push.tp * ep.push.rows))
        return cudaErrorInvalidValue;
    const bool i8 = plan.kind == kGemmI8;
    switch (plan.bn) {
        case 64: return i8 ? launch_t<64, true>(plan, args, stream) : launch_t<64, false>(plan, args, stream);
        case 128: return i8 ? launch_t<128, true>(plan, args, stream) : launch_t<128, false>(plan, args, stream);
        case 224: return i8 ? launch_t<224, true>(plan, args, stream) : launch_t<224, false>(plan, args, stream);
        case 256: return i8 ? launch_t<256, true>(plan, args, stream) : launch_t<256, false>(plan, args, stream);
        default: return cudaErrorInvalidValue;
    }
}

int gemm_plan_tiles(const GemmPlan& plan) {
    const int n_out = plan.gate ? plan.N / 2 : plan.N;
    const int out_cols = plan.gate ? plan.bn / 2 : plan.bn;
    return ((n_out + out_cols - 1) / out_cols) * ((plan.M + kBM - 1) / kBM);
}

cudaError_t gemm_splitk_epilogue(int kind, int splits, int M, int N, int gate, const void* raw,
                                 const GemmEpilogue& ep, cudaStream_t stream) {
    const int n_out = gate ? N / 2 : N;
    int64_t groups = static_cast<int64_t>(M) * (n_out / 4);
    int64_t grid = (groups + 255) / 256;
    if (grid > int64_t(current_sm_count()) * 8) grid = int64_t(current_sm_count()) * 8;
    if (grid < 1) grid = 1;
    if (kind == kGemmI8)
        splitk_epilogue_kernel<true><<<static_cast<int>(grid), 256, 0, stream>>>(
            static_cast<const uint32_t*>(raw), splits, M, N, gate, ep);
    else
        splitk_epilogue_kernel<false><<<static_cast<int>(grid), 256, 0, stream>>>(
            static_cast<const uint32_t*>(raw), splits, M, N, gate, ep);
    return cudaGetLastError();
}

cudaError_t gemm_sum_planes_i32(const int* raw, int splits, int64_t elems, int* out, cudaStream_t stream) {
    int64_t grid = (elems + 255) / 256;
    if (grid > int64_t(current_sm_count()) * 8) grid = int64_t(current_sm_count()) * 8;
    if (grid < 1) grid = 1;
    sum_planes_i32_kernel<<<static_cast<int>(grid), 256, 0, stream>>>(raw, splits, elems, out);
    return cudaGetLastError();
}

}  // namespace b200
