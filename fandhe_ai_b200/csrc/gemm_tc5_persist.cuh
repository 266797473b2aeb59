// Persistent form of the tcgen05 GEMM for problems with at least a few waves of tiles.  Included by gemm_tc5.cu
// inside its anonymous namespace (it uses kBM, kBK, kUmmaK, kABytes, acc_to_f32 and store_out4).
//
// One CTA per SM stays resident and takes the 128 x BN output tiles round-robin (tile = cta + i * grid), numbered
// in bands of `group_m` tile rows so that the CTAs of one wave work on neighbouring tiles and share operand tiles
// through L2.  Warp 0 is the TMA producer, warp 1 issues the MMAs, warps 2..9 are the epilogue.  There are two
// accumulator buffers in TMEM: the MMA warp fills one while the epilogue drains the other, so the operand ring
// never waits for an epilogue.  With K = 4096 a tile's main loop is only about 16k cycles, which the epilogue has
// to beat: it runs on eight warps (two per TMEM lane quarter, half of the columns each), loads the per-column
// scales and bias with 16-byte loads once per 32 columns, and converts / stores 16 bytes at a time.
//
// Pair form (kPair): two CTAs of a cluster share one 256 x BN accumulator tile through tcgen05.mma.cta_group::2.  CTA
// rank r holds the A rows [256 t + 128 r, + 128) and HALF of the B rows (BN / 2), and finds the accumulator rows of its
// A rows in its own tensor memory; the even CTA issues the MMAs for both, reading both CTAs' shared memory.  Per MMA
// volume a CTA then moves 16 KB + 16 KB per K block through its shared memory instead of 16 KB + 32 KB: the operand
// feed from L2, which limits the 128 x 256 form, drops by a third.  Every CTA fetches its own operand halves (no
// multicast loads); what crosses the pair are barrier arrivals: both CTAs' loads count on the leader's full barriers,
// the leader's commits arrive on both CTAs' empty / accumulator-full barriers, and both CTAs' epilogue threads arrive on
// the leader's accumulator-empty barriers.
//
// Output (tma_store): every epilogue warp stages 32 rows x 32 columns of finished values (32 f32 / raw accumulators per row; 32 bf16 = 64 bytes) in
// its own 4 KB of shared memory, in the swizzle pattern of the tensor map (128-byte rows: 16-byte piece t of row r at
// piece t ^ (r & 7), so that the 32 lanes, one row each, write without bank conflicts), and one lane sends the box with
// a TMA store, which also drops what lies beyond M or N.  The warp waits for the store to have read the buffer only
// when it comes back to fill it again.  Output planes whose base or row pitch is not a multiple of 16 bytes keep the
// per-thread 16-byte stores.
//
// The arithmetic per element is that of the one-tile kernel: y = act(fma(float(acc), sa * sb, bias)) (+ residual),
// except that SiLU uses the fast exponential and reciprocal.

constexpr int kPersistThreads = 320;      // 2 + 8 warps
constexpr int kEpilogueThreads = 256;

struct PersistArgs {
    int M, N, K;
    int stages;
    int kb_total;          // K blocks per tile
    int tiles_m, tiles_n;  // tile grid (columns counted in output columns per CTA)
    int group_m;           // tiles are numbered in bands of group_m tile rows, row-fastest inside a band
    int gate;              // B tile = BN/2 gate rows + BN/2 up rows
    int n_half;            // N / 2 in the gate form
    int vec16;             // the scale and bias vectors start on 16-byte boundaries (16-byte loads allowed)
    int tma_store;         // the output goes through shared memory and TMA stores (tma_out is valid)
    GemmEpilogue ep;
    uint32_t* err;
};

__device__ __forceinline__ void tile_origin(const PersistArgs& p, int tile, int& m_idx, int& n_idx) {
    const int band_tiles = p.group_m * p.tiles_n;
    const int band = tile / band_tiles;
    const int r = tile % band_tiles;
    int gm = p.tiles_m - band * p.group_m;
    if (gm > p.group_m) gm = p.group_m;
    m_idx = band * p.group_m + r % gm;
    n_idx = r / gm;
}

// two f32 -> packed bf16 pair (round to nearest even), first value in the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// x * sigmoid(x) with the fast exponential and reciprocal (relative error about 1e-6)
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// 32 consecutive f32 values starting at a 16-byte aligned address (the same address in every lane: one transaction)
__device__ __forceinline__ void load32(const float* __restrict__ src, float (&v)[32]) {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(src) + t);
        v[4 * t] = x.x; v[4 * t + 1] = x.y; v[4 * t + 2] = x.z; v[4 * t + 3] = x.w;
    }
}

// Writes 32 finished values of one row: f32 or bf16, with the optional residual added first.
__device__ __forceinline__ void store32(const GemmEpilogue& ep, size_t idx, float (&y)[32]) {
    if (ep.residual) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const float4 r = *reinterpret_cast<const float4*>(ep.residual + idx + 4 * t);
            y[4 * t] += r.x; y[4 * t + 1] += r.y; y[4 * t + 2] += r.z; y[4 * t + 3] += r.w;
        }
    }
    if (ep.out_bf16) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(ep.out) + idx);
#pragma unroll
        for (int t = 0; t < 4; ++t)
            dst[t] = make_uint4(pack_bf16x2(y[8 * t], y[8 * t + 1]), pack_bf16x2(y[8 * t + 2], y[8 * t + 3]),
                                pack_bf16x2(y[8 * t + 4], y[8 * t + 5]), pack_bf16x2(y[8 * t + 6], y[8 * t + 7]));
    } else {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(ep.out) + idx);
#pragma unroll
        for (int t = 0; t < 8; ++t) dst[t] = make_float4(y[4 * t], y[4 * t + 1], y[4 * t + 2], y[4 * t + 3]);
    }
}

constexpr int kOutStageBytes = 4096;        // per epilogue warp: 32 rows x 128 bytes
constexpr int kOutStageTotal = (kEpilogueThreads / 32) * kOutStageBytes;

// Staging of one warp's finished values for TMA stores (see the file comment): 32 columns of the warp's 32 rows per
// store.  `rows` = rows of the output (a warp whose rows all lie beyond it sends nothing).
struct OutStage {
    const CUtensorMap* map;
    uint32_t buf;        // shared address of the warp's buffer (1024-byte aligned)
    int lane;
    int rows;

    __device__ __forceinline__ void begin() {
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
    }
    __device__ __forceinline__ void st4(uint32_t dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
    }
    __device__ __forceinline__ void send(int x, int y) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && y < rows) {
            tma_store_2d(map, buf, x, y);
            bulk_commit_group();
        }
    }
    // 32 words (f32 values or raw accumulators) of columns n .. n + 31: 128-byte rows, 128-byte swizzle
    __device__ __forceinline__ void put_words(const uint32_t (&w)[32], int n, int row0) {
        begin();
#pragma unroll
        for (int t = 0; t < 8; ++t)
            st4(buf + static_cast<uint32_t>(lane * 128 + ((t ^ (lane & 7)) << 4)), w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
        send(n, row0);
    }
    __device__ __forceinline__ void put_f32(const float (&y)[32], int n, int row0) {
        begin();
#pragma unroll
        for (int t = 0; t < 8; ++t)
            st4(buf + static_cast<uint32_t>(lane * 128 + ((t ^ (lane & 7)) << 4)), __float_as_uint(y[4 * t]),
                __float_as_uint(y[4 * t + 1]), __float_as_uint(y[4 * t + 2]), __float_as_uint(y[4 * t + 3]));
        send(n, row0);
    }
    // 32 bf16 values per row: 64-byte rows, 64-byte swizzle (piece t of row r at piece t ^ ((r >> 1) & 3))
    __device__ __forceinline__ void put_bf16(const float (&y)[32], int n, int row0) {
        begin();
#pragma unroll
        for (int t = 0; t < 4; ++t)
            st4(buf + static_cast<uint32_t>(lane * 64 + ((t ^ ((lane >> 1) & 3)) << 4)), pack_bf16x2(y[8 * t], y[8 * t + 1]),
                pack_bf16x2(y[8 * t + 2], y[8 * t + 3]), pack_bf16x2(y[8 * t + 4], y[8 * t + 5]), pack_bf16x2(y[8 * t + 6], y[8 * t + 7]));
        send(n, row0);
    }
};

// Adds the residual row segment to 32 finished values (columns n .. n + 31 of row `row`; the segment is whole).
__device__ __forceinline__ void add_residual32(const GemmEpilogue& ep, size_t idx, float (&y)[32]) {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const float4 r = *reinterpret_cast<const float4*>(ep.residual + idx + 4 * t);
        y[4 * t] += r.x; y[4 * t + 1] += r.y; y[4 * t + 2] += r.z; y[4 * t + 3] += r.w;
    }
}

template <int BN, bool kInt8, bool kPair>
__global__ void __launch_bounds__(kPersistThreads, 1)
gemm_tc5_persist_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const __grid_constant__ CUtensorMap tma_out, PersistArgs p) {
    constexpr int kBRows = kPair ? BN / 2 : BN;      // B rows this CTA brings in per stage
    constexpr int kBBytes = kBRows * kBK;
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr int kTileRows = kPair ? 2 * kBM : kBM; // accumulator rows per tile (pair: over both CTAs)
    constexpr uint32_t kTmemCols = 2 * BN;      // two accumulator buffers
    constexpr uint32_t kIdesc = kInt8 ? umma_idesc(1, 2, kTileRows, BN) : umma_idesc(0, 1, kTileRows, BN);

    extern __shared__ uint8_t smem_dyn[];
    // [output staging of the epilogue warps (tma_store)] [operand ring] [barriers]
    const uint32_t out_stage_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t smem_base = out_stage_base + (p.tma_store ? static_cast<uint32_t>(kOutStageTotal) : 0u);
    const uint32_t bar_base = smem_base + p.stages * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (p.stages + s); };
    auto tmem_full = [&](int b) { return bar_base + 8u * (2 * p.stages + b); };
    auto tmem_empty = [&](int b) { return bar_base + 8u * (2 * p.stages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * p.stages + 4);
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_dyn + (tmem_slot - smem_u32(smem_dyn)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;          // 0: the CTA that issues the MMAs
    const int grid = static_cast<int>(gridDim.x) / (kPair ? 2 : 1);    // tiles in flight: CTAs, or CTA pairs
    const int cta = static_cast<int>(blockIdx.x) / (kPair ? 2 : 1);
    const int tiles = p.tiles_m * p.tiles_n;

    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        if (p.tma_store) tma_prefetch_desc(&tma_out);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full(b), 1);
            mbar_init(tmem_empty(b), kEpilogueThreads * (kPair ? 2 : 1));
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (kPair) {
            tmem_alloc_pair(tmem_slot, kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, kTmemCols);
            tmem_relinquish();
        }
    }
    tc5_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();      // the peer's barriers exist before anything arrives on them
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const int out_cols = p.gate ? BN / 2 : BN;

    if (warp == 0) {
        const bool leader = elect_one();
        bool b_in_flight = false;
        if (!kPair && p.ep.wait.flags != nullptr && cta < tiles) {
            // The A operand comes from other GPUs: weight tiles of the first ring pass first, then the lanes wait for
            // the peers' flags (one flag per lane), then the A tiles (see GemmPeerWait).
            if (leader) {
                int m_idx, n_idx;
                tile_origin(p, cta, m_idx, n_idx);
                const int n0 = n_idx * out_cols;
                const int pre = p.kb_total < p.stages ? p.kb_total : p.stages;
                for (int k = 0; k < pre; ++k) {
                    mbar_arrive_expect_tx(full_bar(k), kStageBytes);
                    const uint32_t b_dst = smem_base + k * kStageBytes + kABytes;
                    tma_load_2d(b_dst, &tma_b, full_bar(k), k * kBK, n0);
                    if (p.gate) tma_load_2d(b_dst + (BN / 2) * kBK, &tma_b, full_bar(k), k * kBK, p.n_half + n0);
                }
            }
            __syncwarp();
            pdl_wait();
            if (lane < p.ep.wait.n) wait_peer_flag(p.ep.wait.flags + lane, *p.ep.wait.epoch, p.err, p.ep.wait.timeout_ns);
            __syncwarp();
            b_in_flight = true;
        }
        if (leader) {
            if (b_in_flight) fence_proxy_async_all();
            int i = 0;                 // K blocks issued so far: ring position and phase
            bool waited = false;       // griddepcontrol.wait done
            bool ok = true;
            for (int tile = cta; ok && tile < tiles; tile += grid) {
                int m_idx, n_idx;
                tile_origin(p, tile, m_idx, n_idx);
                const int m0 = m_idx * kTileRows + static_cast<int>(rank) * kBM, n0 = n_idx * out_cols;
                if constexpr (kPair) {
                    // this CTA's operand halves; their bytes count on the leader's full barrier, which expects both CTAs'
                    if (!waited) {
                        pdl_wait();
                        pdl_launch_dependents();
                        waited = true;
                    }
                    const int nb0 = p.gate ? (rank == 0 ? n0 : p.n_half + n0) : n0 + static_cast<int>(rank) * (BN / 2);
                    for (int kb = 0; kb < p.kb_total; ++kb, ++i) {
                        const int s = i % p.stages;
                        const uint32_t ph = (i / p.stages) & 1;
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, p.err, kErrProducerWait)) { ok = false; break; }
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * kStageBytes);
                        const uint32_t bar = mapa_shared(full_bar(s), 0);
                        tma_load_2d_pair(smem_base + s * kStageBytes, &tma_a, bar, kb * kBK, m0);
                        tma_load_2d_pair(smem_base + s * kStageBytes + kABytes, &tma_b, bar, kb * kBK, nb0);
                    }
                    continue;
                }
                auto load_b = [&](int kb, int s) {
                    const uint32_t b_dst = smem_base + s * kStageBytes + kABytes;
                    tma_load_2d(b_dst, &tma_b, full_bar(s), kb * kBK, n0);
                    if (p.gate) tma_load_2d(b_dst + (BN / 2) * kBK, &tma_b, full_bar(s), kb * kBK, p.n_half + n0);
                };
                auto load_a = [&](int kb, int s) { tma_load_2d(smem_base + s * kStageBytes, &tma_a, full_bar(s), kb * kBK, m0); };
                int kb = 0;
                if (!waited) {
                    // The B operand (weights) does not depend on the kernel before this one: fill the ring with B
                    // tiles while that kernel drains, then wait for it and add the A tiles.
                    const int pre = p.kb_total < p.stages ? p.kb_total : p.stages;
                    if (!b_in_flight) {
                        for (int k = 0; k < pre; ++k) {
                            mbar_arrive_expect_tx(full_bar(k), kStageBytes);
                            load_b(k, k);
                        }
                        pdl_wait();
                    }
                    pdl_launch_dependents();
                    waited = true;
                    for (int k = 0; k < pre; ++k) load_a(k, k);
                    kb = pre;
                    i = pre;
                }
                for (; kb < p.kb_total; ++kb, ++i) {
                    const int s = i % p.stages;
                    const uint32_t ph = (i / p.stages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, p.err, kErrProducerWait)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(s), kStageBytes);
                    load_a(kb, s);
                    load_b(kb, s);
                }
            }
            if (!waited) {
                pdl_wait();
                pdl_launch_dependents();
            }
        }
    } else if (warp == 1) {
        if (elect_one() && rank == 0) {
            int i = 0, j = 0;
            bool ok = true;
            for (int tile = cta; ok && tile < tiles; tile += grid, ++j) {
                const int buf = j & 1;
                ok = mbar_wait(tmem_empty(buf), ((j >> 1) & 1) ^ 1u, p.err, kErrMmaWait);
                if (!ok) break;
                tc5_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
                for (int kb = 0; kb < p.kb_total; ++kb, ++i) {
                    const int s = i % p.stages;
                    const uint32_t ph = (i / p.stages) & 1;
                    ok = mbar_wait(full_bar(s), ph, p.err, kErrMmaWait);
                    if (!ok) break;
                    tc5_fence_after();
                    const uint32_t a_src = smem_base + s * kStageBytes;
                    const uint64_t adesc = umma_desc_k128(a_src);
                    const uint64_t bdesc = umma_desc_k128(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        if constexpr (kPair) umma_ss_pair<kInt8>(d_tmem, adesc + 2u * k, bdesc + 2u * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
                        else umma_ss<kInt8>(d_tmem, adesc + 2u * k, bdesc + 2u * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    if constexpr (kPair) tc5_commit_pair(empty_bar(s), 3);      // the stage is free in both CTAs
                    else tc5_commit(empty_bar(s));
                }
                if (!ok) break;
                if constexpr (kPair) tc5_commit_pair(tmem_full(buf), 3);       // each CTA drains its own accumulator rows
                else tc5_commit(tmem_full(buf));
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9; TMEM lane quarter = warp % 4, column half = (warp - 2) / 4
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int rl = q * 32 + lane;                 // row inside the tile
        const GemmEpilogue& ep = p.ep;
        OutStage st{&tma_out, out_stage_base + static_cast<uint32_t>((warp - 2) * kOutStageBytes), lane, p.M};
        const bool staged = p.tma_store != 0;
        pdl_wait();      // scales, bias, residual and the output buffers belong to the surrounding kernels
        bool ok = true;
        int j = 0;
        for (int tile = cta; tile < tiles; tile += grid, ++j) {
            const int buf = j & 1;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(tmem_full(buf), (j >> 1) & 1, p.err, kErrEpilogueWait)) != 0;
            tc5_fence_after();
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(buf * BN) + (static_cast<uint32_t>(q * 32) << 16);
            int m_idx, n_idx;
            tile_origin(p, tile, m_idx, n_idx);
            const int m0 = m_idx * kTileRows + static_cast<int>(rank) * kBM, n0 = n_idx * out_cols;
            const int row = m0 + rl;
            const int row0 = m0 + q * 32;                 // first row of this warp
            const bool row_ok = row < p.M;
            const size_t row_c = static_cast<size_t>(row_ok ? row : 0);
            if (ok && !ep.fused) {
                uint32_t* raw = static_cast<uint32_t*>(ep.raw) + row_c * p.N;
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32) {
                    if (n0 + c0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
                    if (staged) st.put_words(v, n0 + c0, row0);
                    else if (row_ok) {
#pragma unroll
                        for (int t = 0; t < 32; t += 4) {
                            const int n = n0 + c0 + t;
                            if (n < p.N) *reinterpret_cast<uint4*>(raw + n) = make_uint4(v[t], v[t + 1], v[t + 2], v[t + 3]);
                        }
                    }
                }
            } else if (ok && !p.gate) {
                const float sa = ep.a_scale[ep.a_per_row ? row_c : 0];
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32) {
                    const int n = n0 + c0;
                    if (n >= p.N) break;
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    float y[32];
                    const bool whole = n + 32 <= p.N;       // N is a multiple of 16: a chunk is whole or half
                    const bool vec = whole && p.vec16;
                    if (ep.b_per_col) {
                        if (vec) load32(ep.b_scale + n, y);
                        else {
#pragma unroll
                            for (int t = 0; t < 32; ++t) y[t] = n + t < p.N ? ep.b_scale[n + t] : 0.0f;
                        }
                    } else {
                        const float sb = ep.b_scale[0];
#pragma unroll
                        for (int t = 0; t < 32; ++t) y[t] = sb;
                    }
                    float bias[32];
                    if (ep.bias) {
                        if (vec) load32(ep.bias + n, bias);
                        else {
#pragma unroll
                            for (int t = 0; t < 32; ++t) bias[t] = n + t < p.N ? ep.bias[n + t] : 0.0f;
                        }
                    } else {
#pragma unroll
                        for (int t = 0; t < 32; ++t) bias[t] = 0.0f;
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        float x = fmaf(acc_to_f32<kInt8>(v[t]), sa * y[t], bias[t]);
                        if (ep.act == kActSilu) x = silu_fast(x);
                        else if (ep.act == kActRelu) x = fmaxf(x, 0.0f);
                        y[t] = x;
                    }
                    if (staged) {
                        if (ep.residual && row_ok) {
                            if (whole) add_residual32(ep, row_c * p.N + n, y);
                            else {
#pragma unroll
                                for (int t = 0; t < 16; ++t) y[t] += ep.residual[row_c * p.N + n + t];
                            }
                        }
                        if (ep.out_bf16) st.put_bf16(y, n, row0);
                        else st.put_f32(y, n, row0);
                    } else if (row_ok) {
                        if (whole) store32(ep, row_c * p.N + n, y);
                        else {
#pragma unroll
                            for (int t = 0; t < 16; t += 4) store_out4(ep, row_c * p.N + n + t, y[t], y[t + 1], y[t + 2], y[t + 3]);
                        }
                    }
                }
            } else if (ok) {
                // gate form: accumulator columns [0, BN/2) hold gate, [BN/2, BN) hold up, outputs n0 .. n0 + BN/2;
                // this warp's half of them
                const float sa = ep.a_scale[ep.a_per_row ? row_c : 0];
                constexpr int kHalf = BN / 2;
                for (int c0 = half * (kHalf / 2); c0 < (half + 1) * (kHalf / 2); c0 += 32) {
                    const int n = n0 + c0;
                    if (n >= p.n_half) break;
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_row + c0, g);
                    tmem_ld_32x32(t_row + kHalf + c0, u);
                    float y[32], su[32];
                    const bool whole = n + 32 <= p.n_half;
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const bool in = whole || n + t < p.n_half;
                        y[t] = in ? ep.b_scale[ep.b_per_col ? n + t : 0] : 0.0f;
                        su[t] = in ? ep.b_scale[ep.b_per_col ? p.n_half + n + t : 0] : 0.0f;
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const bool in = whole || n + t < p.n_half;
                        const float bg = (ep.bias && in) ? ep.bias[n + t] : 0.0f;
                        const float bu = (ep.bias && in) ? ep.bias[p.n_half + n + t] : 0.0f;
                        const float gv = fmaf(acc_to_f32<kInt8>(g[t]), sa * y[t], bg);
                        const float uv = fmaf(acc_to_f32<kInt8>(u[t]), sa * su[t], bu);
                        y[t] = silu_fast(gv) * uv;
                    }
                    if (staged) {
                        if (ep.residual && row_ok) {
                            if (whole) add_residual32(ep, row_c * p.n_half + n, y);
                            else {
#pragma unroll
                                for (int t = 0; t < 16; ++t) y[t] += ep.residual[row_c * p.n_half + n + t];
                            }
                        }
                        if (ep.out_bf16) st.put_bf16(y, n, row0);
                        else st.put_f32(y, n, row0);
                    } else if (row_ok) {
                        if (whole) store32(ep, row_c * p.n_half + n, y);
                        else {
#pragma unroll
                            for (int t = 0; t < 16; t += 4) store_out4(ep, row_c * p.n_half + n + t, y[t], y[t + 1], y[t + 2], y[t + 3]);
                        }
                    }
                }
            }
            // hand the accumulator buffer back to the MMA warp (of the leader CTA)
            tc5_fence_before();
            if (kPair && rank != 0) mbar_arrive_cluster(mapa_shared(tmem_empty(buf), 0));
            else mbar_arrive(tmem_empty(buf));
        }
        if (staged && lane == 0) bulk_wait_all();      // the staging buffers stay valid until the last store has read them
    }

    tc5_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();      // neither CTA frees tensor or shared memory the other may still use
    if (warp == 1) {
        __syncwarp();
        tc5_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
}
