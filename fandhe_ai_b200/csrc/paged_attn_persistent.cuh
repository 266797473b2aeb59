// Split-K decode attention: persistent CTAs, tensor-core contractions.  Included by paged_kv.cu inside its
// anonymous namespace (it uses kD, kBS, kTileBytes, kStages, kStagesPerWarp, kConsumerWarps, kFastThreads).
//
// Work item = one (query row, kv-head slot, chunk of `chunk_blocks` KV blocks); G = 1, 2 or 4 query heads share
// the kv head.  A fixed number of CTAs per SM stays resident and pulls items from a global counter.  In each
// CTA a producer warp runs ahead of four consumer warps: it takes the next item, publishes its descriptor,
// copies the item's query rows into shared memory with a bulk copy, and streams the item's K and V tiles
// through the block table - per block two TMA boxes of [16 tokens x 64 dims] for K, then two for V (128-byte
// rows, 128-byte swizzle, so ldmatrix reads them without bank conflicts) - while the consumers are still
// finishing the previous item, so the load pipeline never drains between items.
//
// Stage ownership: consumer warp w owns stages [w * kStagesPerWarp, (w + 1) * kStagesPerWarp) and blocks
// w, w + 4, ... of every item; it counts its tiles across items, so consecutive uses of a stage are waited
// for by the same warp in order and a parity wait is never two phases ahead of its barrier (such a wait
// would pass at once on a stage whose data has not landed).
//
// Both contractions run on mma.sync.m16n8k16 (bf16 x bf16 -> f32) with the f32 operand split into three
// bf16 terms that sum to it exactly (hi + mid + lo), one term per group of four rows of the 16-row A
// operand: row 4 * term + head.  The products with the bf16 K / V values are therefore exact and only the
// f32 accumulation order differs from a scalar f32 loop.
//   scores:  A = split(q * scale) [16 x 128],  B = K tile^T  -> C[row][token];  s = C[h] + C[4 + h] + C[8 + h]
//   output:  A = split(p)         [16 x 16],   B = V tile    -> D[row][dim];    o = D[h] + D[4 + h] + D[8 + h]
// The folded score of a thread lands exactly where the A operand of the second product wants it, so the
// softmax weights never leave registers; every warp keeps a running (max, sum, accumulator) and the four
// warps are merged per item.

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// untiled bulk copy global -> shared, completion counted in bytes on an mbarrier (16-byte aligned, size % 16 == 0)
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}

// x = hi + mid + lo with every term a bf16 value.  Each term keeps the top 8 significand bits of what is
// left (truncation), so the subtractions are exact in f32 and 24 bits are used up after three terms.
__device__ __forceinline__ void split3(float x, float& hi, float& mid, float& lo) {
    hi = __uint_as_float(__float_as_uint(x) & 0xFFFF0000u);
    const float r1 = x - hi;
    mid = __uint_as_float(__float_as_uint(r1) & 0xFFFF0000u);
    lo = r1 - mid;
}
// 2^x on the special-function unit (relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// bf16 pair (first value in the low half) of two values that are already exactly representable in bf16
__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
    return __byte_perm(__float_as_uint(lo_elem), __float_as_uint(hi_elem), 0x7632);
}
// The two A-operand registers of one thread for values (x0, x1) at consecutive k: `upper` is the register of
// row g (term hi for g < 4, mid for g >= 4), `lower` the register of row g + 8 (term lo for g < 4, zero else).
__device__ __forceinline__ void split_pair(float x0, float x1, bool first_four, uint32_t& upper, uint32_t& lower) {
    float h0, m0, l0, h1, m1, l1;
    split3(x0, h0, m0, l0);
    split3(x1, h1, m1, l1);
    upper = first_four ? pack_bf16(h0, h1) : pack_bf16(m0, m1);
    lower = first_four ? pack_bf16(l0, l1) : 0u;
}

// byte offset inside a 4 KB tile of the 16-byte piece `chunk` (0..15 = 8 dims each) of token `tok`
__device__ __forceinline__ uint32_t tile_offset(int tok, int chunk) {
    return static_cast<uint32_t>((chunk >> 3) * 2048 + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4));
}

struct AttnItem {       // what the producer tells the consumers about a work item
    int row;            // query row = b * l_new + i
    int h0;             // first query head
    int chunk;
    int ntok;           // tokens of this chunk that take part
    int nb;             // blocks of this chunk
    int done;           // no more items
    int pad0, pad1;
};

constexpr int kItemSlots = 2;
constexpr int kQaStride = 272;          // bytes per row of the split q operand (16 bytes of padding: no bank conflicts)
constexpr float kLog2e = 1.4426950408889634f;

__host__ __device__ constexpr int attn_smem_bytes() {
    return 1024 + kStages * kTileBytes + kItemSlots * 4 * kD * 4 + kConsumerWarps * 4 * kD * 4 + 192 + 12 * kQaStride +
           kItemSlots * 32 + (2 * kStages + 3 * kItemSlots) * 8 + 64;
}

template <int G>
__global__ void __launch_bounds__(kFastThreads, kCtasPerSm)
paged_attention_decode_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                              const float* __restrict__ q, const uint32_t* __restrict__ block_tables,
                              const uint32_t* __restrict__ seq_lens, PagedAttnShape sh, int chunk_blocks,
                              int max_chunks, float* __restrict__ part_o, float* __restrict__ part_ml,
                              unsigned int* __restrict__ work_counter, uint32_t* err) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_dyn + (ring - smem_u32(smem_dyn));
    float* qbuf = reinterpret_cast<float*>(ring_ptr + kStages * kTileBytes);       // [slots][4 heads][128]
    float* red = qbuf + kItemSlots * 4 * kD;                                       // [4 warps][4 heads][128]
    float* red_m = red + kConsumerWarps * 4 * kD;                                  // [4 warps][4 heads]
    float* red_l = red_m + 16;
    int* abort_flag = reinterpret_cast<int*>(red_l + 16);                          // a consumer gave up waiting
    AttnItem* items = reinterpret_cast<AttnItem*>(red_l + 32);                     // [slots]
    uint8_t* qa_s = reinterpret_cast<uint8_t*>(items + kItemSlots);                // split q: [3 terms][4 heads] rows
    const uint32_t bars = smem_u32(qa_s + 12 * kQaStride);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    auto item_full = [&](int s) { return bars + 8u * (2 * kStages + s); };
    auto item_empty = [&](int s) { return bars + 8u * (2 * kStages + kItemSlots + s); };
    auto q_full = [&](int s) { return bars + 8u * (2 * kStages + 2 * kItemSlots + s); };

    pdl_wait();                 // q, the new K / V rows, seq_lens and the work counter come from earlier work
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 12 * kQaStride / 4; i += kFastThreads) reinterpret_cast<uint32_t*>(qa_s)[i] = 0u;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < kItemSlots; ++s) {
            mbar_init(item_full(s), 1);
            mbar_init(item_empty(s), kConsumerWarps);
            mbar_init(q_full(s), 1);
        }
        fence_barrier_init();
    }
    __syncthreads();

    const int chunk_tokens = chunk_blocks * kBS;
    const int group = sh.num_q_heads / sh.num_kv_heads;
    const int subs = group / G;                          // 1, or 2 when 8 query heads share a kv head
    const int nslots = sh.num_kv_heads * subs;
    const int rows = sh.batch * sh.l_new;
    const unsigned int total = static_cast<unsigned int>(max_chunks) * rows * nslots;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer warp
        if (lane == 0) { tma_prefetch_desc(&tma_k); tma_prefetch_desc(&tma_v); }
        int cnt[kConsumerWarps] = {0, 0, 0, 0};           // tiles handed to each consumer warp so far
        bool ok = true;
        for (int it = 0; ok; ++it) {
            // next non-empty item: chunk-major order, so the (always present) first chunks come first
            unsigned int idx = 0;
            int row = 0, kv_slot = 0, chunk = 0, ntok = 0;
            bool have = false;
            while (true) {
                if (lane == 0) idx = atomicAdd(work_counter, 1u);
                idx = __shfl_sync(0xffffffffu, idx, 0);
                if (idx >= total) break;
                chunk = idx / (rows * nslots);
                const int rem = idx % (rows * nslots);
                row = rem / nslots;
                kv_slot = rem % nslots;
                const int b = row / sh.l_new, i = row % sh.l_new;
                // a length above the table width or the planned number of chunks is clamped and flagged: neither
                // the table row nor the partials of another row are ever touched
                int64_t len = seq_lens[b];
                int64_t cap = int64_t(sh.max_blocks_per_seq) * sh.block_size;
                if (cap > int64_t(max_chunks) * chunk_tokens) cap = int64_t(max_chunks) * chunk_tokens;
                if (len > cap) {
                    if (lane == 0) atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnSeqLen));
                    len = cap;
                }
                const int limit = int(len) - sh.l_new + i + 1;
                ntok = limit - chunk * chunk_tokens;
                if (ntok > 0) { have = true; break; }
            }
            const int slot = it % kItemSlots;
            const uint32_t use_ph = (it / kItemSlots) & 1;
            if (lane == 0) ok = mbar_wait(item_empty(slot), use_ph ^ 1u, err, kErrProducerWait);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (!have) {
                if (lane == 0) {
                    items[slot].done = 1;
                    mbar_arrive(item_full(slot));
                }
                break;
            }
            if (ntok > chunk_tokens) ntok = chunk_tokens;
            const int nb = (ntok + kBS - 1) / kBS;
            const int kvh = kv_slot / subs;
            const int h0 = kvh * group + (kv_slot % subs) * G;
            if (lane == 0) {
                AttnItem d;
                d.row = row; d.h0 = h0; d.chunk = chunk; d.ntok = ntok; d.nb = nb; d.done = 0; d.pad0 = d.pad1 = 0;
                items[slot] = d;
                mbar_arrive_expect_tx(q_full(slot), G * kD * 4);
                bulk_load_1d(smem_u32(qbuf + slot * 4 * kD), q + (int64_t(row) * sh.num_q_heads + h0) * kD, G * kD * 4,
                             q_full(slot));
                mbar_arrive(item_full(slot));
            }
            const uint32_t* trow = block_tables + int64_t(row / sh.l_new) * sh.max_blocks_per_seq + chunk * chunk_blocks;
            uint32_t my_blk = 0;
            for (int j0 = 0; j0 < nb && ok; j0 += kConsumerWarps) {
                if ((j0 & 31) == 0) {                   // the lanes fetch the next 32 block ids in one go
                    my_blk = (j0 + lane < nb) ? trow[j0 + lane] : 0u;
                    if (my_blk >= uint32_t(sh.num_blocks)) {
                        atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnBlockId));
                        my_blk = 0;
                    }
                }
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {      // block j0 + w goes to consumer warp w
                    const uint32_t blk = __shfl_sync(0xffffffffu, my_blk, (j0 + w) & 31);
                    if (j0 + w < nb) {
                        if (lane == 0) {
#pragma unroll
                            for (int kv = 0; kv < 2 && ok; ++kv) {
                                const int li = cnt[w] + kv;
                                const int s = w * kStagesPerWarp + li % kStagesPerWarp;
                                const uint32_t ph = (li / kStagesPerWarp) & 1;
                                ok = mbar_wait(empty_bar(s), ph ^ 1u, err, kErrProducerWait);
                                if (ok) {
                                    mbar_arrive_expect_tx(full_bar(s), kTileBytes);
                                    tma_load_3d(ring + s * kTileBytes, kv == 0 ? &tma_k : &tma_v, full_bar(s), kvh * kD,
                                                int(blk) * kBS, 0);
                                }
                            }
                        }
                        cnt[w] += 2;
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
        return;
    }

    // ------------------------------------------------------------ consumers
    const int g = lane >> 2, t = lane & 3;      // fragment coordinates of this thread
    const int head = g & 3;                     // the query head this thread's rows belong to
    const bool first_four = g < 4;
    const bool head_ok = head < G;
    const int mat = lane >> 3, r8 = lane & 7;
    int my_tiles = 0;                           // tiles this warp has consumed so far (across items)
    // `ok` stays warp-uniform (every wait is followed by a vote), so the warp-wide instructions below always
    // run with all lanes.  A warp whose wait ran out keeps meeting the other warps at the two named barriers of
    // the item, raises abort_flag, and all four warps leave together after the merge step.
    bool ok = true;
    auto wait_warp = [&](uint32_t bar, uint32_t parity) {
        const bool r = mbar_wait(bar, parity, err, kErrAttnLoadWait);
        return __all_sync(0xffffffffu, r) != 0;
    };

    for (int it = 0;; ++it) {
        const int slot = it % kItemSlots;
        const uint32_t use_ph = (it / kItemSlots) & 1;
        if (ok) ok = wait_warp(item_full(slot), use_ph);
        AttnItem item;
        item.row = item.h0 = item.chunk = item.ntok = item.nb = 0;
        item.done = 1;
        if (ok) item = items[slot];
        const bool work = ok && !item.done;
        const int row = item.row, h0 = item.h0, chunk = item.chunk, ntok = item.ntok;
        const int nb = work ? item.nb : 0;

        // A operand of the score product: q * scale * log2(e) split into three bf16 terms (row 4 * term + head).
        // The 128 consumers build it once per item in shared memory, then every thread picks up its fragments
        // of all eight 16-dim k-steps.  (Scores come out in log2 units, so the softmax needs exp2 only.)
        if (work) ok = wait_warp(q_full(slot), use_ph);
        {
            const float qscale = sh.scale * kLog2e;
            const float* qp = qbuf + slot * 4 * kD;
            for (int pr = threadIdx.x; pr < G * (kD / 2); pr += 32 * kConsumerWarps) {
                const int hh = pr / (kD / 2), d = 2 * (pr % (kD / 2));
                const float2 x = *reinterpret_cast<const float2*>(qp + hh * kD + d);
                float h0v, m0v, l0v, h1v, m1v, l1v;
                split3(x.x * qscale, h0v, m0v, l0v);
                split3(x.y * qscale, h1v, m1v, l1v);
                *reinterpret_cast<uint32_t*>(qa_s + hh * kQaStride + 2 * d) = pack_bf16(h0v, h1v);
                *reinterpret_cast<uint32_t*>(qa_s + (4 + hh) * kQaStride + 2 * d) = pack_bf16(m0v, m1v);
                *reinterpret_cast<uint32_t*>(qa_s + (8 + hh) * kQaStride + 2 * d) = pack_bf16(l0v, l1v);
            }
        }
        consumer_sync();
        uint32_t qa[8][4];
        {
            const uint8_t* up = qa_s + g * kQaStride + 4 * t;            // row g: hi (g < 4) or mid term
            const uint8_t* lw = qa_s + (8 + (g & 3)) * kQaStride + 4 * t;  // row g + 8: lo term (g < 4) or zero
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qa[ks][0] = *reinterpret_cast<const uint32_t*>(up + 32 * ks);
                qa[ks][2] = *reinterpret_cast<const uint32_t*>(up + 32 * ks + 16);
                qa[ks][1] = first_four ? *reinterpret_cast<const uint32_t*>(lw + 32 * ks) : 0u;
                qa[ks][3] = first_four ? *reinterpret_cast<const uint32_t*>(lw + 32 * ks + 16) : 0u;
            }
        }

        float m_run = -INFINITY;        // running max of this thread's head over the warp's blocks
        float l_run = 0.0f;             // running sum of exp over this thread's four token columns
        float acc[16][4];               // acc[n] = D fragment of dims [8 n, 8 n + 8)
#pragma unroll
        for (int n = 0; n < 16; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;

        for (int j = warp; j < nb; j += kConsumerWarps) {
            // ---- scores of block j
            const int tk = my_tiles;
            const int sk = warp * kStagesPerWarp + tk % kStagesPerWarp;
            if (ok) ok = wait_warp(full_bar(sk), (tk / kStagesPerWarp) & 1);
            const uint32_t ktile = ring + sk * kTileBytes;
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};   // tokens 0..7 and 8..15
            {
                const int tok = (mat >> 1) * 8 + r8;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t kb[4];
                    ldmatrix_x4(ktile + tile_offset(tok, 2 * ks + (mat & 1)), kb);
                    mma_bf16(c0, qa[ks], kb[0], kb[1]);
                    mma_bf16(c1, qa[ks], kb[2], kb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(sk));
            // rows g and g + 8 of this thread, then the partner lane with the other rows of the same head
            float s00 = c0[0] + c0[2], s01 = c0[1] + c0[3], s10 = c1[0] + c1[2], s11 = c1[1] + c1[3];
            s00 += __shfl_xor_sync(0xffffffffu, s00, 16);
            s01 += __shfl_xor_sync(0xffffffffu, s01, 16);
            s10 += __shfl_xor_sync(0xffffffffu, s10, 16);
            s11 += __shfl_xor_sync(0xffffffffu, s11, 16);
            const int ct = j * kBS + 2 * t;             // token inside the chunk of the first of the four columns
            if (ct + 9 >= ntok) {                       // only the last block of a sequence has masked columns
                if (ct >= ntok) s00 = -INFINITY;
                if (ct + 1 >= ntok) s01 = -INFINITY;
                if (ct + 8 >= ntok) s10 = -INFINITY;
                s11 = -INFINITY;
            }
            float mt = fmaxf(fmaxf(s00, s01), fmaxf(s10, s11));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
            const float m_new = fmaxf(m_run, mt);       // finite: every block in range holds a valid token
            const float corr = exp2_fast(m_run - m_new);     // 2^(-inf) = 0 on the first block
            const float p00 = exp2_fast(s00 - m_new), p01 = exp2_fast(s01 - m_new);
            const float p10 = exp2_fast(s10 - m_new), p11 = exp2_fast(s11 - m_new);
            l_run = fmaf(l_run, corr, (p00 + p01) + (p10 + p11));
            m_run = m_new;
            if (corr != 1.0f) {
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    acc[n][0] *= corr; acc[n][1] *= corr; acc[n][2] *= corr; acc[n][3] *= corr;
                }
            }
            uint32_t pa[4];
            split_pair(p00, p01, first_four, pa[0], pa[1]);
            split_pair(p10, p11, first_four, pa[2], pa[3]);

            // ---- weighted sum of block j's V rows
            const int tv = tk + 1;
            const int sv = warp * kStagesPerWarp + tv % kStagesPerWarp;
            if (ok) ok = wait_warp(full_bar(sv), (tv / kStagesPerWarp) & 1);
            const uint32_t vtile = ring + sv * kTileBytes;
            const int valid = ntok - j * kBS;
            if (valid < kBS) {
                // rows past the sequence end may hold anything (0 x NaN would poison the sums): clear them
                uint8_t* tp = ring_ptr + sv * kTileBytes;
                for (int idx = lane; idx < (kBS - valid) * 16; idx += 32) {
                    const int tok = valid + idx / 16, ch = idx % 16;
                    *reinterpret_cast<uint4*>(tp + tile_offset(tok, ch)) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async();      // these stores precede the next TMA write into the same stage
                __syncwarp();
            }
            {
                const int tok = (mat & 1) * 8 + r8;
#pragma unroll
                for (int n2 = 0; n2 < 8; ++n2) {          // two 8-dim groups per ldmatrix
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vtile + tile_offset(tok, 2 * n2 + (mat >> 1)), vb);
                    mma_bf16(acc[2 * n2], pa, vb[0], vb[1]);
                    mma_bf16(acc[2 * n2 + 1], pa, vb[2], vb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(sv));
            my_tiles += 2;
        }

        // ---- park the warp's (max, sum, output) per head; rows h, 4 + h, 8 + h of the accumulator are head h
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (!ok && lane == 0) *abort_flag = 1;
        if (first_four && head_ok && t == 0) {
            red_m[warp * 4 + head] = m_run;
            red_l[warp * 4 + head] = l_run;
        }
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            float o0 = acc[n][0] + acc[n][2], o1 = acc[n][1] + acc[n][3];
            o0 += __shfl_xor_sync(0xffffffffu, o0, 16);
            o1 += __shfl_xor_sync(0xffffffffu, o1, 16);
            if (first_four && head_ok)
                *reinterpret_cast<float2*>(red + (warp * 4 + head) * kD + 8 * n + 2 * t) = make_float2(o0, o1);
        }
        consumer_sync();
        const bool leave = *abort_flag != 0 || item.done;     // the same answer in all four warps
        // ---- merge the four warps (warp order) and write the chunk's partial: unnormalised sum relative to
        // the chunk max, plus (max, sum)
        const int ctid = threadIdx.x;                    // 0..127
        for (int idx = ctid; work && idx < G * kD; idx += 128) {
            const int hh = idx / kD, d = idx % kD;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) mm = fmaxf(mm, red_m[w * 4 + hh]);
            float o = 0.0f, l = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float mw = red_m[w * 4 + hh];
                const float wgt = mw == -INFINITY ? 0.0f : exp2_fast(mw - mm);
                o = fmaf(red[(w * 4 + hh) * kD + d], wgt, o);
                l = fmaf(red_l[w * 4 + hh], wgt, l);
            }
            part_o[((int64_t(row) * sh.num_q_heads + h0 + hh) * max_chunks + chunk) * kD + d] = leave ? __int_as_float(0x7FC00000) : o;
            if (d == 0) {
                float* ml = part_ml + ((int64_t(row) * sh.num_q_heads + h0 + hh) * max_chunks + chunk) * 2;
                ml[0] = mm;
                ml[1] = l;
            }
        }
        consumer_sync();        // the parking area is free again before any warp parks the next item
        if (leave) break;
        if (lane == 0) mbar_arrive(item_empty(slot));
    }
}
