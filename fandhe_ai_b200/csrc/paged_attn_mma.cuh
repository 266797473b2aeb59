// Split-K decode attention, tensor-core form.  Included by paged_kv.cu inside its anonymous namespace
// (it uses kD, kBS, kTileBytes, kStages, kConsumerWarps, kFastThreads defined there).
//
// One CTA = one (query row, kv head, chunk of `chunk_blocks` KV blocks); G = 1, 2 or 4 query heads share the
// kv head.  A producer warp walks the chunk's block ids and, per block, issues the K tile and then the V tile
// as two TMA boxes each of [16 tokens x 64 dims] (128-byte rows, 128-byte swizzle, so ldmatrix reads them
// without bank conflicts) into kStages 4 KB stages.  Four consumer warps take blocks round-robin and keep a
// running (max, sum, accumulator) each - no barrier inside the chunk - and are merged at the end.  Every warp
// cycles through kStagesPerWarp stages of its own: consecutive uses of a stage are then waited for by the
// same warp in order, so a parity wait can never be two phases ahead of its barrier (a wait that far ahead
// would pass at once on a stage whose data has not landed).
//
// Both contractions run on mma.sync.m16n8k16 (bf16 x bf16 -> f32) with the f32 operand split into three
// bf16 terms that sum to it exactly (hi + mid + lo), one term per group of four rows of the 16-row A
// operand: row 4 * term + head.  The products with the bf16 K / V values are therefore exact and only the
// f32 accumulation order differs from a scalar f32 loop.
//   scores:  A = split(q * scale) [16 x 128],  B = K tile^T  -> C[row][token];  s = C[h] + C[4 + h] + C[8 + h]
//   output:  A = split(p)         [16 x 16],   B = V tile    -> D[row][dim];    o = D[h] + D[4 + h] + D[8 + h]
// The folded score of a thread lands exactly where the A operand of the second product wants it, so the
// weights never leave registers.

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

// x = hi + mid + lo with every term a bf16 value (the subtractions are exact in f32).
__device__ __forceinline__ void split3(float x, float& hi, float& mid, float& lo) {
    hi = bf16_bits_to_f32(f32_to_bf16_bits(x));
    const float r1 = x - hi;
    mid = bf16_bits_to_f32(f32_to_bf16_bits(r1));
    lo = bf16_bits_to_f32(f32_to_bf16_bits(r1 - mid));
}
// bf16 pair (first value in the low half) of two values that are already exactly representable in bf16
__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
    return (__float_as_uint(lo_elem) >> 16) | (__float_as_uint(hi_elem) & 0xFFFF0000u);
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

template <int G>
__global__ void __launch_bounds__(kFastThreads, 3)
paged_attention_decode_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                              const float* __restrict__ q, const uint32_t* __restrict__ block_tables,
                              const uint32_t* __restrict__ seq_lens, PagedAttnShape sh, int chunk_blocks,
                              int max_chunks, float* __restrict__ part_o, float* __restrict__ part_ml, uint32_t* err) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_dyn + (ring - smem_u32(smem_dyn));
    float* red = reinterpret_cast<float*>(ring_ptr + kStages * kTileBytes);   // [4 warps][4 heads][128]
    float* red_m = red + kConsumerWarps * 4 * kD;                             // [4 warps][4 heads]
    float* red_l = red_m + 16;                                                // [4 warps][4 heads]
    const uint32_t bars = smem_u32(red_l + 16);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };

    pdl_wait();                 // q, the new K / V rows and seq_lens come from the kernels before this one
    pdl_launch_dependents();
    const int chunk_tokens = chunk_blocks * kBS;
    // the kv heads of one (row, chunk) are neighbours in the grid: they run at about the same time and read
    // adjacent 256-byte pieces of the same 2 KB token rows
    const int kv_slot = blockIdx.x;
    const int chunk = blockIdx.y;
    const int row = blockIdx.z;
    const int b = row / sh.l_new, i = row % sh.l_new;
    const int group = sh.num_q_heads / sh.num_kv_heads;
    const int subs = group / G;
    const int kvh = kv_slot / subs;
    const int h0 = kvh * group + (kv_slot % subs) * G;
    const int limit = int(seq_lens[b]) - sh.l_new + i + 1;
    const int tok0 = chunk * chunk_tokens;
    if (tok0 >= limit) return;                      // the whole CTA leaves together
    int ntok = limit - tok0;
    if (ntok > chunk_tokens) ntok = chunk_tokens;
    const int nb = (ntok + kBS - 1) / kBS;          // blocks of this chunk

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer warp: tile 2 j = K of block j, tile 2 j + 1 = V of block j
        if (lane == 0) { tma_prefetch_desc(&tma_k); tma_prefetch_desc(&tma_v); }
        const uint32_t* trow = block_tables + int64_t(b) * sh.max_blocks_per_seq + chunk * chunk_blocks;
        uint32_t my_blk = 0;
        bool ok = true;
        for (int j = 0; j < nb; ++j) {
            if ((j & 31) == 0) {                    // the lanes fetch the next 32 block ids in one go
                my_blk = (j + lane < nb) ? trow[j + lane] : 0u;
                if (my_blk >= uint32_t(sh.num_blocks)) {
                    atomicCAS(err, 0u, static_cast<uint32_t>(kErrAttnBlockId));
                    my_blk = 0;
                }
            }
            const uint32_t blk = __shfl_sync(0xffffffffu, my_blk, j & 31);
            if (lane == 0) {
#pragma unroll
                for (int kv = 0; kv < 2 && ok; ++kv) {
                    // warp j % 4 owns block j; its tiles cycle through that warp's private stages
                    const int li = 2 * (j / kConsumerWarps) + kv;
                    const int s = (j % kConsumerWarps) * kStagesPerWarp + li % kStagesPerWarp;
                    const uint32_t ph = (li / kStagesPerWarp) & 1;
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, err, kErrProducerWait);
                    if (ok) {
                        mbar_arrive_expect_tx(full_bar(s), kTileBytes);
                        const CUtensorMap* map = kv == 0 ? &tma_k : &tma_v;
                        tma_load_2d(ring + s * kTileBytes, map, full_bar(s), kvh * kD, int(blk) * kBS);
                        tma_load_2d(ring + s * kTileBytes + 2048, map, full_bar(s), kvh * kD + 64, int(blk) * kBS);
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers
    const int g = lane >> 2, t = lane & 3;      // fragment coordinates of this thread
    const int head = g & 3;                     // the query head this thread's rows belong to
    const bool first_four = g < 4;
    const bool head_ok = head < G;

    // A operand of the score product: q * scale split into three bf16 terms, all eight 16-dim k-steps
    uint32_t qa[8][4];
    {
        const float* qp = q + (int64_t(row) * sh.num_q_heads + h0 + (head_ok ? head : 0)) * kD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            float2 x = *reinterpret_cast<const float2*>(qp + 16 * ks + 2 * t);
            float2 y = *reinterpret_cast<const float2*>(qp + 16 * ks + 2 * t + 8);
            if (!head_ok) { x = make_float2(0.f, 0.f); y = make_float2(0.f, 0.f); }
            split_pair(x.x * sh.scale, x.y * sh.scale, first_four, qa[ks][0], qa[ks][1]);
            split_pair(y.x * sh.scale, y.y * sh.scale, first_four, qa[ks][2], qa[ks][3]);
        }
    }

    float m_run = -INFINITY;        // running max of this thread's head over the warp's blocks
    float l_run = 0.0f;             // running sum of exp over this thread's four token columns
    float acc[16][4];               // acc[n] = D fragment of dims [8 n, 8 n + 8)
#pragma unroll
    for (int n = 0; n < 16; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    bool ok = true;
    const int mat = lane >> 3, r8 = lane & 7;

    for (int j = warp; j < nb; j += kConsumerWarps) {
        // ---- scores of block j
        const int tk = 2 * (j / kConsumerWarps);    // index of the K tile among this warp's tiles
        const int sk = warp * kStagesPerWarp + tk % kStagesPerWarp;
        ok = ok && mbar_wait(full_bar(sk), (tk / kStagesPerWarp) & 1, err, kErrAttnLoadWait);
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
        if (ct >= ntok) s00 = -INFINITY;
        if (ct + 1 >= ntok) s01 = -INFINITY;
        if (ct + 8 >= ntok) s10 = -INFINITY;
        if (ct + 9 >= ntok) s11 = -INFINITY;
        float mt = fmaxf(fmaxf(s00, s01), fmaxf(s10, s11));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
        const float m_new = fmaxf(m_run, mt);       // finite: every block in range holds a valid token
        const float corr = expf(m_run - m_new);     // exp(-inf) = 0 on the first block
        const float p00 = expf(s00 - m_new), p01 = expf(s01 - m_new);
        const float p10 = expf(s10 - m_new), p11 = expf(s11 - m_new);
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
        ok = ok && mbar_wait(full_bar(sv), (tv / kStagesPerWarp) & 1, err, kErrAttnLoadWait);
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
    }

    // ---- park the warp's (max, sum, output) per head; rows h, 4 + h, 8 + h of the accumulator are head h
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
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
    // ---- merge the four warps (warp order) and write the chunk's partial: unnormalised sum relative to the
    // chunk max, plus (max, sum)
    const int ctid = threadIdx.x;                    // 0..127
    for (int idx = ctid; idx < G * kD; idx += 128) {
        const int hh = idx / kD, d = idx % kD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) mm = fmaxf(mm, red_m[w * 4 + hh]);
        float o = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const float mw = red_m[w * 4 + hh];
            const float wgt = mw == -INFINITY ? 0.0f : expf(mw - mm);
            o = fmaf(red[(w * 4 + hh) * kD + d], wgt, o);
            l = fmaf(red_l[w * 4 + hh], wgt, l);
        }
        part_o[((int64_t(row) * sh.num_q_heads + h0 + hh) * max_chunks + chunk) * kD + d] = ok ? o : __int_as_float(0x7FC00000);
        if (d == 0) {
            float* ml = part_ml + ((int64_t(row) * sh.num_q_heads + h0 + hh) * max_chunks + chunk) * 2;
            ml[0] = mm;
            ml[1] = l;
        }
    }
}
