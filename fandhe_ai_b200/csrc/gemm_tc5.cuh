// Interface of the tcgen05 quantized GEMM (defined in gemm_tc5.cu).
//
//   acc[m, n] = sum_k A[m, k] * B[n, k]      A: [M, K] row-major, B: [N, K] row-major (both K-major)
//
// 8-bit operands (signed int8 -> s32 accumulator, or FP8 E4M3 -> f32 accumulator).
// Output is either the raw accumulators, optionally split along K into `splits`
// partial planes [splits][M][N] that a later row-wise kernel sums in plane order,
// or the fused epilogue  y = act(acc * sa[m] * sb[n] + bias[n]) (+ residual).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum GemmKind : int { kGemmI8 = 0, kGemmFp8 = 1 };
enum GemmAct : int { kActNone = 0, kActRelu = 1, kActSilu = 2, kActSiluGate = 3 };

// Optional finish of a QKV projection whose tiles are exactly one head wide (BN = head_dim = 128): dequantise
// (GemmEpilogue::a_scale per row, b_scale per column), rotate-half RoPE for the q and k heads with the row's
// position, then q as f32 [M, hq, 128] and k / v as bf16 into the paged pools at the slot the block table gives.
// Only the one-tile kernel with split-K inside a cluster implements it (gemm_launch refuses other plans).
struct GemmRope {
    int enabled = 0;
    int hq = 0, hkv = 0;                    // heads in this GEMM's N = (hq + 2 hkv) * 128
    const float* cos_t = nullptr;           // [max_pos, 64]
    const float* sin_t = nullptr;
    int max_pos = 0;
    const uint32_t* positions = nullptr;    // [M] position of the token of each row
    const uint32_t* active = nullptr;       // [M] or null: rows with active[m] == 0 leave the pools untouched
    const uint32_t* block_tables = nullptr; // [M, max_blocks_per_seq]
    int max_blocks_per_seq = 0, block_size = 0, num_blocks = 0;
    float* q_out = nullptr;
    uint16_t* k_pool = nullptr;
    uint16_t* v_pool = nullptr;
};

// Optional wait of a GEMM whose A operand (and per-row scales) are delivered by other GPUs: right before the first
// A tile is loaded, the producer warp waits until each of the `n` flags (epoch counters in this GPU's memory, raised
// by the peers) has reached *epoch.  The weight tiles of the first ring pass are already in flight by then.
struct GemmPeerWait {
    const uint32_t* flags = nullptr;   // [n]; null: no wait
    int n = 0;
    const uint32_t* epoch = nullptr;   // device word holding the epoch to wait for
    uint64_t timeout_ns = 0;
};

// Optional scatter of a row-parallel output over the GPUs of a tensor-parallel group (a reduce-scatter fused into the
// GEMM): the f32 rows of the fused epilogue are stored not into `out` but into the exchange block of the rank that
// owns the row (rank = row / rows), plane `rank` of its receive area [tp][rows][N], through the peer mappings with
// plain stores.  Every finished tile counts itself in *arrived (this GPU's memory); the tile that completes the launch
// resets that counter and adds one to count[rank] in the block of every rank (system-scope release), and the owner's
// finish kernel waits for the counts and sums its planes from local memory.
// Needs fused = 1 with f32 output, no residual and no gate; one-tile kernel only.
struct GemmPush {
    uint8_t* const* peers = nullptr;   // device table [tp] of block bases (this rank's own included); null: off
    size_t o_part = 0;                 // byte offset of the receive area in a block
    size_t o_count = 0;                // byte offset of count[tp] in a block
    int tp = 0, rank = 0;
    int rows = 0;                      // rows per owner
    unsigned int* arrived = nullptr;   // tiles of the running launch that have stored their rows (zero between launches)
};

struct GemmEpilogue {
    int fused = 0;                 // 0: write raw accumulators to `raw`; 1: fused epilogue to `out`
    void* raw = nullptr;           // [splits][M][N] int32 (i8) or f32 (fp8)
    const float* a_scale = nullptr;  // [M] when a_per_row else [1]
    int a_per_row = 0;
    const float* b_scale = nullptr;  // [N] when b_per_col else [1]
    int b_per_col = 0;
    const float* bias = nullptr;     // [N] (for the gate form: [N], gate half then up half) or null
    const float* residual = nullptr; // [M][N_out] f32 or null
    void* out = nullptr;             // [M][N_out] f32 or bf16
    int out_bf16 = 0;
    int act = kActNone;              // kActSiluGate: B rows [0, N/2) are gate, [N/2, N) are up, N_out = N/2
    GemmRope rope;                   // see GemmRope; needs fused = 1 with per-row / per-column scales, no bias
    GemmPeerWait wait;               // see GemmPeerWait
    GemmPush push;                   // see GemmPush
    // Profiling aid of the one-tile kernel: when not null, the first CTA of the launch writes %globaltimer (ns) at
    // nine points of its life (kGemmStamp*); costs one predicated branch per point otherwise.
    unsigned long long* stamps = nullptr;
};

enum GemmStamp : int {
    kGemmStampEntry = 0,        // first instruction of the CTA
    kGemmStampSetup = 1,        // barriers initialised, tensor memory allocated, CTA barrier passed
    kGemmStampDepWait = 2,      // producer: the kernel before this one has completed (griddepcontrol.wait returned)
    kGemmStampLoadsIssued = 3,  // producer: first pass over the ring issued (A and B tiles)
    kGemmStampFirstTile = 4,    // MMA warp: first stage has landed in shared memory
    kGemmStampMmaIssued = 5,    // MMA warp: last MMA issued and committed
    kGemmStampAccReady = 6,     // epilogue: accumulator complete in tensor memory
    kGemmStampStored = 7,       // epilogue: the first epilogue warp has issued its stores (after the cluster reduction, if any)
    kGemmStampExit = 8,         // tensor memory freed
    kGemmStampCount = 9
};

struct GemmPlan {
    CUtensorMap tma_a;
    CUtensorMap tma_b;
    int kind = kGemmI8;
    int M = 0, N = 0, K = 0;
    int bn = 128;      // CTA tile width (output columns; for the gate form bn/2 gate + bn/2 up rows of B)
    int stages = 3;
    int splits = 1;
    int gate = 0;
    int cluster = 0;     // the splits of a tile run as one cluster and reduce through distributed shared memory
    int out_planes = 1;  // raw planes the kernel writes: 1 with the cluster reduction, else `splits`
    // persistent form (gemm_plan_make_persistent): one CTA per SM takes whole tiles round-robin
    int persist = 0;
    int grid = 0;        // resident CTAs
    int pair = 0;        // persistent form on CTA pairs (cta_group::2): 256-row tiles, each CTA loads half of the B rows
    const void* b_ptr = nullptr;   // operand B as given to gemm_make_plan (the pair form re-encodes its tensor map)
};

// Output tiles of a one-tile-kernel launch of the plan.
int gemm_plan_tiles(const GemmPlan& plan);

// Switches a plan to the persistent kernel when the problem has enough tiles for `sm_count` SMs: half a wave when
// the launch will use a fused epilogue, two waves for raw accumulator output.  Afterwards splits == 1,
// out_planes == 1 and every epilogue (raw, fused, gated) is produced inside the launch.
void gemm_plan_make_persistent(GemmPlan* plan, int sm_count, bool fused_epilogue);

// Picks tile width / stage count / split count for a shape.  `want_splits` <= 0
// lets the heuristic choose (it only splits when the tile grid alone would leave
// most of the 148 SMs idle); the fused epilogue requires splits == 1.
// Returns cudaSuccess or an error; `why` receives a static message on failure.
// encode_maps = false fills in the shape decisions only (no tensor maps; the plan cannot be launched).
cudaError_t gemm_make_plan(GemmPlan* plan, int kind, const void* a, const void* b, int M, int N, int K,
                           int gate, int want_splits, int want_bn, const char** why, bool encode_maps = true);

// True when a launch of this plan may carry a GemmRope epilogue for hq + 2 hkv heads of 128.
bool gemm_plan_can_rope(const GemmPlan& plan, int hq, int hkv);

// Enqueues the GEMM on `stream`.  `err` is the context's device error word.
cudaError_t gemm_launch(const GemmPlan& plan, const GemmEpilogue& ep, uint32_t* err, cudaStream_t stream);

// Finish for raw planes: sums the `splits` planes [splits][M][N] in plane order and applies
// the epilogue (same arithmetic as the fused path).  With `gate` the planes come from a
// plain (gate = 0) plan over all N = 2F weight rows: gate columns [0, N/2), up columns [N/2, N).
cudaError_t gemm_splitk_epilogue(int kind, int splits, int M, int N, int gate, const void* raw,
                                 const GemmEpilogue& ep, cudaStream_t stream);
cudaError_t gemm_sum_planes_i32(const int* raw, int splits, int64_t elems, int* out, cudaStream_t stream);

// 2-D tensor map over a row-major [rows, cols] matrix of bytes with boxes of [box_rows, 128 bytes] and the 128-byte
// swizzle: the operand layout every tcgen05 kernel of this library consumes.
bool gemm_make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// ---- gemm_block_scaled.cu: INT8 GEMM under the block-scale contract (one power-of-two scale per 128 values of K on
// both operands; per block: s32 partial -> f32 -> one multiplication by the composed scale -> widened to f64; the
// blocks added in ascending order in f64; one narrowing to f32).
//   a [M, K] int8, a_delta [M, nb] f32;  b [N, K] int8, b_delta [nb, N] f32;  out [M, N] f32;  nb = ceil(K / 128).
// `status` is a device word: bit 1 is set when a result is not finite after the narrowing.
cudaError_t gemm_i8_block_scaled(const void* a, const float* a_delta, const void* b, const float* b_delta, int M, int N, int K,
                                 float* out, uint32_t* status, uint32_t* err, cudaStream_t stream, const char** why);

// Required raw-output elements for a plan: splits * M * N.
inline size_t gemm_raw_elems(const GemmPlan& p) { return size_t(p.out_planes) * size_t(p.M) * size_t(p.N); }

}  // namespace b200
