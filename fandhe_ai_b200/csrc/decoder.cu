// C-ABI implementation, part 3: the decode driver.
//
//  - BlockTable: the host page table of the reference (crates/autodiff/src/nn/paged_kv.rs:158-364):
//    LIFO stack of returned blocks, then fresh ids counted up from 0; row-major slot mapping
//    block_id * block_size + pos % block_size; flattened [B, max_blocks_per_seq] padded with
//    0xFFFFFFFF; rewind returns tail blocks.  Extension: per-row reservation for ragged batches.
//  - ParamStore: flat device buffers (int8 payload, f32 scales, f32 vectors) addressed by
//    offset, the addressing model of DeviceParamStore
//    (crates/autodiff/src/optim/device_store.rs:1288-1364).
//  - Decoder: a Llama-style stack (RMSNorm, RoPE, GQA paged attention, SwiGLU) run as one CUDA
//    graph per decode step; greedy sampling on the device; only token ids cross to the host
//    (the reference's generate() loop, crates/autodiff/src/generate/mod.rs:500-613, pulls full
//    logits to the host each step).
//  - Tensor parallelism: QKV / gate / up column-parallel, O / down row-parallel, KV cache sharded
//    by KV head; the row-parallel outputs are summed across ranks with ncclAllReduce on the
//    context's stream.  NCCL is loaded with dlopen so that single-GPU use has no such dependency.
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "backend.h"
#include "gemm_tc5.cuh"
#include "kernels.cuh"
#include "safetensors.h"

using namespace b200;

// ------------------------------------------------------------------------------------ BlockTable
struct b200_block_table {
    uint64_t max_blocks = 0;
    uint64_t block_size = 1;
    std::vector<uint32_t> returned;
    uint64_t next_unused = 0;
    std::vector<std::vector<uint32_t>> tables;
    std::vector<uint64_t> seq_lens;
    bool has_batch = false;

    uint64_t free_blocks() const { return returned.size() + (max_blocks > next_unused ? max_blocks - next_unused : 0); }
    bool alloc(uint32_t* out) {
        if (!returned.empty()) {
            *out = returned.back();
            returned.pop_back();
            return true;
        }
        if (next_unused < max_blocks) {
            *out = static_cast<uint32_t>(next_unused++);
            return true;
        }
        return false;
    }
    void reset() {
        returned.clear();
        next_unused = 0;
        tables.clear();
        seq_lens.clear();
        has_batch = false;
    }
    uint64_t seq_len() const { return seq_lens.empty() ? 0 : seq_lens[0]; }
};

namespace {

int32_t bt_invalid(const std::string& m) { return fail(B200_INVALID_ARGUMENT, "block_table: " + m); }

// Grows row `row` so that it can hold `total` tokens.  Returns false when the pool runs out.
bool bt_reserve_row(b200_block_table* t, size_t row, uint64_t total) {
    const uint64_t need = (total + t->block_size - 1) / t->block_size;
    while (t->tables[row].size() < need) {
        uint32_t id;
        if (!t->alloc(&id)) return false;
        t->tables[row].push_back(id);
    }
    return true;
}

}  // namespace

extern "C" {

int32_t b200_block_table_create(uint64_t max_blocks, uint64_t block_size, b200_block_table** out) {
    if (!out) return bt_invalid("out is null");
    *out = nullptr;
    if (block_size == 0 || block_size > 256 || (block_size & (block_size - 1)) != 0)
        return bt_invalid("block_size must be a power of two in 1..256");
    if (max_blocks == 0 || max_blocks >= 0xFFFFFFFFull) return bt_invalid("max_blocks must be in 1..u32::MAX-1");
    b200_block_table* t = new (std::nothrow) b200_block_table();
    if (!t) return fail(B200_DEVICE_ALLOCATION_FAILED, "block_table: host allocation failed");
    t->max_blocks = max_blocks;
    t->block_size = block_size;
    *out = t;
    return B200_OK;
}

void b200_block_table_destroy(b200_block_table* t) { delete t; }

// BlockTable::extend_for_append (paged_kv.rs:206-297): all rows advance by l_new; slots are row-major.
// State is left unchanged on failure.
int32_t b200_block_table_extend_for_append(b200_block_table* t, uint64_t batch, uint64_t l_new, uint32_t* slots_out,
                                           uint64_t slots_capacity, uint64_t* n_slots) {
    if (!t) return bt_invalid("table is null");
    if (n_slots) *n_slots = 0;
    if (batch == 0) return bt_invalid("batch size 0 cannot be appended");
    if (t->has_batch && t->tables.size() != batch)
        return bt_invalid("batch " + std::to_string(batch) + " differs from the cache's " + std::to_string(t->tables.size()));
    if (l_new == 0) return B200_OK;
    const uint64_t s_prev = t->seq_len();
    uint64_t s_total, extra_total, rows;
    if (__builtin_add_overflow(s_prev, l_new, &s_total)) return bt_invalid("sequence length overflows");
    const uint64_t held = (s_prev + t->block_size - 1) / t->block_size;
    const uint64_t extra_per_row = (s_total + t->block_size - 1) / t->block_size - held;
    if (__builtin_mul_overflow(extra_per_row, batch, &extra_total)) return bt_invalid("needed block count overflows");
    if (extra_total > t->free_blocks())
        return bt_invalid("not enough free blocks (needed " + std::to_string(extra_total) + ", free " +
                          std::to_string(t->free_blocks()) + ")");
    if (__builtin_mul_overflow(batch, l_new, &rows)) return bt_invalid("append row count overflows");
    if (rows > slots_capacity || !slots_out) return bt_invalid("slot buffer too small");
    if ((t->max_blocks * t->block_size) > 0xFFFFFFFFull) return bt_invalid("slot number does not fit u32");
    if (!t->has_batch) {
        t->tables.assign(batch, {});
        t->seq_lens.assign(batch, 0);
        t->has_batch = true;
    }
    uint64_t at = 0;
    for (uint64_t row = 0; row < batch; ++row) {
        for (uint64_t i = 0; i < l_new; ++i) {
            const uint64_t pos = s_prev + i;
            if (pos % t->block_size == 0) {
                uint32_t id = 0;
                t->alloc(&id);   // cannot fail: checked above
                t->tables[row].push_back(id);
            }
            const uint32_t blk = t->tables[row][pos / t->block_size];
            slots_out[at++] = static_cast<uint32_t>(uint64_t(blk) * t->block_size + pos % t->block_size);
        }
    }
    for (auto& l : t->seq_lens) l = s_total;
    if (n_slots) *n_slots = rows;
    return B200_OK;
}

// BlockTable::flatten_tables (paged_kv.rs:299-322)
int32_t b200_block_table_flatten(const b200_block_table* t, uint64_t max_blocks_per_seq, uint32_t* out, uint64_t capacity) {
    if (!t) return bt_invalid("table is null");
    uint64_t n;
    if (__builtin_mul_overflow(uint64_t(t->tables.size()), max_blocks_per_seq, &n)) return bt_invalid("flattened size overflows");
    if (n > capacity || (n > 0 && !out)) return bt_invalid("output buffer too small");
    uint64_t at = 0;
    for (const auto& row : t->tables) {
        if (row.size() > max_blocks_per_seq) return bt_invalid("a row holds more blocks than max_blocks_per_seq");
        for (uint32_t id : row) out[at++] = id;
        for (uint64_t i = row.size(); i < max_blocks_per_seq; ++i) out[at++] = 0xFFFFFFFFu;
    }
    return B200_OK;
}

// BlockTable::rewind_to (paged_kv.rs:324-364)
int32_t b200_block_table_rewind_to(b200_block_table* t, uint64_t new_len) {
    if (!t) return bt_invalid("table is null");
    const uint64_t cur = t->seq_len();
    if (new_len > cur) return bt_invalid("rewind target " + std::to_string(new_len) + " exceeds the length " + std::to_string(cur));
    if (!t->has_batch || new_len == cur) return B200_OK;
    if (new_len == 0) {
        t->reset();
        return B200_OK;
    }
    const uint64_t keep = (new_len + t->block_size - 1) / t->block_size;
    for (auto& row : t->tables)
        while (row.size() > keep) {
            t->returned.push_back(row.back());
            row.pop_back();
        }
    for (auto& l : t->seq_lens) l = new_len;
    return B200_OK;
}

void b200_block_table_clear(b200_block_table* t) {
    if (t) t->reset();
}
uint64_t b200_block_table_seq_len(const b200_block_table* t) { return t ? t->seq_len() : 0; }
uint64_t b200_block_table_free_blocks(const b200_block_table* t) { return t ? t->free_blocks() : 0; }
uint64_t b200_block_table_used_blocks(const b200_block_table* t) {
    if (!t) return 0;
    uint64_t n = 0;
    for (const auto& r : t->tables) n += r.size();
    return n;
}
int64_t b200_block_table_batch(const b200_block_table* t) { return (t && t->has_batch) ? int64_t(t->tables.size()) : -1; }

}  // extern "C"

// ------------------------------------------------------------------------------------ NCCL (dlopen)
namespace {

// Head of an exchange block: ready[tp] at +0, delivered[tp] at +256, count[tp] at +512 (32-bit words).
constexpr size_t kTpCountOffset = 512;
constexpr size_t kTpFlagBytes = 768;

typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
enum { kNcclInt8 = 0, kNcclInt32 = 2, kNcclFloat32 = 7 };
enum { kNcclSum = 0, kNcclMax = 2 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.handle) return a;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(a.handle, "ncclAllGather"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce;
        return a;
    }();
    return api;
}

}  // namespace

// ------------------------------------------------------------------------------------ Decoder
struct LayerParams {
    size_t wqkv = 0, wo = 0, wgu = 0, wdown = 0;                  // byte offsets into the int8 payload
    size_t s_qkv = 0, s_o = 0, s_gu = 0, s_down = 0;              // element offsets into the scale buffer
    size_t attn_norm = 0, mlp_norm = 0;                           // element offsets into the vector buffer
    void* k_pool = nullptr;
    void* v_pool = nullptr;
    GemmPlan p_qkv, p_o, p_gu, p_down;
    bool rope_fused = false;                    // the QKV GEMM finishes with RoPE + cache append itself
    PagedAttnPlan attn;
};

struct b200_decoder {
    b200_ctx* ctx = nullptr;
    uint64_t generation = 0;                    // generation of the context at creation
    b200_decoder_config cfg{};
    int hq_l = 0, hkv_l = 0, f_l = 0;           // per-rank head counts and d_ff
    int n_qkv = 0;                              // (hq_l + 2 hkv_l) * head_dim
    // ParamStore
    int8_t* payload = nullptr;
    float* scales = nullptr;
    float* vectors = nullptr;                   // norm weights
    float* embed = nullptr;                     // [vocab, d] f32
    size_t payload_bytes = 0, scales_elems = 0, vectors_elems = 0;
    std::vector<LayerParams> layers;
    size_t w_lm = 0, s_lm = 0, final_norm = 0;
    GemmPlan p_lm;
    // rope
    float* cos_t = nullptr;
    float* sin_t = nullptr;
    // step state
    int batch = 0;
    int max_total_len = 0;
    std::vector<int> row_limits;                // tokens each row may hold in this generation
    bool planned = false;
    b200_block_table* table = nullptr;
    uint32_t* tables_dev = nullptr;
    uint32_t* seq_lens_dev = nullptr;
    uint32_t* pos_dev = nullptr;                // position of the token being added, per row
    uint32_t* active_dev = nullptr;             // 1: the row takes part in the step, 0: it sits the step out
    uint32_t* active_pinned = nullptr;
    std::vector<uint8_t> active_host;           // what active_dev holds
    int max_blocks_per_seq = 0;
    int* ids_dev = nullptr;
    int* next_ids_dev = nullptr;
    float* h = nullptr;
    int8_t* xq = nullptr;
    float* sx = nullptr;
    int* raw = nullptr;
    size_t raw_elems = 0;
    float* q = nullptr;
    float* attn_out = nullptr;
    float* part = nullptr;                      // [M, d] f32 addend of the cross-rank sum
    float* logits = nullptr;
    void* attn_scratch = nullptr;
    int* ids_pinned = nullptr;
    cudaEvent_t ids_copied = nullptr;           // the staged ids of the previous step have reached the device
    bool ids_copy_pending = false;
    int* next_pinned = nullptr;
    // graph
    cudaGraphExec_t graph = nullptr;
    int eager_steps_done = 0;
    uint64_t steps = 0;
    bool store_poisoned = false;
    // tensor parallel
    ncclComm_t comm = nullptr;
    // Exchange block (tp_size > 1): flags, sx, xq and the f32 partial `part` live in one allocation that the other
    // ranks map through CUDA IPC, so that the finish kernel can read partials from and deliver rows to every rank.
    uint8_t* tp_block = nullptr;
    size_t tp_block_bytes = 0;
    size_t tp_o_sx = 0, tp_o_xq = 0, tp_o_part = 0;
    void* tp_peer_ptrs[16] = {};                // host copy of the mapped bases (own block at tp_rank)
    uint8_t** tp_peers_dev = nullptr;           // the same table on the device
    uint32_t* tp_epoch = nullptr;               // [0] call counter, [1] CTA arrival counter of the finish kernel,
                                                // [2] scattered outputs finished so far, [3] tile counter of the
                                                // GEMM that scatters
    bool tp_push = true;                        // row-parallel GEMMs scatter their rows over the owners' blocks
    bool tp_push_all = true;                    // ... and every row-parallel GEMM of the last enqueued step could
    bool tp_exchange = false;                   // peers are mapped: use the finish kernel instead of ncclAllReduce
    uint64_t tp_timeout_ns = 0;                 // bound of every cross-GPU wait (0: the kernels' default of two seconds)
    // exact integer sums under tensor parallelism (cfg.tp_exact_int8): merged row maxima, f32 rows before the
    // quantiser, the int32 sum of the planes that goes through the all-reduce
    float* tp_amax = nullptr;                   // [M]
    float* tp_rows_f32 = nullptr;               // [M, max(f_l, hq_l * head_dim)]
    int* tp_acc = nullptr;                      // [M, d_model]
    uint64_t launches_per_step = 0;
    // multi-token prefill: buffers for up to prefill_rows token rows (grown on demand)
    struct Prefill {
        size_t rows = 0;
        int* ids = nullptr;
        uint32_t* pos = nullptr;
        float* h = nullptr;
        int8_t* xq = nullptr;
        float* sx = nullptr;
        int* raw = nullptr;
        size_t raw_elems = 0;
        float* q = nullptr;
        float* attn = nullptr;
        float* part = nullptr;
        void* attn_scratch = nullptr;
        size_t attn_scratch_bytes = 0;
    } pf;
};

namespace {

int32_t dec_fail(b200_decoder* d, int32_t st, const std::string& msg) {
    if (d) d->store_poisoned = true;
    return fail_runtime(d ? d->ctx : nullptr, st, msg);
}

#define CU_TRY(expr)                                                                                         \
    do {                                                                                                     \
        cudaError_t _e = (expr);                                                                             \
        if (_e != cudaSuccess)                                                                               \
            return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

template <typename T>
cudaError_t dmalloc(T** p, size_t elems) {
    return cudaMalloc(reinterpret_cast<void**>(p), elems * sizeof(T) > 0 ? elems * sizeof(T) : 16);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int32_t check_config(const b200_decoder_config& c) {
    auto bad = [](const char* m) { return fail(B200_INVALID_ARGUMENT, std::string("decoder config: ") + m); };
    if (c.n_layers <= 0 || c.d_model <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.d_ff <= 0 ||
        c.vocab <= 0)
        return bad("all sizes must be positive");
    if (c.n_heads % c.n_kv_heads != 0) return bad("n_heads must be a multiple of n_kv_heads");
    if (c.head_dim % 2 != 0) return bad("head_dim must be even (rotary pairs)");
    if (c.tp_size <= 0 || c.tp_rank < 0 || c.tp_rank >= c.tp_size) return bad("tp_rank / tp_size out of range");
    if (c.n_kv_heads % c.tp_size != 0 || c.d_ff % c.tp_size != 0) return bad("n_kv_heads and d_ff must divide by tp_size");
    if (c.d_model % 16 != 0 || (c.d_ff / c.tp_size) % 16 != 0 || (c.n_heads / c.tp_size * c.head_dim) % 16 != 0 ||
        c.vocab % 16 != 0 || (c.head_dim * (c.n_heads + 2 * c.n_kv_heads) / c.tp_size) % 16 != 0)
        return fail(B200_UNSUPPORTED, "decoder config: GEMM dimensions must be multiples of 16");
    if (c.max_batch <= 0 || c.max_seq_len <= 0) return bad("max_batch / max_seq_len must be positive");
    if (c.tp_exact_int8 && c.tp_size > 1 &&
        (!rows_scaled_supported(c.d_ff / c.tp_size) || !rows_scaled_supported(c.n_heads / c.tp_size * c.head_dim)))
        return fail(B200_UNSUPPORTED, "decoder config: tp_exact_int8 needs rows of at most 16384 columns per rank");
    if (c.act_fp8) {
        if (c.tp_exact_int8) return fail(B200_UNSUPPORTED, "decoder config: act_fp8 and tp_exact_int8 exclude each other");
        if (!rows_scaled_supported(c.d_model) || !rows_scaled_supported(c.d_ff / c.tp_size) || !rows_scaled_supported(c.d_ff) ||
            !rows_scaled_supported(c.n_heads / c.tp_size * c.head_dim) || !rows_scaled_supported(c.n_heads * c.head_dim))
            return fail(B200_UNSUPPORTED, "decoder config: act_fp8 needs rows of at most 16384 columns, multiples of 4");
    }
    if (c.block_size <= 0 || c.block_size > 256 || (c.block_size & (c.block_size - 1))) return bad("block_size must be a power of two <= 256");
    if (c.num_blocks <= 0) return bad("num_blocks must be positive");
    if (!(c.rms_eps >= 0.0f) || !std::isfinite(c.rms_eps)) return bad("rms_eps must be finite and non-negative");
    if (!(c.rope_theta > 0.0f)) return bad("rope_theta must be positive");
    return B200_OK;
}

int32_t dec_check(b200_decoder* d) {
    if (!d) return fail(B200_INVALID_ARGUMENT, "decoder is null");
    if (d->store_poisoned) return fail(B200_STORE_POISONED, "the decoder's device state is poisoned by an earlier runtime failure; re-create it");
    if (int32_t st = check_ctx(d->ctx)) return st;
    if (d->generation != d->ctx->generation)
        return fail(B200_STALE_DEVICE_GENERATION, "the decoder belongs to an earlier generation of its context (the context was recovered); re-create it");
    return set_device(d->ctx);
}

void drop_graph(b200_decoder* d) {
    if (d->graph) {
        cudaGraphExecDestroy(d->graph);
        d->graph = nullptr;
    }
    d->eager_steps_done = 0;
}

// Keeps this rank's shard of a full quantised matrix (int8 [rows, cols] and one scale per row, both on the device):
// either a row subset or a column slice goes into the payload; the scales follow.
int32_t store_weight_q(b200_decoder* d, const int8_t* q_full, const float* s_full, int64_t cols,
                       const std::vector<std::pair<int64_t, int64_t>>& row_ranges, int64_t c0, int64_t ccount, size_t payload_off,
                       size_t scale_off) {
    cudaStream_t s = d->ctx->stream;
    size_t out_row = 0;
    for (auto rr : row_ranges) {
        const int64_t r0 = rr.first, rn = rr.second;
        CU_TRY(slice_cols_i8(q_full + r0 * cols, rn, cols, c0, ccount, d->payload + payload_off + out_row * ccount, s));
        CU_TRY(cudaMemcpyAsync(d->scales + scale_off + out_row, s_full + r0, rn * sizeof(float), cudaMemcpyDeviceToDevice, s));
        out_row += rn;
    }
    CU_TRY(cudaStreamSynchronize(s));
    return B200_OK;
}

// Quantises a full f32 matrix [rows, cols] (device, temporary) per row and keeps this rank's shard.
int32_t store_weight(b200_decoder* d, const float* w_full, int64_t rows, int64_t cols, const std::vector<std::pair<int64_t, int64_t>>& row_ranges,
                     int64_t c0, int64_t ccount, size_t payload_off, size_t scale_off) {
    cudaStream_t s = d->ctx->stream;
    int8_t* q_full = nullptr;
    float* s_full = nullptr;
    CU_TRY(dmalloc(&q_full, size_t(rows) * cols));
    CU_TRY(dmalloc(&s_full, size_t(rows)));
    if (d->cfg.act_fp8) {
        // E4M3 codes under one scale per output row (amax / 448): the row quantiser of the activations, run over the weight rows
        if (rows > 0x7FFFFFFF || cols > 0x7FFFFFFF) return fail(B200_UNSUPPORTED, "decoder: weight too large for the FP8 encoder");
        CU_TRY(quantize_rows_auto(w_full, int(rows), int(cols), q_full, s_full, s, 1));
    } else {
        CU_TRY(quantize_i8_per_row(w_full, rows, cols, q_full, s_full, s));
    }
    const int32_t st = store_weight_q(d, q_full, s_full, cols, row_ranges, c0, ccount, payload_off, scale_off);
    cudaFree(q_full);
    cudaFree(s_full);
    return st;
}

struct TensorShape {
    int64_t rows, cols;                                        // full (unsharded) shape
    std::vector<std::pair<int64_t, int64_t>> row_ranges;       // rows kept by this rank
    int64_t c0, ccount;                                        // columns kept by this rank
    size_t payload_off, scale_off;
};

// Which rows and columns of a full weight matrix rank `tp_rank` keeps (pure host arithmetic):
// column-parallel matrices (QKV, gate/up) keep row ranges, row-parallel ones (O, down) keep a column range.
bool shard_of(const b200_decoder_config& c, int which, TensorShape* t) {
    const int tp = c.tp_size, r = c.tp_rank;
    const int64_t dh = c.head_dim, dm = c.d_model;
    const int64_t hq = c.n_heads, hkv = c.n_kv_heads, F = c.d_ff;
    switch (which) {
        case B200_W_LM_HEAD:
            *t = {c.vocab, dm, {{0, c.vocab}}, 0, dm, 0, 0};
            return true;
        case B200_W_QKV:
            *t = {(hq + 2 * hkv) * dh, dm,
                  {{r * (hq / tp) * dh, (hq / tp) * dh}, {hq * dh + r * (hkv / tp) * dh, (hkv / tp) * dh},
                   {(hq + hkv) * dh + r * (hkv / tp) * dh, (hkv / tp) * dh}},
                  0, dm, 0, 0};
            return true;
        case B200_W_O:
            *t = {dm, hq * dh, {{0, dm}}, r * (hq / tp) * dh, (hq / tp) * dh, 0, 0};
            return true;
        case B200_W_GATE_UP:
            *t = {2 * F, dm, {{r * (F / tp), F / tp}, {F + r * (F / tp), F / tp}}, 0, dm, 0, 0};
            return true;
        case B200_W_DOWN:
            *t = {dm, F, {{0, dm}}, r * (F / tp), F / tp, 0, 0};
            return true;
        default: return false;
    }
}

bool tensor_shape(const b200_decoder* d, int which, int layer, TensorShape* t) {
    if (!shard_of(d->cfg, which, t)) return false;
    if (which == B200_W_LM_HEAD) {
        t->payload_off = d->w_lm;
        t->scale_off = d->s_lm;
        return true;
    }
    if (layer < 0 || layer >= d->cfg.n_layers) return false;
    const LayerParams& L = d->layers[layer];
    switch (which) {
        case B200_W_QKV: t->payload_off = L.wqkv; t->scale_off = L.s_qkv; break;
        case B200_W_O: t->payload_off = L.wo; t->scale_off = L.s_o; break;
        case B200_W_GATE_UP: t->payload_off = L.wgu; t->scale_off = L.s_gu; break;
        default: t->payload_off = L.wdown; t->scale_off = L.s_down; break;
    }
    return true;
}

// Maps every other rank's exchange block into this process (CUDA IPC; the 64-byte handles travel through an
// ncclAllGather) and uploads the table of bases.  On any failure the decoder keeps the ncclAllReduce path.
// B200_TP_EXCHANGE=0 in the environment keeps that path too.
void map_peer_blocks(b200_decoder* d) {
    d->tp_exchange = false;
    const int tp = d->cfg.tp_size, rank = d->cfg.tp_rank;
    const char* env = std::getenv("B200_TP_EXCHANGE");
    if (env && env[0] == '0') return;
    if (tp < 2 || tp > 16 || !d->tp_block || !nccl().AllGather) return;
    if (d->cfg.tp_exact_int8) return;          // the exact mode sums integers through ncclAllReduce
    if (d->cfg.max_batch % tp != 0 || !tp_finish_supported(d->cfg.d_model)) return;
    cudaStream_t s = d->ctx->stream;
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, d->tp_block) != cudaSuccess) { cudaGetLastError(); return; }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    uint8_t* dev = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&dev), size_t(tp) * 64) != cudaSuccess) { cudaGetLastError(); return; }
    std::vector<cudaIpcMemHandle_t> all(tp);
    bool ok = cudaMemcpyAsync(dev + size_t(rank) * 64, &mine, 64, cudaMemcpyHostToDevice, s) == cudaSuccess;
    ok = ok && nccl().AllGather(dev + size_t(rank) * 64, dev, 64, kNcclInt8, d->comm, s) == 0;
    ok = ok && cudaMemcpyAsync(all.data(), dev, size_t(tp) * 64, cudaMemcpyDeviceToHost, s) == cudaSuccess;
    ok = ok && cudaStreamSynchronize(s) == cudaSuccess;
    cudaFree(dev);
    if (!ok) { cudaGetLastError(); return; }
    for (int p = 0; p < tp; ++p) {
        if (p == rank) { d->tp_peer_ptrs[p] = d->tp_block; continue; }
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            for (int q = 0; q < p; ++q)
                if (q != rank && d->tp_peer_ptrs[q]) { cudaIpcCloseMemHandle(d->tp_peer_ptrs[q]); d->tp_peer_ptrs[q] = nullptr; }
            ok = false;
            break;
        }
        d->tp_peer_ptrs[p] = ptr;
    }
    // every rank must take the same path: agree through a sum over the ranks
    int* flag = nullptr;
    int agreed = 0;
    if (cudaMalloc(reinterpret_cast<void**>(&flag), sizeof(int)) == cudaSuccess) {
        const int one = ok ? 1 : 0;
        bool f = cudaMemcpyAsync(flag, &one, sizeof(int), cudaMemcpyHostToDevice, s) == cudaSuccess;
        f = f && nccl().AllReduce(flag, flag, 1, kNcclInt32, kNcclSum, d->comm, s) == 0;
        f = f && cudaMemcpyAsync(&agreed, flag, sizeof(int), cudaMemcpyDeviceToHost, s) == cudaSuccess;
        f = f && cudaStreamSynchronize(s) == cudaSuccess;
        cudaFree(flag);
        if (!f) agreed = 0;
    }
    cudaGetLastError();
    if (agreed != tp) return;
    if (cudaMemcpy(d->tp_peers_dev, d->tp_peer_ptrs, size_t(tp) * sizeof(void*), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    d->tp_exchange = true;
}

int32_t all_reduce_max_f32(b200_decoder* d, float* buf, size_t n) {
    int rc = nccl().AllReduce(buf, buf, n, kNcclFloat32, kNcclMax, d->comm, d->ctx->stream);
    if (rc != 0) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, "ncclAllReduce (max) failed");
    return B200_OK;
}

int32_t all_reduce_sum_i32(b200_decoder* d, int* buf, size_t n) {
    int rc = nccl().AllReduce(buf, buf, n, kNcclInt32, kNcclSum, d->comm, d->ctx->stream);
    if (rc != 0) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, "ncclAllReduce (int32 sum) failed");
    return B200_OK;
}

int32_t all_reduce_sum_f32(b200_decoder* d, float* buf, size_t n) {
    int rc = nccl().AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, d->comm, d->ctx->stream);
    if (rc != 0) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, "ncclAllReduce failed");
    return B200_OK;
}

// Enqueues one decode step for the current batch on the context's stream.
int32_t enqueue_step(b200_decoder* d, bool eager = false) {
    const auto& c = d->cfg;
    cudaStream_t s = d->ctx->stream;
    uint32_t* err = d->ctx->err_dev;
    const int M = d->batch, dm = c.d_model, dh = c.head_dim;
    const bool tp = c.tp_size > 1;
    const int fp8 = c.act_fp8 ? 1 : 0;      // E4M3 activations and f32 accumulators instead of int8 / int32
    uint64_t launches = 0;
    GemmEpilogue ep;
    ep.raw = d->raw;
    // With the exchange blocks mapped, the int8 rows a GEMM reads after a row-parallel output were stored by the other
    // ranks' finish kernels: such a GEMM waits for their delivered flags (after it has put its weight tiles in flight).
    const bool exchange = tp && d->tp_exchange && M % c.tp_size == 0;
    GemmPeerWait delivered;
    if (exchange) {
        delivered.flags = reinterpret_cast<const uint32_t*>(d->tp_block) + 64;
        delivered.n = c.tp_size;
        delivered.epoch = d->tp_epoch;
        delivered.timeout_ns = 0;
    }
    // Bound of the cross-GPU waits of this step.  A step that is launched kernel by kernel (the first one of a decoder)
    // also waits for the other ranks' HOST work between their launches - first-use loading of every kernel - so it gets
    // a longer bound than the replayed graph.
    uint64_t wait_ns = d->tp_timeout_ns ? d->tp_timeout_ns : kCrossGpuWaitNs;
    if (eager && wait_ns < 10 * kCrossGpuWaitNs) wait_ns = 10 * kCrossGpuWaitNs;
    auto after_exchange = [&](GemmEpilogue e) {
        if (exchange) {
            e.wait = delivered;
            e.wait.timeout_ns = wait_ns;
        }
        return e;
    };
    CU_TRY(begin_step(d->seq_lens_dev, d->pos_dev, d->active_dev, M, s));
    ++launches;
    CU_TRY(embed_norm_quant_auto(d->ids_dev, d->embed, c.vocab, M, dm, d->vectors + d->layers[0].attn_norm, c.rms_eps, d->h,
                            d->xq, d->sx, err, s, fp8));
    ++launches;
    // A row-parallel projection and what follows it: residual add, RMSNorm with `norm`, per-token int8 rows in xq.
    // One rank: the row kernel reads the raw accumulators.  Several ranks: the GEMM writes its dequantised f32
    // partial into the exchange block; then either the finish kernel sums the partials over the ranks' blocks and
    // delivers the rows (peers mapped), or ncclAllReduce sums them and every rank finishes all rows itself.
    const bool exact_tp = tp && c.tp_exact_int8 != 0;
    // Exact integer sums: the A rows were quantised under the row maximum merged over all ranks (quant_global below),
    // so the ranks' int32 partials add up to the accumulators of one GPU; the dequantisation is the one-GPU kernel.
    auto row_parallel_exact = [&](const GemmPlan& p, size_t s_off, const float* norm) -> int32_t {
        CU_TRY(gemm_launch(p, ep, err, s));
        int* acc = d->raw;
        if (p.out_planes > 1) {
            CU_TRY(gemm_sum_planes_i32(d->raw, p.out_planes, int64_t(M) * dm, d->tp_acc, s));
            acc = d->tp_acc;
            ++launches;
        }
        if (int32_t st = all_reduce_sum_i32(d, acc, size_t(M) * dm)) return st;
        CU_TRY(resid_norm_quant_auto(acc, 1, M, dm, d->sx, d->scales + s_off, nullptr, norm, c.rms_eps, d->h, d->xq, d->sx, s, fp8));
        launches += 3;
        return B200_OK;
    };
    // rows [M, n] of this rank -> int8 under the maximum over the whole row (all ranks)
    auto quant_global = [&](const float* rows, int n) -> int32_t {
        if (int32_t st = all_reduce_max_f32(d, d->tp_amax, size_t(M))) return st;
        CU_TRY(quantize_rows_with_amax(rows, M, n, d->tp_amax, d->xq, d->sx, s));
        launches += 2;
        return B200_OK;
    };
    auto row_parallel = [&](const GemmPlan& p, size_t s_off, const float* norm) -> int32_t {
        if (exact_tp) return row_parallel_exact(p, s_off, norm);
        const bool fused_ok = p.persist || p.splits == 1 || p.cluster;
        if (!tp) {
            CU_TRY(gemm_launch(p, ep, err, s));
            CU_TRY(resid_norm_quant_auto(d->raw, p.out_planes, M, dm, d->sx, d->scales + s_off, nullptr, norm, c.rms_eps, d->h,
                                         d->xq, d->sx, s, fp8));
            launches += 2;
            return B200_OK;
        }
        // Peers mapped and the one-tile kernel with a fused epilogue: the GEMM stores every row straight into the block
        // of the rank that owns it and counts its tiles there, and the finish kernel reads local memory only.
        const bool push = exchange && d->tp_push && fused_ok && !p.persist;
        if (exchange && !push) d->tp_push_all = false;
        if (fused_ok) {
            GemmEpilogue pe;
            pe.fused = 1;
            pe.a_scale = d->sx;
            pe.a_per_row = 1;
            pe.b_scale = d->scales + s_off;
            pe.b_per_col = 1;
            pe.out = d->part;
            if (push) {
                pe.push.peers = d->tp_peers_dev;
                pe.push.o_part = d->tp_o_part;
                pe.push.o_count = kTpCountOffset;
                pe.push.tp = c.tp_size;
                pe.push.rank = c.tp_rank;
                pe.push.rows = M / c.tp_size;
                pe.push.arrived = d->tp_epoch + 3;
            }
            CU_TRY(gemm_launch(p, pe, err, s));
            ++launches;
        } else {
            if (fp8) return fail(B200_UNSUPPORTED, "decoder: this GEMM shape has no fused epilogue, which the FP8 form needs under tensor parallelism");
            CU_TRY(gemm_launch(p, ep, err, s));
            CU_TRY(dequant_planes(d->raw, p.out_planes, M, dm, d->sx, d->scales + s_off, d->part, s));
            launches += 2;
        }
        if (exchange) {
            CU_TRY(tp_finish(d->tp_peers_dev, d->tp_o_sx, d->tp_o_xq, d->tp_o_part, c.tp_size, c.tp_rank, M / c.tp_size, dm, norm,
                             c.rms_eps, d->h, d->tp_epoch, d->tp_epoch + 1, err, s, wait_ns, kTpCountOffset,
                             push ? 1u : 0u, d->tp_epoch + 2, fp8));
            ++launches;
            return B200_OK;
        }
        if (int32_t st = all_reduce_sum_f32(d, d->part, size_t(M) * dm)) return st;
        CU_TRY(resid_norm_quant_auto(d->raw, p.out_planes, M, dm, d->sx, d->scales + s_off, d->part, norm, c.rms_eps, d->h, d->xq,
                                     d->sx, s, fp8));
        launches += 2;
        return B200_OK;
    };
    for (int l = 0; l < c.n_layers; ++l) {
        LayerParams& L = d->layers[l];
        // QKV projection -> RoPE -> append to the paged cache
        if (L.rope_fused) {
            // dequant + RoPE + cache append inside the GEMM's split-K reduction (one tile = one head)
            GemmEpilogue qe;
            qe.fused = 1;
            qe.a_scale = d->sx;
            qe.a_per_row = 1;
            qe.b_scale = d->scales + L.s_qkv;
            qe.b_per_col = 1;
            qe.rope.enabled = 1;
            qe.rope.hq = d->hq_l;
            qe.rope.hkv = d->hkv_l;
            qe.rope.cos_t = d->cos_t;
            qe.rope.sin_t = d->sin_t;
            qe.rope.max_pos = c.max_seq_len;
            qe.rope.positions = d->pos_dev;
            qe.rope.active = d->active_dev;
            qe.rope.block_tables = d->tables_dev;
            qe.rope.max_blocks_per_seq = d->max_blocks_per_seq;
            qe.rope.block_size = c.block_size;
            qe.rope.num_blocks = c.num_blocks;
            qe.rope.q_out = d->q;
            qe.rope.k_pool = static_cast<uint16_t*>(L.k_pool);
            qe.rope.v_pool = static_cast<uint16_t*>(L.v_pool);
            CU_TRY(gemm_launch(L.p_qkv, l > 0 ? after_exchange(qe) : qe, err, s));
            launches -= 1;
        } else {
            CU_TRY(gemm_launch(L.p_qkv, l > 0 ? after_exchange(ep) : ep, err, s));
            CU_TRY(qkv_rope_append_auto(d->raw, L.p_qkv.out_planes, M, d->hq_l, d->hkv_l, dh, d->sx, d->scales + L.s_qkv,
                                        d->cos_t, d->sin_t, c.max_seq_len, d->pos_dev, d->active_dev, d->tables_dev, d->max_blocks_per_seq,
                                        c.block_size, c.num_blocks, d->q, static_cast<uint16_t*>(L.k_pool),
                                        static_cast<uint16_t*>(L.v_pool), err, s, 1, fp8));
        }
        // attention over the cache (this rank's KV heads), then per-token quantisation
        if (exact_tp) {
            CU_TRY(paged_attention_launch(L.attn, d->q, L.k_pool, L.v_pool, d->tables_dev, d->seq_lens_dev, d->attn_out,
                                          d->attn_scratch, d->ctx->attn_counter, d->ctx->sm_count, err, s));
            CU_TRY(rows_amax(d->attn_out, M, d->hq_l * dh, d->tp_amax, s));
            if (int32_t st = quant_global(d->attn_out, d->hq_l * dh)) return st;
            launches += 1 - (paged_attention_can_quantize(L.attn) ? 0 : 1);
        } else if (paged_attention_can_quantize(L.attn)) {
            CU_TRY(paged_attention_launch(L.attn, d->q, L.k_pool, L.v_pool, d->tables_dev, d->seq_lens_dev, nullptr,
                                          d->attn_scratch, d->ctx->attn_counter, d->ctx->sm_count, err, s, d->xq, d->sx, fp8));
        } else {
            CU_TRY(paged_attention_launch(L.attn, d->q, L.k_pool, L.v_pool, d->tables_dev, d->seq_lens_dev, d->attn_out,
                                          d->attn_scratch, d->ctx->attn_counter, d->ctx->sm_count, err, s));
            CU_TRY(quantize_rows_auto(d->attn_out, M, d->hq_l * dh, d->xq, d->sx, s, fp8));
        }
        // O projection (row-parallel) -> residual -> norm -> quant
        launches += paged_attention_can_quantize(L.attn) ? 4 : 5;
        if (int32_t st = row_parallel(L.p_o, L.s_o, d->vectors + L.mlp_norm)) return st;
        // gate / up (column-parallel) -> SiLU gate -> quant
        CU_TRY(gemm_launch(L.p_gu, after_exchange(ep), err, s));
        if (exact_tp) {
            CU_TRY(gate_rows_f32(d->raw, L.p_gu.out_planes, M, d->f_l, d->sx, d->scales + L.s_gu, d->tp_rows_f32, d->tp_amax, s));
            if (int32_t st = quant_global(d->tp_rows_f32, d->f_l)) return st;
        } else
        CU_TRY(gate_quant_auto(d->raw, L.p_gu.out_planes, M, d->f_l, d->sx, d->scales + L.s_gu, d->xq, d->sx, s, fp8));
        // down (row-parallel) -> residual -> next norm -> quant
        const float* next_norm = d->vectors + (l + 1 < c.n_layers ? d->layers[l + 1].attn_norm : d->final_norm);
        launches += 2;
        if (int32_t st = row_parallel(L.p_down, L.s_down, next_norm)) return st;
    }
    // lm_head with the dequant epilogue fused into the GEMM, then greedy argmax on the device
    GemmEpilogue lm;
    lm.fused = 1;
    lm.a_scale = d->sx;
    lm.a_per_row = 1;
    lm.b_scale = d->scales + d->s_lm;
    lm.b_per_col = 1;
    lm.out = d->logits;
    CU_TRY(gemm_launch(d->p_lm, after_exchange(lm), err, s));
    CU_TRY(argmax_rows_auto(d->logits, M, c.vocab, d->next_ids_dev, s));
    launches += 2;
    d->launches_per_step = launches;
    return B200_OK;
}

void free_step_state(b200_decoder* d) {
    drop_graph(d);
    d->planned = false;
}

}  // namespace

extern "C" {

int32_t b200_decoder_create(b200_ctx* ctx, const b200_decoder_config* cfg, b200_decoder** out) {
    if (!out) return fail(B200_INVALID_ARGUMENT, "decoder_create: out is null");
    *out = nullptr;
    if (int32_t st = check_ctx(ctx)) return st;
    if (!cfg) return fail(B200_INVALID_ARGUMENT, "decoder_create: config is null");
    if (int32_t st = check_config(*cfg)) return st;
    if (int32_t st = set_device(ctx)) return st;
    b200_decoder* d = new (std::nothrow) b200_decoder();
    if (!d) return fail(B200_DEVICE_ALLOCATION_FAILED, "decoder_create: host allocation failed");
    d->ctx = ctx;
    d->generation = ctx->generation;
    d->cfg = *cfg;
    const auto& c = d->cfg;
    const int tp = c.tp_size;
    d->hq_l = c.n_heads / tp;
    d->hkv_l = c.n_kv_heads / tp;
    d->f_l = c.d_ff / tp;
    d->n_qkv = (d->hq_l + 2 * d->hkv_l) * c.head_dim;
    const size_t dm = c.d_model, dh = c.head_dim;
    // ---- ParamStore layout: registration order = layer by layer, qkv, o, gate_up, down; then lm_head
    size_t pay = 0, sc = 0, vec = 0;
    d->layers.resize(c.n_layers);
    for (auto& L : d->layers) {
        L.wqkv = pay; pay += align_up(size_t(d->n_qkv) * dm, 256);
        L.wo = pay; pay += align_up(dm * d->hq_l * dh, 256);
        L.wgu = pay; pay += align_up(size_t(2) * d->f_l * dm, 256);
        L.wdown = pay; pay += align_up(dm * d->f_l, 256);
        L.s_qkv = sc; sc += align_up(d->n_qkv, 64);
        L.s_o = sc; sc += align_up(dm, 64);
        L.s_gu = sc; sc += align_up(size_t(2) * d->f_l, 64);
        L.s_down = sc; sc += align_up(dm, 64);
        L.attn_norm = vec; vec += align_up(dm, 64);
        L.mlp_norm = vec; vec += align_up(dm, 64);
    }
    d->w_lm = pay; pay += align_up(size_t(c.vocab) * dm, 256);
    d->s_lm = sc; sc += align_up(c.vocab, 64);
    d->final_norm = vec; vec += align_up(dm, 64);
    d->payload_bytes = pay; d->scales_elems = sc; d->vectors_elems = vec;
    const size_t M = c.max_batch;
    const size_t pool_elems = size_t(c.num_blocks) * c.block_size * d->hkv_l * dh;
    const size_t widest = std::max<size_t>(std::max<size_t>(dm, d->f_l), size_t(d->hq_l) * dh);
    cudaError_t e = cudaSuccess;
    auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    A(dmalloc(&d->payload, pay));
    A(dmalloc(&d->scales, sc));
    A(dmalloc(&d->vectors, vec));
    A(dmalloc(&d->embed, size_t(c.vocab) * dm));
    A(dmalloc(&d->cos_t, size_t(c.max_seq_len) * dh / 2));
    A(dmalloc(&d->sin_t, size_t(c.max_seq_len) * dh / 2));
    for (auto& L : d->layers) {
        A(cudaMalloc(&L.k_pool, pool_elems * 2));
        A(cudaMalloc(&L.v_pool, pool_elems * 2));
    }
    d->max_blocks_per_seq = (c.max_seq_len + c.block_size - 1) / c.block_size;
    A(dmalloc(&d->tables_dev, M * d->max_blocks_per_seq));
    A(dmalloc(&d->seq_lens_dev, M));
    A(dmalloc(&d->pos_dev, M));
    A(dmalloc(&d->active_dev, M));
    A(cudaMallocHost(reinterpret_cast<void**>(&d->active_pinned), M * sizeof(uint32_t)));
    A(dmalloc(&d->ids_dev, M));
    A(dmalloc(&d->next_ids_dev, M));
    A(dmalloc(&d->h, M * dm));
    if (tp > 1) {
        size_t off = kTpFlagBytes;                               // ready[tp] at +0, delivered[tp] at +256, count[tp] at +512
        d->tp_o_sx = off; off += align_up(M * sizeof(float), 256);
        d->tp_o_xq = off; off += align_up(M * widest, 256);
        d->tp_o_part = off; off += align_up(M * dm * sizeof(float), 256);
        d->tp_block_bytes = off;
        A(cudaMalloc(reinterpret_cast<void**>(&d->tp_block), off));
        if (e == cudaSuccess) e = cudaMemset(d->tp_block, 0, off);
        if (e == cudaSuccess) {
            d->sx = reinterpret_cast<float*>(d->tp_block + d->tp_o_sx);
            d->xq = reinterpret_cast<int8_t*>(d->tp_block + d->tp_o_xq);
            d->part = reinterpret_cast<float*>(d->tp_block + d->tp_o_part);
        }
        A(dmalloc(&d->tp_epoch, 4));
        if (e == cudaSuccess) e = cudaMemset(d->tp_epoch, 0, 4 * sizeof(uint32_t));
        if (const char* v = std::getenv("B200_TP_PUSH")) d->tp_push = v[0] != '0';     // 0: the pulled form, for measurements
        A(cudaMalloc(reinterpret_cast<void**>(&d->tp_peers_dev), 16 * sizeof(uint8_t*)));
    } else {
        A(dmalloc(&d->xq, M * widest));
        A(dmalloc(&d->sx, M));
        A(dmalloc(&d->part, M * dm));
    }
    if (tp > 1 && c.tp_exact_int8) {
        A(dmalloc(&d->tp_amax, M));
        A(dmalloc(&d->tp_rows_f32, M * std::max<size_t>(d->f_l, size_t(d->hq_l) * dh)));
        A(dmalloc(&d->tp_acc, M * dm));
    }
    A(dmalloc(&d->q, M * d->hq_l * dh));
    A(dmalloc(&d->attn_out, M * d->hq_l * dh));
    A(dmalloc(&d->logits, M * size_t(c.vocab)));
    A(cudaMallocHost(reinterpret_cast<void**>(&d->ids_pinned), M * sizeof(int)));
    A(cudaEventCreateWithFlags(&d->ids_copied, cudaEventDisableTiming));
    A(cudaMallocHost(reinterpret_cast<void**>(&d->next_pinned), M * sizeof(int)));
    if (e == cudaSuccess) e = cudaMemsetAsync(d->vectors, 0, vec * sizeof(float), ctx->stream);
    if (e != cudaSuccess) {
        std::string msg = std::string("decoder_create: allocation failed: ") + cudaGetErrorString(e);
        cudaGetLastError();
        b200_decoder_destroy(d);
        return fail(B200_DEVICE_ALLOCATION_FAILED, msg);
    }
    // rope table in f64 on the host: angle = pos * theta^(-2i/dh)
    {
        const size_t half = dh / 2;
        std::vector<float> ct(size_t(c.max_seq_len) * half), stv(ct.size());
        for (int p = 0; p < c.max_seq_len; ++p)
            for (size_t i = 0; i < half; ++i) {
                const double inv = std::pow(double(c.rope_theta), -2.0 * double(i) / double(dh));
                const double ang = double(p) * inv;
                ct[p * half + i] = float(std::cos(ang));
                stv[p * half + i] = float(std::sin(ang));
            }
        e = cudaMemcpyAsync(d->cos_t, ct.data(), ct.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d->sin_t, stv.data(), stv.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            b200_decoder_destroy(d);
            return fail_runtime(ctx, B200_TRANSFER_FAILED, std::string("decoder_create: ") + cudaGetErrorString(e));
        }
    }
    if (int32_t st = b200_block_table_create(uint64_t(c.num_blocks), uint64_t(c.block_size), &d->table)) {
        b200_decoder_destroy(d);
        return st;
    }
    *out = d;
    return B200_OK;
}

int32_t b200_decoder_destroy(b200_decoder* d) {
    if (!d) return B200_OK;
    cudaSetDevice(d->ctx->ordinal);
    cudaStreamSynchronize(d->ctx->stream);
    drop_graph(d);
    if (d->comm && nccl().ok) nccl().CommDestroy(d->comm);
    for (auto& L : d->layers) {
        cudaFree(L.k_pool);
        cudaFree(L.v_pool);
    }
    if (d->tp_block) {      // xq, sx and part are carved out of the exchange block
        for (int p = 0; p < d->cfg.tp_size && p < 16; ++p)
            if (p != d->cfg.tp_rank && d->tp_peer_ptrs[p]) cudaIpcCloseMemHandle(d->tp_peer_ptrs[p]);
        d->xq = nullptr;
        d->sx = nullptr;
        d->part = nullptr;
    }
    void* pf_ptrs[] = {d->pf.ids, d->pf.pos, d->pf.h, d->pf.xq, d->pf.sx, d->pf.raw, d->pf.q, d->pf.attn, d->pf.part, d->pf.attn_scratch};
    for (void* p : pf_ptrs) cudaFree(p);
    void* ptrs[] = {d->payload, d->scales, d->vectors, d->embed, d->cos_t, d->sin_t, d->tables_dev, d->seq_lens_dev, d->pos_dev,
                    d->ids_dev, d->next_ids_dev, d->h, d->xq, d->sx, d->raw, d->q, d->attn_out, d->part, d->logits,
                    d->attn_scratch, d->tp_block, d->tp_epoch, d->tp_peers_dev, d->active_dev, d->tp_amax, d->tp_rows_f32, d->tp_acc};
    for (void* p : ptrs) cudaFree(p);
    if (d->ids_pinned) cudaFreeHost(d->ids_pinned);
    if (d->active_pinned) cudaFreeHost(d->active_pinned);
    if (d->ids_copied) cudaEventDestroy(d->ids_copied);
    if (d->next_pinned) cudaFreeHost(d->next_pinned);
    b200_block_table_destroy(d->table);
    cudaGetLastError();
    delete d;
    return B200_OK;
}

int32_t b200_decoder_load_tensor(b200_decoder* d, int32_t which, int32_t layer, const float* host, int64_t rows, int64_t cols) {
    if (int32_t st = dec_check(d)) return st;
    if (!host) return fail(B200_INVALID_ARGUMENT, "decoder_load_tensor: host pointer is null");
    const auto& c = d->cfg;
    cudaStream_t s = d->ctx->stream;
    const size_t dm = c.d_model;
    if (which == B200_W_EMBED || which == B200_W_ATTN_NORM || which == B200_W_MLP_NORM || which == B200_W_FINAL_NORM) {
        float* dst = nullptr;
        int64_t want_rows = 1, want_cols = int64_t(dm);
        if (which == B200_W_EMBED) { dst = d->embed; want_rows = c.vocab; }
        else if (which == B200_W_FINAL_NORM) dst = d->vectors + d->final_norm;
        else {
            if (layer < 0 || layer >= c.n_layers) return fail(B200_INVALID_ARGUMENT, "decoder_load_tensor: layer out of range");
            dst = d->vectors + (which == B200_W_ATTN_NORM ? d->layers[layer].attn_norm : d->layers[layer].mlp_norm);
        }
        if (rows != want_rows || cols != want_cols) return fail(B200_SHAPE_MISMATCH, "decoder_load_tensor: shape differs from the config");
        CU_TRY(cudaMemcpyAsync(dst, host, size_t(rows) * cols * 4, cudaMemcpyHostToDevice, s));
        CU_TRY(cudaStreamSynchronize(s));
        return B200_OK;
    }
    TensorShape t;
    if (!tensor_shape(d, which, layer, &t)) return fail(B200_INVALID_ARGUMENT, "decoder_load_tensor: unknown tensor or layer");
    if (rows != t.rows || cols != t.cols) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "decoder_load_tensor: shape [%lld, %lld] differs from the expected [%lld, %lld]",
                      (long long)rows, (long long)cols, (long long)t.rows, (long long)t.cols);
        return fail(B200_SHAPE_MISMATCH, msg);
    }
    float* tmp = nullptr;
    CU_TRY(dmalloc(&tmp, size_t(rows) * cols));
    CU_TRY(cudaMemcpyAsync(tmp, host, size_t(rows) * cols * 4, cudaMemcpyHostToDevice, s));
    int32_t st = store_weight(d, tmp, rows, cols, t.row_ranges, t.c0, t.ccount, t.payload_off, t.scale_off);
    cudaFree(tmp);
    return st;
}

// The same for a matrix that is already quantised: int8 payload [rows, cols] with one f32 scale per row, as a weight
// file stores it (see b200_decoder_load_safetensors).  Nothing is re-quantised; the rank keeps its shard.
int32_t b200_decoder_load_tensor_i8(b200_decoder* d, int32_t which, int32_t layer, const int8_t* q_host, const float* scale_host,
                                    int64_t rows, int64_t cols) {
    if (int32_t st = dec_check(d)) return st;
    if (!q_host || !scale_host) return fail(B200_INVALID_ARGUMENT, "decoder_load_tensor_i8: host pointer is null");
    TensorShape t;
    if (!tensor_shape(d, which, layer, &t)) return fail(B200_INVALID_ARGUMENT, "decoder_load_tensor_i8: not a quantised matrix, or layer out of range");
    if (rows != t.rows || cols != t.cols) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "decoder_load_tensor_i8: shape [%lld, %lld] differs from the expected [%lld, %lld]",
                      (long long)rows, (long long)cols, (long long)t.rows, (long long)t.cols);
        return fail(B200_SHAPE_MISMATCH, msg);
    }
    cudaStream_t s = d->ctx->stream;
    int8_t* q_full = nullptr;
    float* s_full = nullptr;
    CU_TRY(dmalloc(&q_full, size_t(rows) * cols));
    CU_TRY(dmalloc(&s_full, size_t(rows)));
    CU_TRY(cudaMemcpyAsync(q_full, q_host, size_t(rows) * cols, cudaMemcpyHostToDevice, s));
    CU_TRY(cudaMemcpyAsync(s_full, scale_host, size_t(rows) * 4, cudaMemcpyHostToDevice, s));
    int32_t st = B200_OK;
    if (d->cfg.act_fp8) {
        // the FP8 form re-encodes an int8 payload: dequantise to f32, then E4M3 codes under new per-row scales
        float* w_full = nullptr;
        CU_TRY(dmalloc(&w_full, size_t(rows) * cols));
        cudaError_t e = dequantize_i8_per_row(q_full, s_full, rows, cols, w_full, s);
        st = e == cudaSuccess ? store_weight(d, w_full, rows, cols, t.row_ranges, t.c0, t.ccount, t.payload_off, t.scale_off)
                              : dec_fail(d, B200_KERNEL_LAUNCH_FAILED, cudaGetErrorString(e));
        cudaFree(w_full);
    } else {
        st = store_weight_q(d, q_full, s_full, cols, t.row_ranges, t.c0, t.ccount, t.payload_off, t.scale_off);
    }
    cudaFree(q_full);
    cudaFree(s_full);
    return st;
}

// Loads every tensor of the decoder from a safetensors buffer.  Names (no renaming, no transposition, as in the
// reference's loader): "embed.weight" F32 [vocab, d], "final_norm.weight" F32 [d], "layers.<l>.attn_norm.weight" and
// "layers.<l>.mlp_norm.weight" F32 [d], and for each matrix M in {"lm_head", "layers.<l>.wqkv", ".wo", ".wgu",
// ".wdown"} either "M.qweight" I8 [rows, cols] with "M.scale" F32 [rows], or "M.weight" F32 [rows, cols] (quantised on
// the device).  Every missing name is reported in one error; a tensor with another dtype or shape is an error, never
// skipped; tensors the decoder does not know are an error too.
int32_t b200_decoder_load_safetensors_bytes(b200_decoder* d, const uint8_t* bytes, size_t len) {
    if (int32_t st = dec_check(d)) return st;
    std::vector<StTensor> ts;
    std::string err;
    if (!safetensors_parse(bytes, len, &ts, &err)) return fail(B200_INVALID_ARGUMENT, err);
    std::map<std::string, const StTensor*> by_name;
    for (const StTensor& t : ts) by_name[t.name] = &t;
    const auto& c = d->cfg;
    struct Want { std::string name; int which; int layer; bool matrix; };
    std::vector<Want> wants;
    wants.push_back({"embed", B200_W_EMBED, 0, false});
    wants.push_back({"final_norm", B200_W_FINAL_NORM, 0, false});
    wants.push_back({"lm_head", B200_W_LM_HEAD, 0, true});
    for (int l = 0; l < c.n_layers; ++l) {
        const std::string pre = "layers." + std::to_string(l) + ".";
        wants.push_back({pre + "attn_norm", B200_W_ATTN_NORM, l, false});
        wants.push_back({pre + "wqkv", B200_W_QKV, l, true});
        wants.push_back({pre + "wo", B200_W_O, l, true});
        wants.push_back({pre + "mlp_norm", B200_W_MLP_NORM, l, false});
        wants.push_back({pre + "wgu", B200_W_GATE_UP, l, true});
        wants.push_back({pre + "wdown", B200_W_DOWN, l, true});
    }
    std::string missing;
    size_t used = 0;
    for (const Want& w : wants) {
        const bool has_f32 = by_name.count(w.name + ".weight") != 0;
        const bool has_q = w.matrix && by_name.count(w.name + ".qweight") != 0 && by_name.count(w.name + ".scale") != 0;
        if (!has_f32 && !has_q) missing += (missing.empty() ? "" : ", ") + w.name + (w.matrix ? ".qweight + .scale (or .weight)" : ".weight");
        used += has_q ? 2 : (has_f32 ? 1 : 0);
    }
    if (!missing.empty()) return fail(B200_INVALID_ARGUMENT, "load_safetensors: missing tensors: " + missing);
    if (used != ts.size()) {
        for (const StTensor& t : ts) {
            bool known = false;
            for (const Want& w : wants) {
                const bool q_form = w.matrix && by_name.count(w.name + ".qweight") != 0 && by_name.count(w.name + ".scale") != 0;
                if ((q_form && (t.name == w.name + ".qweight" || t.name == w.name + ".scale")) || (!q_form && t.name == w.name + ".weight"))
                    known = true;
            }
            if (!known) return fail(B200_INVALID_ARGUMENT, "load_safetensors: tensor " + t.name + " is not part of this decoder (or is given twice, as .weight and .qweight)");
        }
    }
    auto shape2 = [](const StTensor& t, int64_t* rows, int64_t* cols) {
        if (t.shape.size() == 1) { *rows = 1; *cols = int64_t(t.shape[0]); return true; }
        if (t.shape.size() == 2) { *rows = int64_t(t.shape[0]); *cols = int64_t(t.shape[1]); return true; }
        return false;
    };
    for (const Want& w : wants) {
        int64_t rows = 0, cols = 0;
        const bool q_form = w.matrix && by_name.count(w.name + ".qweight") != 0;
        if (q_form) {
            const StTensor& q = *by_name[w.name + ".qweight"];
            const StTensor& sc = *by_name[w.name + ".scale"];
            if (q.dtype != "I8") return fail(B200_UNSUPPORTED, "load_safetensors: " + q.name + " has dtype " + q.dtype + ", expected I8");
            if (sc.dtype != "F32") return fail(B200_UNSUPPORTED, "load_safetensors: " + sc.name + " has dtype " + sc.dtype + ", expected F32");
            if (!shape2(q, &rows, &cols) || q.shape.size() != 2) return fail(B200_SHAPE_MISMATCH, "load_safetensors: " + q.name + " must be a matrix");
            if (sc.shape.size() != 1 || int64_t(sc.shape[0]) != rows)
                return fail(B200_SHAPE_MISMATCH, "load_safetensors: " + sc.name + " must hold one scale per row of " + q.name);
            // the scales start on a 4-byte boundary inside the file only by luck: copy them to an aligned vector
            std::vector<float> scales(size_t(rows), 0.0f);
            std::memcpy(scales.data(), sc.data, size_t(rows) * 4);
            if (int32_t st = b200_decoder_load_tensor_i8(d, w.which, w.layer, reinterpret_cast<const int8_t*>(q.data), scales.data(), rows, cols))
                return st;
        } else {
            const StTensor& t = *by_name[w.name + ".weight"];
            if (t.dtype != "F32") return fail(B200_UNSUPPORTED, "load_safetensors: " + t.name + " has dtype " + t.dtype + ", expected F32");
            if (!shape2(t, &rows, &cols)) return fail(B200_SHAPE_MISMATCH, "load_safetensors: " + t.name + " must have one or two dimensions");
            std::vector<float> vals(size_t(rows) * cols);
            std::memcpy(vals.data(), t.data, vals.size() * 4);
            if (int32_t st = b200_decoder_load_tensor(d, w.which, w.layer, vals.data(), rows, cols)) return st;
        }
    }
    return B200_OK;
}

int32_t b200_decoder_load_safetensors(b200_decoder* d, const char* path) {
    if (int32_t st = dec_check(d)) return st;
    if (!path) return fail(B200_INVALID_ARGUMENT, "load_safetensors: path is null");
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(B200_INVALID_ARGUMENT, std::string("load_safetensors: cannot open ") + path);
    std::vector<uint8_t> bytes;
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    bool ok = n >= 0;
    if (ok) {
        bytes.resize(size_t(n));
        ok = n == 0 || std::fread(bytes.data(), 1, size_t(n), f) == size_t(n);
    }
    std::fclose(f);
    if (!ok) return fail(B200_TRANSFER_FAILED, std::string("load_safetensors: cannot read ") + path);
    return b200_decoder_load_safetensors_bytes(d, bytes.data(), bytes.size());
}

int32_t b200_decoder_init_random(b200_decoder* d, uint64_t seed, float std) {
    if (int32_t st = dec_check(d)) return st;
    const auto& c = d->cfg;
    cudaStream_t s = d->ctx->stream;
    const size_t dm = c.d_model;
    CU_TRY(fill_normal(d->embed, int64_t(c.vocab) * dm, seed, 1, std, s));
    {
        std::vector<float> ones(d->vectors_elems, 1.0f);
        CU_TRY(cudaMemcpyAsync(d->vectors, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice, s));
        CU_TRY(cudaStreamSynchronize(s));
    }
    size_t max_elems = size_t(c.vocab) * dm;
    max_elems = std::max(max_elems, size_t(2) * c.d_ff * dm);
    max_elems = std::max(max_elems, size_t(c.n_heads + 2 * c.n_kv_heads) * c.head_dim * dm);
    float* tmp = nullptr;
    CU_TRY(dmalloc(&tmp, max_elems));
    int32_t st = B200_OK;
    const int kinds[4] = {B200_W_QKV, B200_W_O, B200_W_GATE_UP, B200_W_DOWN};
    for (int l = 0; l < c.n_layers && st == B200_OK; ++l)
        for (int k = 0; k < 4 && st == B200_OK; ++k) {
            TensorShape t;
            tensor_shape(d, kinds[k], l, &t);
            cudaError_t e = fill_normal(tmp, t.rows * t.cols, seed, 16 + uint64_t(l) * 8 + k, std, s);
            if (e != cudaSuccess) { st = dec_fail(d, B200_KERNEL_LAUNCH_FAILED, cudaGetErrorString(e)); break; }
            st = store_weight(d, tmp, t.rows, t.cols, t.row_ranges, t.c0, t.ccount, t.payload_off, t.scale_off);
        }
    if (st == B200_OK) {
        TensorShape t;
        tensor_shape(d, B200_W_LM_HEAD, 0, &t);
        cudaError_t e = fill_normal(tmp, t.rows * t.cols, seed, 2, std, s);
        if (e != cudaSuccess) st = dec_fail(d, B200_KERNEL_LAUNCH_FAILED, cudaGetErrorString(e));
        else st = store_weight(d, tmp, t.rows, t.cols, t.row_ranges, t.c0, t.ccount, t.payload_off, t.scale_off);
    }
    cudaStreamSynchronize(s);
    cudaFree(tmp);
    return st;
}

int32_t b200_nccl_unique_id(uint8_t* out128) {
    if (!out128) return fail(B200_INVALID_ARGUMENT, "nccl_unique_id: out is null");
    if (!nccl().ok) return fail(B200_UNSUPPORTED, "nccl_unique_id: libnccl.so.2 could not be loaded");
    NcclUniqueId id;
    if (nccl().GetUniqueId(&id) != 0) return fail(B200_DEVICE_UNAVAILABLE, "ncclGetUniqueId failed");
    std::memcpy(out128, id.internal, 128);
    return B200_OK;
}

int32_t b200_decoder_init_tp(b200_decoder* d, const uint8_t* unique_id128) {
    if (int32_t st = dec_check(d)) return st;
    if (d->cfg.tp_size == 1) return B200_OK;
    if (!unique_id128) return fail(B200_INVALID_ARGUMENT, "decoder_init_tp: unique id is null");
    if (!nccl().ok) return fail(B200_UNSUPPORTED, "decoder_init_tp: libnccl.so.2 could not be loaded");
    NcclUniqueId id;
    std::memcpy(id.internal, unique_id128, 128);
    int rc = nccl().CommInitRank(&d->comm, d->cfg.tp_size, id, d->cfg.tp_rank);
    if (rc != 0) return fail(B200_DEVICE_UNAVAILABLE, "ncclCommInitRank failed");
    map_peer_blocks(d);
    return B200_OK;
}

int32_t b200_decoder_tp_exchange(const b200_decoder* d) {
    if (!d || !d->tp_exchange) return 0;
    return d->tp_push && d->tp_push_all ? 2 : 1;
}

// Failure-detection self-test of the cross-GPU finish kernel on one GPU: launches it as rank 0 of 2 over a scratch
// exchange block in which nobody ever raises rank 1's flags.  The kernel's bounded wait (20 ms here) runs out, it
// records kErrPeerWait in the context's error word, skips its loads and stores, writes the poison value into the
// flags it owns at its peer (so that the peer would stop with an error of its own) and returns; the next
// synchronisation reports the failure and poisons the context, and the device stays usable.
int32_t b200_selftest_peer_wait(b200_ctx* ctx) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = set_device(ctx)) return st;
    const int d = 512, rows = 2, tp = 2;
    const size_t o_sx = 512, o_xq = 1024, o_part = 1024 + 4096;
    const size_t bytes = o_part + size_t(tp) * rows * d * sizeof(float);
    uint8_t* block = nullptr;        // rank 0's block
    uint8_t* peer_block = nullptr;   // "rank 1": a block whose owner never runs
    uint8_t** peers = nullptr;
    float* h = nullptr;
    float* w = nullptr;
    uint32_t* counters = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&block), bytes);
    if (e == cudaSuccess) e = cudaMemset(block, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&peer_block), bytes);
    if (e == cudaSuccess) e = cudaMemset(peer_block, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&peers), tp * sizeof(uint8_t*));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h), size_t(tp) * rows * d * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(h, 0, size_t(tp) * rows * d * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&w), d * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(w, 0, d * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&counters), 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(counters, 0, 2 * sizeof(uint32_t));
    uint8_t* host_peers[2] = {block, peer_block};
    if (e == cudaSuccess) e = cudaMemcpy(peers, host_peers, sizeof(host_peers), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = tp_finish(peers, o_sx, o_xq, o_part, tp, 0, rows, d, w, 1e-5f, h, counters, counters + 1, ctx->err_dev, ctx->stream,
                      20ull * 1000 * 1000);
    uint32_t peer_flags[128] = {};
    if (e == cudaSuccess) e = cudaMemcpyAsync(peer_flags, peer_block, sizeof(peer_flags), cudaMemcpyDeviceToHost, ctx->stream);
    int32_t st = B200_OK;
    if (e != cudaSuccess) st = fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("selftest_peer_wait: ") + cudaGetErrorString(e));
    else st = b200_synchronize(ctx);              // reports the device error word
    cudaFree(block);
    cudaFree(peer_block);
    cudaFree(peers);
    cudaFree(h);
    cudaFree(w);
    cudaFree(counters);
    if (st == B200_KERNEL_LAUNCH_FAILED && (peer_flags[0] != 0xFFFFFFFFu || peer_flags[64] != 0xFFFFFFFFu))
        return fail(B200_INVALID_ARGUMENT, "selftest_peer_wait: the wait ran out but the peer's flags were not poisoned");
    return st;
}

// Numerical self-test of the finish kernel on one GPU, with nothing to wait for: `tp` exchange blocks live on this
// device, every rank's partial [tp * rows, d] is uploaded into its block and all ready flags are raised by the host
// beforehand; the kernel then runs as rank `rank`.  Returns, for the rows that rank owns, the updated residual rows,
// the int8 rows and scales as delivered into EVERY block ([tp][rows][d] and [tp][rows]), and the flags words of every
// block ([tp][128]) so that the caller can check the delivered epoch.
int32_t b200_selftest_tp_finish(b200_ctx* ctx, int32_t tp, int32_t rank, int32_t rows, int32_t d, const float* partials,
                                const float* residual, const float* norm_w, float eps, float* h_out, int8_t* xq_out,
                                float* sx_out, uint32_t* flags_out) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (tp < 1 || tp > 16 || rank < 0 || rank >= tp || rows <= 0 || d <= 0 || !partials || !residual || !norm_w || !h_out ||
        !xq_out || !sx_out || !flags_out)
        return fail(B200_INVALID_ARGUMENT, "selftest_tp_finish: bad argument");
    if (!tp_finish_supported(d)) return fail(B200_UNSUPPORTED, "selftest_tp_finish: row width not supported by the finish kernel");
    if (int32_t st = set_device(ctx)) return st;
    const size_t M = size_t(tp) * rows;
    const size_t o_sx = 512;
    const size_t o_xq = o_sx + (M * 4 + 255) / 256 * 256;
    const size_t o_part = o_xq + (M * d + 255) / 256 * 256;
    const size_t bytes = o_part + M * d * sizeof(float);
    std::vector<uint8_t*> blocks(tp, nullptr);
    uint8_t** peers = nullptr;
    float* h = nullptr;
    float* w = nullptr;
    uint32_t* counters = nullptr;
    cudaStream_t s = ctx->stream;
    cudaError_t e = cudaSuccess;
    std::vector<uint32_t> ready(128, 0u);
    for (int p = 0; p < tp; ++p) ready[p] = 1u;          // epoch 1: every partial is complete
    for (int p = 0; p < tp && e == cudaSuccess; ++p) {
        e = cudaMalloc(reinterpret_cast<void**>(&blocks[p]), bytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(blocks[p], 0, bytes, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(blocks[p], ready.data(), 512, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(blocks[p] + o_part, partials + size_t(p) * M * d, M * d * sizeof(float), cudaMemcpyHostToDevice, s);
    }
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&peers), tp * sizeof(uint8_t*));
    if (e == cudaSuccess) e = cudaMemcpyAsync(peers, blocks.data(), tp * sizeof(uint8_t*), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h), M * d * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpyAsync(h, residual, M * d * sizeof(float), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&w), d * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpyAsync(w, norm_w, d * sizeof(float), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&counters), 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemsetAsync(counters, 0, 2 * sizeof(uint32_t), s);
    if (e == cudaSuccess)
        e = tp_finish(peers, o_sx, o_xq, o_part, tp, rank, rows, d, w, eps, h, counters, counters + 1, ctx->err_dev, s,
                      50ull * 1000 * 1000);
    const size_t row0 = size_t(rank) * rows;
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, h + row0 * d, size_t(rows) * d * sizeof(float), cudaMemcpyDeviceToHost, s);
    for (int p = 0; p < tp && e == cudaSuccess; ++p) {
        e = cudaMemcpyAsync(xq_out + size_t(p) * rows * d, blocks[p] + o_xq + row0 * d, size_t(rows) * d, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(sx_out + size_t(p) * rows, blocks[p] + o_sx + row0 * 4, size_t(rows) * 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(flags_out + size_t(p) * 128, blocks[p], 512, cudaMemcpyDeviceToHost, s);
    }
    int32_t st = B200_OK;
    if (e != cudaSuccess) st = fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("selftest_tp_finish: ") + cudaGetErrorString(e));
    else st = b200_synchronize(ctx);
    for (uint8_t* b : blocks) cudaFree(b);
    cudaFree(peers);
    cudaFree(h);
    cudaFree(w);
    cudaFree(counters);
    return st;
}

// Numerical self-test on one GPU of a row-parallel GEMM that scatters its rows (GemmPush) followed by the scattered
// form of the finish kernel, with nothing to wait for: `tp` exchange blocks live on this device.  For every rank s the
// GEMM [M = tp * rows, d] = a_q[s] [M, k] x w_q[s] [d, k]^T with the dequantising epilogue is launched as rank s
// (splits / tile as in b200_set_tuning, 0 = heuristic); all ranks' GEMMs have completed when the finish kernel then
// runs as rank 0, 1, ... .  Returns the residual rows [M, d], the int8 rows and scales as delivered into the first and
// into the last block ([2][M][d], [2][M]) and the launch counts of every block ([tp][tp]: one per rank's GEMM).
int32_t b200_selftest_tp_scatter(b200_ctx* ctx, int32_t tp, int32_t rows, int32_t d, int32_t k, int32_t splits, int32_t tile,
                                 const int8_t* a_q, const float* a_scale, const int8_t* w_q, const float* w_scale,
                                 const float* residual, const float* norm_w, float eps, float* h_out, int8_t* xq_out,
                                 float* sx_out, uint32_t* counts_out) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (tp < 1 || tp > 16 || rows <= 0 || d <= 0 || k <= 0 || !a_q || !a_scale || !w_q || !w_scale || !residual || !norm_w ||
        !h_out || !xq_out || !sx_out || !counts_out)
        return fail(B200_INVALID_ARGUMENT, "selftest_tp_scatter: bad argument");
    if (!tp_finish_supported(d)) return fail(B200_UNSUPPORTED, "selftest_tp_scatter: row width not supported by the finish kernel");
    if (int32_t st = set_device(ctx)) return st;
    const size_t M = size_t(tp) * rows;
    const size_t o_sx = kTpFlagBytes;
    const size_t o_xq = o_sx + (M * 4 + 255) / 256 * 256;
    const size_t o_part = o_xq + (M * d + 255) / 256 * 256;
    const size_t bytes = o_part + M * d * sizeof(float);
    std::vector<uint8_t*> blocks(tp, nullptr);
    std::vector<void*> owned;
    cudaStream_t s = ctx->stream;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](size_t n) -> void* {
        void* p = nullptr;
        if (e == cudaSuccess) e = cudaMalloc(&p, n);
        if (p) owned.push_back(p);
        return p;
    };
    for (int p = 0; p < tp; ++p) {
        blocks[p] = static_cast<uint8_t*>(alloc(bytes));
        if (e == cudaSuccess) e = cudaMemsetAsync(blocks[p], 0, bytes, s);
    }
    uint8_t** peers = static_cast<uint8_t**>(alloc(tp * sizeof(uint8_t*)));
    float* h = static_cast<float*>(alloc(M * d * sizeof(float)));
    float* w = static_cast<float*>(alloc(d * sizeof(float)));
    uint32_t* counters = static_cast<uint32_t*>(alloc((size_t(tp) * 4 + 1) * sizeof(uint32_t)));
    int8_t* aq = static_cast<int8_t*>(alloc(size_t(tp) * M * k));
    int8_t* wq = static_cast<int8_t*>(alloc(size_t(tp) * d * k));
    float* as = static_cast<float*>(alloc(size_t(tp) * M * sizeof(float)));
    float* ws = static_cast<float*>(alloc(size_t(tp) * d * sizeof(float)));
    if (e == cudaSuccess) e = cudaMemcpyAsync(peers, blocks.data(), tp * sizeof(uint8_t*), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h, residual, M * d * sizeof(float), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w, norm_w, d * sizeof(float), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(counters, 0, (size_t(tp) * 4 + 1) * sizeof(uint32_t), s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(aq, a_q, size_t(tp) * M * k, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(wq, w_q, size_t(tp) * d * k, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(as, a_scale, size_t(tp) * M * sizeof(float), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ws, w_scale, size_t(tp) * d * sizeof(float), cudaMemcpyHostToDevice, s);
    const char* why = "";
    for (int r = 0; r < tp && e == cudaSuccess; ++r) {
        GemmPlan plan;
        e = gemm_make_plan(&plan, kGemmI8, aq + size_t(r) * M * k, wq + size_t(r) * d * k, int(M), d, k, 0, splits, tile, &why);
        if (e != cudaSuccess) break;
        if (!(plan.splits == 1 || plan.cluster)) {
            for (void* p : owned) cudaFree(p);
            return fail(B200_UNSUPPORTED, "selftest_tp_scatter: the plan has no fused epilogue");
        }
        GemmEpilogue pe;
        pe.fused = 1;
        pe.a_scale = as + size_t(r) * M;
        pe.a_per_row = 1;
        pe.b_scale = ws + size_t(r) * d;
        pe.b_per_col = 1;
        pe.out = h;                      // never written: every row goes to its owner's block
        pe.push.peers = peers;
        pe.push.o_part = o_part;
        pe.push.o_count = kTpCountOffset;
        pe.push.tp = tp;
        pe.push.rank = r;
        pe.push.rows = rows;
        pe.push.arrived = counters + 4 * tp;
        e = gemm_launch(plan, pe, ctx->err_dev, s);
    }
    for (int r = 0; r < tp && e == cudaSuccess; ++r)
        e = tp_finish(peers, o_sx, o_xq, o_part, tp, r, rows, d, w, eps, h, counters + 4 * r, counters + 4 * r + 1, ctx->err_dev, s,
                      50ull * 1000 * 1000, kTpCountOffset, 1u, counters + 4 * r + 2);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, h, M * d * sizeof(float), cudaMemcpyDeviceToHost, s);
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
        const uint8_t* b = blocks[i == 0 ? 0 : tp - 1];
        e = cudaMemcpyAsync(xq_out + size_t(i) * M * d, b + o_xq, M * d, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(sx_out + size_t(i) * M, b + o_sx, M * 4, cudaMemcpyDeviceToHost, s);
    }
    for (int p = 0; p < tp && e == cudaSuccess; ++p)
        e = cudaMemcpyAsync(counts_out + size_t(p) * tp, blocks[p] + kTpCountOffset, size_t(tp) * 4, cudaMemcpyDeviceToHost, s);
    int32_t st = B200_OK;
    if (e != cudaSuccess) st = fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("selftest_tp_scatter: ") + why + " " + cudaGetErrorString(e));
    else st = b200_synchronize(ctx);
    for (void* p : owned) cudaFree(p);
    return st;
}

// Starts a generation: clears the page table, reserves blocks for `max_total_len[b]` tokens per row
// (the reference's generate() always runs to max_length, so the final length is known up front), uploads
// the flattened tables once, and sets seq_lens to `start_lens` (0 for a fresh cache).
int32_t b200_decoder_begin(b200_decoder* d, int32_t batch, const int32_t* start_lens, const int32_t* max_total_lens) {
    if (int32_t st = dec_check(d)) return st;
    const auto& c = d->cfg;
    if (batch <= 0 || batch > c.max_batch) return fail(B200_INVALID_ARGUMENT, "decoder_begin: batch out of range");
    if (!max_total_lens) return fail(B200_INVALID_ARGUMENT, "decoder_begin: max_total_lens is null");
    int mx = 0;
    for (int b = 0; b < batch; ++b) {
        const int s0 = start_lens ? start_lens[b] : 0;
        if (s0 < 0 || max_total_lens[b] < s0 || max_total_lens[b] > c.max_seq_len || max_total_lens[b] <= 0)
            return fail(B200_INVALID_ARGUMENT, "decoder_begin: lengths out of range for row " + std::to_string(b));
        mx = std::max(mx, max_total_lens[b]);
    }
    free_step_state(d);
    b200_block_table* t = d->table;
    t->reset();
    t->tables.assign(batch, {});
    t->seq_lens.assign(batch, 0);
    t->has_batch = true;
    d->row_limits.assign(batch, 0);
    for (int b = 0; b < batch; ++b) {
        if (!bt_reserve_row(t, b, uint64_t(max_total_lens[b]))) {
            t->reset();
            return fail(B200_INVALID_ARGUMENT, "decoder_begin: not enough free blocks in the pool");
        }
        t->seq_lens[b] = start_lens ? start_lens[b] : 0;
        d->row_limits[b] = max_total_lens[b];
    }
    std::vector<uint32_t> flat(size_t(batch) * d->max_blocks_per_seq), lens(batch);
    if (int32_t st = b200_block_table_flatten(t, d->max_blocks_per_seq, flat.data(), flat.size())) return st;
    for (int b = 0; b < batch; ++b) lens[b] = uint32_t(t->seq_lens[b]);
    cudaStream_t s = d->ctx->stream;
    CU_TRY(cudaMemcpyAsync(d->tables_dev, flat.data(), flat.size() * 4, cudaMemcpyHostToDevice, s));
    CU_TRY(cudaMemcpyAsync(d->seq_lens_dev, lens.data(), lens.size() * 4, cudaMemcpyHostToDevice, s));
    for (int b = 0; b < batch; ++b) d->active_pinned[b] = 1u;
    d->active_host.assign(batch, 1);
    CU_TRY(cudaMemcpyAsync(d->active_dev, d->active_pinned, size_t(batch) * 4, cudaMemcpyHostToDevice, s));
    CU_TRY(cudaStreamSynchronize(s));
    d->batch = batch;
    d->max_total_len = mx;
    // ---- plans for this batch size
    const int M = batch, dm = c.d_model, dh = c.head_dim;
    const char* why = "";
    size_t raw_need = 0;
    // `fused`: the launch will use a fused epilogue (the row-parallel projections under tensor parallelism write
    // their dequantised partial), which moves the switch to the persistent kernel down to half a wave of tiles
    const int kind = c.act_fp8 ? kGemmFp8 : kGemmI8;
    auto plan = [&](GemmPlan* p, size_t w_off, int N, int K, bool fused = false) -> cudaError_t {
        cudaError_t e = gemm_make_plan(p, kind, d->xq, d->payload + w_off, M, N, K, 0, d->ctx->tune_splits, d->ctx->tune_bn, &why);
        if (e == cudaSuccess && d->ctx->tune_splits == 0) gemm_plan_make_persistent(p, d->ctx->sm_count, fused);
        if (e == cudaSuccess) raw_need = std::max(raw_need, gemm_raw_elems(*p));
        return e;
    };
    PagedAttnShape sh{M, 1, d->hq_l, d->hkv_l, dh, c.block_size, c.num_blocks, d->max_blocks_per_seq, 1.0f / std::sqrt(float(dh))};
    if (!paged_attention_fast_path(sh, 1) && dh > 256) return fail(B200_UNSUPPORTED, "decoder_begin: head_dim above 256");
    size_t attn_need = 0;
    for (auto& L : d->layers) {
        cudaError_t e = plan(&L.p_qkv, L.wqkv, d->n_qkv, dm);
        L.rope_fused = e == cudaSuccess && dh == 128 && gemm_plan_can_rope(L.p_qkv, d->hq_l, d->hkv_l);
        const bool partial_f32 = c.tp_size > 1 && !c.tp_exact_int8;     // the row-parallel GEMMs write dequantised partials
        if (e == cudaSuccess) e = plan(&L.p_o, L.wo, dm, d->hq_l * dh, partial_f32);
        if (e == cudaSuccess) e = plan(&L.p_gu, L.wgu, 2 * d->f_l, dm);
        if (e == cudaSuccess) e = plan(&L.p_down, L.wdown, dm, d->f_l, partial_f32);
        if (e != cudaSuccess) return fail(B200_UNSUPPORTED, std::string("decoder_begin: ") + why);
        e = paged_attention_make_plan(&L.attn, sh, 1, L.k_pool, L.v_pool, mx, d->ctx->tune_attn_chunk_blocks);
        if (e != cudaSuccess) return fail(B200_KERNEL_LAUNCH_FAILED, "decoder_begin: attention plan failed");
        attn_need = std::max(attn_need, paged_attention_scratch_bytes(L.attn));
    }
    {
        cudaError_t e = gemm_make_plan(&d->p_lm, kind, d->xq, d->payload + d->w_lm, M, c.vocab, dm, 0, 1, d->ctx->tune_bn, &why);
        if (e != cudaSuccess) return fail(B200_UNSUPPORTED, std::string("decoder_begin: ") + why);
        if (d->ctx->tune_splits == 0) gemm_plan_make_persistent(&d->p_lm, d->ctx->sm_count, true);
    }
    if (raw_need > d->raw_elems) {
        cudaFree(d->raw);
        d->raw = nullptr;
        CU_TRY(dmalloc(&d->raw, raw_need));
        d->raw_elems = raw_need;
    }
    cudaFree(d->attn_scratch);
    d->attn_scratch = nullptr;
    CU_TRY(cudaMalloc(&d->attn_scratch, attn_need > 0 ? attn_need : 16));
    d->planned = true;
    d->steps = 0;
    if (c.tp_size > 1 && d->comm) {
        // every rank has loaded its weights and uploaded its tables before any rank's first step starts to wait for
        // the others inside a kernel (host skew of seconds between the ranks must not look like a dead peer)
        int* flag = nullptr;
        CU_TRY(dmalloc(&flag, 1));
        cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int), s);
        int rc = e == cudaSuccess ? nccl().AllReduce(flag, flag, 1, kNcclInt32, kNcclSum, d->comm, s) : 1;
        if (rc == 0) e = cudaStreamSynchronize(s);
        cudaFree(flag);
        if (rc != 0 || e != cudaSuccess) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, "decoder_begin: barrier across the ranks failed");
    }
    return B200_OK;
}

// Fills this rank's KV pools with synthetic bf16 N(0, std^2) values (benchmark set-up: stands in for a
// prefill whose results the timed decode steps only read).
int32_t b200_decoder_fill_cache_random(b200_decoder* d, uint64_t seed, float std) {
    if (int32_t st = dec_check(d)) return st;
    const auto& c = d->cfg;
    const int64_t pool_elems = int64_t(c.num_blocks) * c.block_size * d->hkv_l * c.head_dim;
    for (int l = 0; l < c.n_layers; ++l) {
        CU_TRY(fill_normal_bf16(static_cast<uint16_t*>(d->layers[l].k_pool), pool_elems, seed, 1000 + 2 * l, std, d->ctx->stream));
        CU_TRY(fill_normal_bf16(static_cast<uint16_t*>(d->layers[l].v_pool), pool_elems, seed, 1001 + 2 * l, std, d->ctx->stream));
    }
    return B200_OK;
}

// One decode step for every row of the batch.  ids_host != NULL: the step's input ids are copied from
// the host (pinned staging) first; otherwise the ids produced by the previous step are used in place.
// next_ids_host != NULL: the sampled ids are copied back and the call returns when they are final.
int32_t b200_decoder_step(b200_decoder* d, const int32_t* ids_host, int32_t* next_ids_host) {
    return b200_decoder_step_rows(d, ids_host, nullptr, next_ids_host);
}

// One step in which only the rows with active[b] != 0 advance (NULL: all rows).  The other rows run through the
// same kernels on their last position (see begin_step_kernel) and keep their length; their sampled ids mean nothing.
int32_t b200_decoder_step_rows(b200_decoder* d, const int32_t* ids_host, const uint8_t* active, int32_t* next_ids_host) {
    if (int32_t st = dec_check(d)) return st;
    if (!d->planned) return fail(B200_INVALID_ARGUMENT, "decoder_step: call decoder_begin first");
    cudaStream_t s = d->ctx->stream;
    const int M = d->batch;
    auto is_active = [&](int b) { return !active || active[b] != 0; };
    for (int b = 0; b < M; ++b)
        if (is_active(b) && d->table->seq_lens[b] + 1 > uint64_t(d->row_limits[b]))
            return fail(B200_INVALID_ARGUMENT, "decoder_step: row " + std::to_string(b) + " is past its reserved length");
    bool mask_changed = false;
    for (int b = 0; b < M; ++b)
        if ((d->active_host[b] != 0) != is_active(b)) mask_changed = true;
    if (mask_changed) {
        // the previous copy out of the staging buffer has finished: every step that follows a mask change waits below
        CU_TRY(cudaStreamSynchronize(s));
        for (int b = 0; b < M; ++b) {
            d->active_host[b] = is_active(b) ? 1 : 0;
            d->active_pinned[b] = d->active_host[b];
        }
        CU_TRY(cudaMemcpyAsync(d->active_dev, d->active_pinned, size_t(M) * 4, cudaMemcpyHostToDevice, s));
    }
    if (ids_host) {
        // the staging buffer is read when the copy executes, not when it is enqueued
        if (d->ids_copy_pending) CU_TRY(cudaEventSynchronize(d->ids_copied));
        std::memcpy(d->ids_pinned, ids_host, size_t(M) * sizeof(int));
        CU_TRY(cudaMemcpyAsync(d->ids_dev, d->ids_pinned, size_t(M) * sizeof(int), cudaMemcpyHostToDevice, s));
        CU_TRY(cudaEventRecord(d->ids_copied, s));
        d->ids_copy_pending = true;
    } else if (d->steps > 0) {
        CU_TRY(cudaMemcpyAsync(d->ids_dev, d->next_ids_dev, size_t(M) * sizeof(int), cudaMemcpyDeviceToDevice, s));
    }
    if (d->graph) {
        CU_TRY(cudaGraphLaunch(d->graph, s));
    } else if (d->eager_steps_done < 1 || d->cfg.use_graph == 0) {
        // the first step runs eagerly (it also sets the kernels' shared-memory attributes)
        if (int32_t st = enqueue_step(d, true)) return st;
        d->eager_steps_done++;
    } else {
        cudaGraph_t g = nullptr;
        CaptureGuard capturing(d->ctx);     // other threads get DeviceContextCaptureInProgress until the capture ends
        CU_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        int32_t st = enqueue_step(d);
        cudaError_t e = cudaStreamEndCapture(s, &g);
        if (st != B200_OK) {
            if (g) cudaGraphDestroy(g);
            return st;
        }
        if (e != cudaSuccess) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, std::string("graph capture: ") + cudaGetErrorString(e));
        e = cudaGraphInstantiate(&d->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return dec_fail(d, B200_KERNEL_LAUNCH_FAILED, std::string("graph instantiate: ") + cudaGetErrorString(e));
        CU_TRY(cudaGraphLaunch(d->graph, s));
    }
    for (int b = 0; b < M; ++b) {      // commit the logical state after the enqueue succeeded
        if (is_active(b)) d->table->seq_lens[b] += 1;
        else if (d->table->seq_lens[b] == 0) d->table->seq_lens[b] = 1;
    }
    d->steps++;
    if (next_ids_host) {
        CU_TRY(cudaMemcpyAsync(d->next_pinned, d->next_ids_dev, size_t(M) * sizeof(int), cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaStreamSynchronize(s));
        std::memcpy(next_ids_host, d->next_pinned, size_t(M) * sizeof(int));
        if (int32_t st = b200_synchronize(d->ctx)) {
            d->store_poisoned = true;
            return st;
        }
    }
    return B200_OK;
}

// Multi-token prefill: the rows [row0, row0 + count) each consume l_new tokens (ids [count, l_new], host) in one pass
// over M = count * l_new token rows - the GEMMs run at M rows, every token's K / V is appended, attention uses the
// reference's mask j <= seq_len - l_new + i (crates/backend-cpu/src/paged_kv.rs:137-140) - and the rows' lengths grow
// by l_new.  Nothing is sampled: a caller that wants the next token feeds the last prompt token through
// b200_decoder_step.  Prompts longer than the workspace are consumed in chunks, which the mask rule allows (a chunk
// is "l_new tokens on top of a non-empty cache").
namespace {

constexpr int kPrefillRowsCap = 2048;      // token rows per pass

int32_t prefill_pass(b200_decoder* d, int row0, int count, int l_new, const int32_t* ids_host) {
    const auto& c = d->cfg;
    const int fp8 = c.act_fp8 ? 1 : 0;
    cudaStream_t s = d->ctx->stream;
    uint32_t* err = d->ctx->err_dev;
    const int M = count * l_new, dm = c.d_model, dh = c.head_dim;
    const bool tp = c.tp_size > 1;
    auto& pf = d->pf;
    const size_t widest = std::max<size_t>(std::max<size_t>(dm, d->f_l), size_t(d->hq_l) * dh);
    if (pf.rows < size_t(M)) {
        void* old[] = {pf.ids, pf.pos, pf.h, pf.xq, pf.sx, pf.q, pf.attn, pf.part};
        CU_TRY(cudaStreamSynchronize(s));
        for (void* p : old) cudaFree(p);
        pf = b200_decoder::Prefill{};
        const size_t R = size_t(M);
        CU_TRY(dmalloc(&pf.ids, R));
        CU_TRY(dmalloc(&pf.pos, R));
        CU_TRY(dmalloc(&pf.h, R * dm));
        CU_TRY(dmalloc(&pf.xq, R * widest));
        CU_TRY(dmalloc(&pf.sx, R));
        CU_TRY(dmalloc(&pf.q, R * d->hq_l * dh));
        CU_TRY(dmalloc(&pf.attn, R * d->hq_l * dh));
        if (tp) CU_TRY(dmalloc(&pf.part, R * dm));
        pf.rows = R;
    }
    // plans for M rows (raw accumulators everywhere: the row kernels sum the planes and apply the scales)
    const char* why = "";
    GemmPlan p_qkv, p_o, p_gu, p_down;
    size_t raw_need = 0;
    auto plan = [&](GemmPlan* p, const int8_t* w, int N, int K, bool fused) -> cudaError_t {
        cudaError_t e = gemm_make_plan(p, c.act_fp8 ? kGemmFp8 : kGemmI8, pf.xq, w, M, N, K, 0, 0, 0, &why);
        if (e == cudaSuccess) gemm_plan_make_persistent(p, d->ctx->sm_count, fused);
        if (e == cudaSuccess && !(fused && (p->persist || p->splits == 1 || p->cluster))) raw_need = std::max(raw_need, gemm_raw_elems(*p));
        return e;
    };
    PagedAttnShape sh{count, l_new, d->hq_l, d->hkv_l, dh, c.block_size, c.num_blocks, d->max_blocks_per_seq, 1.0f / std::sqrt(float(dh))};
    CU_TRY(cudaMemcpyAsync(pf.ids, ids_host, size_t(M) * sizeof(int), cudaMemcpyHostToDevice, s));
    const uint32_t* tables = d->tables_dev + size_t(row0) * d->max_blocks_per_seq;
    uint32_t* lens = d->seq_lens_dev + row0;
    CU_TRY(prefill_positions(lens, pf.pos, count, l_new, s));
    CU_TRY(prefill_advance(lens, count, l_new, s));
    CU_TRY(embed_norm_quant_auto(pf.ids, d->embed, c.vocab, M, dm, d->vectors + d->layers[0].attn_norm, c.rms_eps, pf.h, pf.xq, pf.sx, err, s, fp8));
    for (int l = 0; l < c.n_layers; ++l) {
        LayerParams& L = d->layers[l];
        raw_need = 0;
        cudaError_t e = plan(&p_qkv, d->payload + L.wqkv, d->n_qkv, dm, false);
        if (e == cudaSuccess) e = plan(&p_o, d->payload + L.wo, dm, d->hq_l * dh, tp);
        if (e == cudaSuccess) e = plan(&p_gu, d->payload + L.wgu, 2 * d->f_l, dm, false);
        if (e == cudaSuccess) e = plan(&p_down, d->payload + L.wdown, dm, d->f_l, tp);
        if (e != cudaSuccess) return fail(B200_UNSUPPORTED, std::string("decoder_prefill: ") + why);
        if (raw_need > pf.raw_elems) {
            CU_TRY(cudaStreamSynchronize(s));
            cudaFree(pf.raw);
            pf.raw = nullptr;
            CU_TRY(dmalloc(&pf.raw, raw_need));
            pf.raw_elems = raw_need;
        }
        PagedAttnPlan ap;
        if (paged_attention_make_plan(&ap, sh, 1, L.k_pool, L.v_pool, d->max_total_len, d->ctx->tune_attn_chunk_blocks) != cudaSuccess)
            return fail(B200_KERNEL_LAUNCH_FAILED, "decoder_prefill: attention plan failed");
        const size_t need = paged_attention_scratch_bytes(ap);
        if (need > pf.attn_scratch_bytes) {
            CU_TRY(cudaStreamSynchronize(s));
            cudaFree(pf.attn_scratch);
            pf.attn_scratch = nullptr;
            CU_TRY(cudaMalloc(&pf.attn_scratch, need));
            pf.attn_scratch_bytes = need;
        }
        GemmEpilogue ep;
        ep.raw = pf.raw;
        CU_TRY(gemm_launch(p_qkv, ep, err, s));
        CU_TRY(qkv_rope_append_auto(pf.raw, p_qkv.out_planes, M, d->hq_l, d->hkv_l, dh, pf.sx, d->scales + L.s_qkv, d->cos_t, d->sin_t,
                                    c.max_seq_len, pf.pos, nullptr, tables, d->max_blocks_per_seq, c.block_size, c.num_blocks, pf.q,
                                    static_cast<uint16_t*>(L.k_pool), static_cast<uint16_t*>(L.v_pool), err, s, l_new, fp8));
        // nothing is sampled from a prefill pass: once the last layer's K / V rows are in the cache the pass is complete
        if (l + 1 == c.n_layers) break;
        CU_TRY(paged_attention_launch(ap, pf.q, L.k_pool, L.v_pool, tables, lens, pf.attn, pf.attn_scratch, d->ctx->attn_counter,
                                      d->ctx->sm_count, err, s));
        CU_TRY(quantize_rows_auto(pf.attn, M, d->hq_l * dh, pf.xq, pf.sx, s, fp8));
        auto row_parallel = [&](const GemmPlan& p, size_t s_off, const float* norm) -> int32_t {
            if (!tp) {
                CU_TRY(gemm_launch(p, ep, err, s));
                CU_TRY(resid_norm_quant_auto(pf.raw, p.out_planes, M, dm, pf.sx, d->scales + s_off, nullptr, norm, c.rms_eps, pf.h, pf.xq, pf.sx, s, fp8));
                return B200_OK;
            }
            if (p.persist || p.splits == 1 || p.cluster) {
                GemmEpilogue pe;
                pe.fused = 1;
                pe.a_scale = pf.sx;
                pe.a_per_row = 1;
                pe.b_scale = d->scales + s_off;
                pe.b_per_col = 1;
                pe.out = pf.part;
                CU_TRY(gemm_launch(p, pe, err, s));
            } else {
                if (fp8) return fail(B200_UNSUPPORTED, "decoder_prefill: this GEMM shape has no fused epilogue, which the FP8 form needs under tensor parallelism");
                CU_TRY(gemm_launch(p, ep, err, s));
                CU_TRY(dequant_planes(pf.raw, p.out_planes, M, dm, pf.sx, d->scales + s_off, pf.part, s));
            }
            if (int32_t st = all_reduce_sum_f32(d, pf.part, size_t(M) * dm)) return st;
            CU_TRY(resid_norm_quant_auto(pf.raw, 1, M, dm, pf.sx, d->scales + s_off, pf.part, norm, c.rms_eps, pf.h, pf.xq, pf.sx, s, fp8));
            return B200_OK;
        };
        if (int32_t st = row_parallel(p_o, L.s_o, d->vectors + L.mlp_norm)) return st;
        CU_TRY(gemm_launch(p_gu, ep, err, s));
        CU_TRY(gate_quant_auto(pf.raw, p_gu.out_planes, M, d->f_l, pf.sx, d->scales + L.s_gu, pf.xq, pf.sx, s, fp8));
        if (int32_t st = row_parallel(p_down, L.s_down, d->vectors + d->layers[l + 1].attn_norm)) return st;
    }
    return B200_OK;
}

}  // namespace

int32_t b200_decoder_prefill(b200_decoder* d, int32_t row0, int32_t count, const int32_t* ids, int32_t l_new) {
    if (int32_t st = dec_check(d)) return st;
    if (!d->planned) return fail(B200_INVALID_ARGUMENT, "decoder_prefill: call decoder_begin first");
    if (row0 < 0 || count <= 0 || row0 + count > d->batch) return fail(B200_INVALID_ARGUMENT, "decoder_prefill: rows out of range");
    if (l_new <= 0 || !ids) return fail(B200_INVALID_ARGUMENT, "decoder_prefill: need l_new > 0 and ids");
    if (d->cfg.tp_size > 1 && d->cfg.tp_exact_int8)
        return fail(B200_UNSUPPORTED, "decoder_prefill: multi-token passes are not implemented for tp_exact_int8; feed the prompt through decoder_step");
    for (int b = row0; b < row0 + count; ++b)
        if (d->table->seq_lens[b] + uint64_t(l_new) > uint64_t(d->row_limits[b]))
            return fail(B200_INVALID_ARGUMENT, "decoder_prefill: row " + std::to_string(b) + " would pass its reserved length");
    for (int64_t i = 0; i < int64_t(count) * l_new; ++i)
        if (ids[i] < 0 || ids[i] >= d->cfg.vocab) return fail(B200_INVALID_ARGUMENT, "decoder_prefill: token id outside the vocabulary");
    int chunk = kPrefillRowsCap / count;
    if (chunk < 1) chunk = 1;
    std::vector<int32_t> part;
    for (int t0 = 0; t0 < l_new; t0 += chunk) {
        const int n = std::min(chunk, l_new - t0);
        part.resize(size_t(count) * n);
        for (int b = 0; b < count; ++b)
            for (int i = 0; i < n; ++i) part[size_t(b) * n + i] = ids[size_t(b) * l_new + t0 + i];
        if (int32_t st = prefill_pass(d, row0, count, n, part.data())) return st;
        CU_TRY(cudaStreamSynchronize(d->ctx->stream));      // `part` is reused by the next chunk
        for (int b = row0; b < row0 + count; ++b) d->table->seq_lens[b] += uint64_t(n);
    }
    return B200_OK;
}

// Empties row `row` between steps and reserves blocks for a new sequence of up to max_total_len tokens in it: the
// row's blocks go back to the free stack (last block first), new ones are taken, the row's slice of the device
// block table and its length (0) are uploaded.  The other rows are untouched.  Continuous batching uses this to
// put a new request into a finished request's slot.
int32_t b200_decoder_row_restart(b200_decoder* d, int32_t row, int32_t max_total_len) {
    if (int32_t st = dec_check(d)) return st;
    if (!d->planned) return fail(B200_INVALID_ARGUMENT, "decoder_row_restart: call decoder_begin first");
    if (row < 0 || row >= d->batch) return fail(B200_INVALID_ARGUMENT, "decoder_row_restart: row out of range");
    if (max_total_len <= 0 || max_total_len > d->max_total_len)
        return fail(B200_INVALID_ARGUMENT, "decoder_row_restart: length exceeds what decoder_begin planned for");
    b200_block_table* t = d->table;
    std::vector<uint32_t> old = t->tables[row];
    for (auto it = t->tables[row].rbegin(); it != t->tables[row].rend(); ++it) t->returned.push_back(*it);
    t->tables[row].clear();
    if (!bt_reserve_row(t, row, uint64_t(max_total_len))) {
        // cannot happen when the new length fits the blocks just returned plus the free ones; restore otherwise
        for (size_t i = 0; i < t->tables[row].size(); ++i) t->returned.push_back(t->tables[row][i]);
        t->tables[row].clear();
        for (size_t i = 0; i < old.size(); ++i) t->returned.pop_back();
        t->tables[row] = old;
        return fail(B200_INVALID_ARGUMENT, "decoder_row_restart: not enough free blocks in the pool");
    }
    t->seq_lens[row] = 0;
    d->row_limits[row] = max_total_len;
    std::vector<uint32_t> slice(size_t(d->max_blocks_per_seq), 0xFFFFFFFFu);
    for (size_t i = 0; i < t->tables[row].size(); ++i) slice[i] = t->tables[row][i];
    const uint32_t zero = 0;
    cudaStream_t s = d->ctx->stream;
    CU_TRY(cudaMemcpyAsync(d->tables_dev + size_t(row) * d->max_blocks_per_seq, slice.data(), slice.size() * 4,
                           cudaMemcpyHostToDevice, s));
    CU_TRY(cudaMemcpyAsync(d->seq_lens_dev + row, &zero, 4, cudaMemcpyHostToDevice, s));
    CU_TRY(cudaStreamSynchronize(s));      // the host vectors above go out of scope
    return B200_OK;
}

// Copies the logits [batch, vocab] of the last step to the host (synchronises).
int32_t b200_decoder_logits(b200_decoder* d, float* host, uint64_t capacity_elems) {
    if (int32_t st = dec_check(d)) return st;
    const size_t n = size_t(d->batch) * d->cfg.vocab;
    if (!host || capacity_elems < n) return fail(B200_INVALID_ARGUMENT, "decoder_logits: host buffer too small");
    CU_TRY(cudaMemcpyAsync(host, d->logits, n * 4, cudaMemcpyDeviceToHost, d->ctx->stream));
    return b200_synchronize(d->ctx);
}

// generate() of the reference (crates/autodiff/src/generate/mod.rs:500-613) with greedy sampling: prefill once -
// all but the last prompt token in multi-token passes, the last one through the decode step that samples the first
// new token - then the model's own tokens are fed back until max_length; out is [batch, max_length] (prompt included).
// There is no end-of-sequence stop, as in the reference.
int32_t b200_decoder_generate(b200_decoder* d, const int32_t* prompt, int32_t batch, int32_t prompt_len, int32_t max_length,
                              int32_t* out) {
    if (int32_t st = dec_check(d)) return st;
    if (!prompt || !out) return fail(B200_INVALID_ARGUMENT, "decoder_generate: null pointer");
    if (prompt_len <= 0 || max_length <= prompt_len) return fail(B200_INVALID_ARGUMENT, "decoder_generate: need 0 < prompt_len < max_length");
    for (int64_t i = 0; i < int64_t(batch) * prompt_len; ++i)
        if (prompt[i] < 0 || prompt[i] >= d->cfg.vocab) return fail(B200_INVALID_ARGUMENT, "decoder_generate: token id outside the vocabulary");
    std::vector<int32_t> lens(batch, max_length - 1);   // the last generated token is never fed back
    if (int32_t st = b200_decoder_begin(d, batch, nullptr, lens.data())) return st;
    std::vector<int32_t> ids(batch), next(batch);
    for (int b = 0; b < batch; ++b)
        for (int t = 0; t < prompt_len; ++t) out[size_t(b) * max_length + t] = prompt[size_t(b) * prompt_len + t];
    // prefill once (all but the last prompt token in multi-token passes), then one forward per token
    int first = 0;
    if (prompt_len > 1 && !(d->cfg.tp_size > 1 && d->cfg.tp_exact_int8)) {
        std::vector<int32_t> head(size_t(batch) * (prompt_len - 1));
        for (int b = 0; b < batch; ++b)
            for (int t = 0; t < prompt_len - 1; ++t) head[size_t(b) * (prompt_len - 1) + t] = prompt[size_t(b) * prompt_len + t];
        if (int32_t st = b200_decoder_prefill(d, 0, batch, head.data(), prompt_len - 1)) return st;
        first = prompt_len - 1;
    }
    for (int t = first; t < max_length - 1; ++t) {
        const bool in_prompt = t < prompt_len;
        if (in_prompt)
            for (int b = 0; b < batch; ++b) ids[b] = prompt[size_t(b) * prompt_len + t];
        const bool need_out = t >= prompt_len - 1;
        if (int32_t st = b200_decoder_step(d, in_prompt ? ids.data() : nullptr, need_out ? next.data() : nullptr)) return st;
        if (need_out)
            for (int b = 0; b < batch; ++b) out[size_t(b) * max_length + t + 1] = next[b];
    }
    return B200_OK;
}

// Tensor-parallel shard of one weight matrix, without a device: validates the configuration and reports
// the full shape, up to three kept row ranges (start, count pairs) and the kept column range.
int32_t b200_decoder_shard_plan(const b200_decoder_config* cfg, int32_t which, int64_t* rows, int64_t* cols,
                                int64_t* row_ranges6, int32_t* n_ranges, int64_t* col_start, int64_t* col_count) {
    if (!cfg || !rows || !cols || !row_ranges6 || !n_ranges || !col_start || !col_count)
        return fail(B200_INVALID_ARGUMENT, "decoder_shard_plan: null pointer");
    if (int32_t st = check_config(*cfg)) return st;
    TensorShape t;
    if (!shard_of(*cfg, which, &t)) return fail(B200_INVALID_ARGUMENT, "decoder_shard_plan: not a sharded matrix");
    *rows = t.rows;
    *cols = t.cols;
    *n_ranges = int32_t(t.row_ranges.size());
    for (size_t i = 0; i < t.row_ranges.size() && i < 3; ++i) {
        row_ranges6[2 * i] = t.row_ranges[i].first;
        row_ranges6[2 * i + 1] = t.row_ranges[i].second;
    }
    *col_start = t.c0;
    *col_count = t.ccount;
    return B200_OK;
}

int32_t b200_decoder_vocab(const b200_decoder* d) { return d ? d->cfg.vocab : 0; }
int32_t b200_decoder_batch(const b200_decoder* d) { return d ? d->batch : 0; }
uint64_t b200_decoder_launches_per_step(const b200_decoder* d) { return d ? d->launches_per_step : 0; }
uint64_t b200_decoder_weight_bytes(const b200_decoder* d) { return d ? d->payload_bytes : 0; }

// Plan summary for benchmarks: tile width and split count of the four per-layer GEMMs and the split
// size of the attention kernel.  out[0..9] = {qkv.bn, qkv.splits, o.bn, o.splits, gu.bn, gu.splits,
// down.bn, down.splits, attn.chunk_blocks, attn.max_chunks}.
int32_t b200_decoder_plan_info(const b200_decoder* d, int32_t* out10) {
    if (!d || !out10 || !d->planned) return fail(B200_INVALID_ARGUMENT, "decoder_plan_info: no plan");
    const LayerParams& L = d->layers[0];
    const int v[10] = {L.p_qkv.bn, L.p_qkv.splits, L.p_o.bn, L.p_o.splits, L.p_gu.bn, L.p_gu.splits,
                       L.p_down.bn, L.p_down.splits, L.attn.chunk_blocks, L.attn.max_chunks};
    for (int i = 0; i < 10; ++i) out10[i] = v[i];
    return B200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------ measurement aids
extern "C" {

// CUDA-event stopwatch on the context's stream (device time of the work enqueued between the two
// calls).  The reference's bench harness waits for completion without a transfer
// (crates/bench-harness/src/lib.rs, module doc); this is the same wait made with events.
int32_t b200_timer_start(b200_ctx* ctx) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = set_device(ctx)) return st;
    if (!ctx->ev_start) {
        cudaError_t e = cudaEventCreate(&ctx->ev_start);
        if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_stop);
        if (e != cudaSuccess) return fail(B200_KERNEL_LAUNCH_FAILED, std::string("timer: ") + cudaGetErrorString(e));
    }
    cudaError_t e = cudaEventRecord(ctx->ev_start, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("timer: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_timer_stop(b200_ctx* ctx, float* elapsed_ms) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (!ctx->ev_start || !elapsed_ms) return fail(B200_INVALID_ARGUMENT, "timer_stop: timer not started");
    cudaError_t e = cudaEventRecord(ctx->ev_stop, ctx->stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(ctx->ev_stop);
    if (e == cudaSuccess) e = cudaEventElapsedTime(elapsed_ms, ctx->ev_start, ctx->ev_stop);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("timer: ") + cudaGetErrorString(e));
    return b200_synchronize(ctx);
}

// Times the decode-attention launch (split kernel + combine) alone on the decoder's current caches:
// `iters` launches cycling over the layers, so consecutive launches read different pools (each far
// larger than L2).  Reports the mean device time per launch and the algorithmic bytes of one launch:
// K and V rows of every cached token of this rank's KV heads, q and out rows, and the used table entries.
int32_t b200_decoder_time_attention(b200_decoder* d, int32_t iters, float* ms_per_launch, uint64_t* bytes_per_launch) {
    if (int32_t st = dec_check(d)) return st;
    if (!d->planned || iters <= 0 || !ms_per_launch) return fail(B200_INVALID_ARGUMENT, "decoder_time_attention: no plan or bad arguments");
    cudaStream_t s = d->ctx->stream;
    const auto& c = d->cfg;
    uint64_t bytes = 0;
    for (int b = 0; b < d->batch; ++b) {
        const uint64_t n = d->table->seq_lens[b];
        bytes += n * uint64_t(d->hkv_l) * c.head_dim * 2 * 2;
        bytes += (n + c.block_size - 1) / c.block_size * 4;
    }
    bytes += uint64_t(d->batch) * d->hq_l * c.head_dim * 4 * 2;
    if (bytes_per_launch) *bytes_per_launch = bytes;
    auto run = [&](int l) {
        LayerParams& L = d->layers[l % c.n_layers];
        return paged_attention_launch(L.attn, d->q, L.k_pool, L.v_pool, d->tables_dev, d->seq_lens_dev, d->attn_out,
                                      d->attn_scratch, d->ctx->attn_counter, d->ctx->sm_count, d->ctx->err_dev, s);
    };
    for (int w = 0; w < 3; ++w) CU_TRY(run(w));
    if (int32_t st = b200_timer_start(d->ctx)) return st;
    for (int i = 0; i < iters; ++i) CU_TRY(run(i + 3));
    float ms = 0.0f;
    if (int32_t st = b200_timer_stop(d->ctx, &ms)) return st;
    *ms_per_launch = ms / float(iters);
    return B200_OK;
}

}  // extern "C"
