// C-ABI implementation, part 2: paged KV cache.  The validators restate
// validate_paged_kv_append / validate_paged_attention of the reference
// (crates/tensor-core/src/paged_kv.rs:220-267, 276-373) with two extensions: the pool
// element type (bf16 or f32) and a separate count of KV heads (grouped-query attention).
// They are pure host functions and run before the first driver call.
#include <algorithm>
#include <cmath>
#include <vector>

#include "backend.h"
#include "kernels.cuh"

using namespace b200;

namespace {

constexpr uint64_t kMaxBlockSize = 256;                 // PAGED_KV_MAX_BLOCK_SIZE
constexpr uint64_t kMaxWorkspaceElems = 1ull << 30;     // PAGED_ATTENTION_MAX_WORKSPACE_ELEMS
constexpr uint64_t kI32Max = 0x7FFFFFFFull;
constexpr uint64_t kU32Max = 0xFFFFFFFFull;
constexpr uint64_t kIsizeMax = 0x7FFFFFFFFFFFFFFFull;

bool cmul(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_mul_overflow(a, b, out); }

int32_t invalid(const std::string& msg) { return fail(B200_INVALID_ARGUMENT, "paged_kv: " + msg); }

size_t elem_size(int32_t dtype) { return dtype == B200_BF16 ? 2 : 4; }

// PagedKvLayout::recheck (paged_kv.rs:77-107)
int32_t layout_recheck(const b200_paged_kv_layout* l) {
    if (!l) return invalid("layout is null");
    if (l->dtype != B200_BF16 && l->dtype != B200_F32) return invalid("pool dtype must be BF16 or F32");
    const uint64_t bs = l->block_size;
    if (bs == 0 || bs > kMaxBlockSize || (bs & (bs - 1)) != 0)
        return invalid("block_size must be a power of two in 1..256 (got " + std::to_string(bs) + ")");
    if (l->num_blocks == 0 || l->num_blocks >= kU32Max)
        return invalid("num_blocks must be in 1..u32::MAX-1 (got " + std::to_string(l->num_blocks) + ")");
    if (l->embed_dim == 0 || l->embed_dim > kI32Max)
        return invalid("embed_dim must be in 1..i32::MAX (got " + std::to_string(l->embed_dim) + ")");
    uint64_t elems, bytes;
    if (!cmul(l->num_blocks, bs, &elems) || !cmul(elems, l->embed_dim, &elems))
        return invalid("pool element count overflows");
    if (!cmul(elems, elem_size(l->dtype), &bytes) || !cmul(bytes, 2, &bytes)) return invalid("pool byte count overflows");
    if (bytes > kIsizeMax) return invalid("pool byte count exceeds isize::MAX");
    return B200_OK;
}
uint64_t pool_elems(const b200_paged_kv_layout* l) { return l->num_blocks * l->block_size * l->embed_dim; }
uint64_t pool_rows(const b200_paged_kv_layout* l) { return l->num_blocks * l->block_size; }

// PagedAttentionArgs::recheck (paged_kv.rs:170-190) + the KV-head extension
int32_t args_recheck(const b200_paged_attention_args* a) {
    if (!a) return invalid("args is null");
    if (int32_t st = layout_recheck(&a->layout)) return st;
    if (a->batch > kI32Max) return invalid("batch exceeds i32::MAX");
    if (a->l_new > kI32Max) return invalid("l_new exceeds i32::MAX");
    if (a->max_blocks_per_seq > kI32Max) return invalid("max_blocks_per_seq exceeds i32::MAX");
    if (a->num_kv_heads == 0 || a->layout.embed_dim % a->num_kv_heads != 0)
        return invalid("num_kv_heads must be >= 1 and divide embed_dim");
    if (a->num_heads == 0 || a->num_heads % a->num_kv_heads != 0 || a->num_heads > kI32Max)
        return invalid("num_heads must be >= 1 and a multiple of num_kv_heads");
    if (!std::isfinite(a->scale)) return invalid("scale must be finite");
    return B200_OK;
}
uint64_t head_dim(const b200_paged_attention_args* a) { return a->layout.embed_dim / a->num_kv_heads; }

int32_t validate_append(uint64_t k_new_numel, uint64_t v_new_numel, uint64_t k_pool_numel, uint64_t v_pool_numel,
                        const uint32_t* slots, uint64_t n_slots, const b200_paged_kv_layout* layout, uint64_t* rows_out) {
    if (int32_t st = layout_recheck(layout)) return st;
    if (n_slots > 0 && !slots) return invalid("slot_mapping is null");
    uint64_t expect;
    if (!cmul(n_slots, layout->embed_dim, &expect)) return invalid("append element count overflows");
    if (k_new_numel != expect || v_new_numel != expect)
        return invalid("k_new / v_new element count differs from slot_mapping.len() * E (k=" + std::to_string(k_new_numel) +
                       ", v=" + std::to_string(v_new_numel) + ", expected " + std::to_string(expect) + ")");
    if (n_slots > kI32Max) return invalid("append row count exceeds i32::MAX");
    const uint64_t pool = pool_elems(layout);
    if (k_pool_numel != pool || v_pool_numel != pool)
        return invalid("pool element count differs from the layout (k=" + std::to_string(k_pool_numel) + ", v=" +
                       std::to_string(v_pool_numel) + ", expected " + std::to_string(pool) + ")");
    const uint64_t rows = pool_rows(layout);
    std::vector<uint32_t> sorted;
    try {
        sorted.assign(slots, slots + n_slots);
    } catch (...) {
        return invalid("allocation of the slot check buffer failed");
    }
    for (uint32_t s : sorted)
        if (uint64_t(s) >= rows) return invalid("slot " + std::to_string(s) + " is >= pool rows " + std::to_string(rows));
    std::sort(sorted.begin(), sorted.end());
    if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end()) return invalid("slot_mapping holds a duplicate slot");
    if (rows_out) *rows_out = n_slots;
    return B200_OK;
}

int32_t validate_attention(uint64_t q_numel, uint64_t k_pool_numel, uint64_t v_pool_numel, const uint32_t* tables,
                           uint64_t n_tables, const uint32_t* seq_lens, uint64_t n_seq,
                           const b200_paged_attention_args* a, b200_paged_attention_plan* plan) {
    if (int32_t st = args_recheck(a)) return st;
    const b200_paged_kv_layout* l = &a->layout;
    const uint64_t eq = a->num_heads * head_dim(a);
    uint64_t out_numel;
    if (!cmul(a->batch, a->l_new, &out_numel) || !cmul(out_numel, eq, &out_numel)) return invalid("output element count overflows");
    if (q_numel != out_numel)
        return invalid("q element count differs from B * L_new * E_q (got " + std::to_string(q_numel) + ", expected " +
                       std::to_string(out_numel) + ")");
    const uint64_t pool = pool_elems(l);
    if (k_pool_numel != pool || v_pool_numel != pool) return invalid("pool element count differs from the layout");
    uint64_t tables_len;
    if (!cmul(a->batch, a->max_blocks_per_seq, &tables_len)) return invalid("block_tables element count overflows");
    if (n_tables != tables_len)
        return invalid("block_tables.len() differs from B * max_blocks_per_seq (got " + std::to_string(n_tables) +
                       ", expected " + std::to_string(tables_len) + ")");
    if (n_seq != a->batch) return invalid("seq_lens.len() differs from B");
    if ((n_tables > 0 && !tables) || (n_seq > 0 && !seq_lens)) return invalid("block_tables / seq_lens is null");
    uint64_t max_seq;
    if (!cmul(a->max_blocks_per_seq, l->block_size, &max_seq)) return invalid("max_blocks_per_seq * block_size overflows");
    uint64_t s_max = 0;
    for (uint64_t b = 0; b < a->batch; ++b) {
        const uint64_t sl = seq_lens[b];
        if (sl < a->l_new || sl > max_seq)
            return invalid("row " + std::to_string(b) + ": seq_len " + std::to_string(sl) + " out of range (L_new=" +
                           std::to_string(a->l_new) + ", limit=" + std::to_string(max_seq) + ")");
        s_max = std::max(s_max, sl);
        const uint64_t used = (sl + l->block_size - 1) / l->block_size;
        const uint32_t* row = tables + b * a->max_blocks_per_seq;
        for (uint64_t slot = 0; slot < used; ++slot)
            if (uint64_t(row[slot]) >= l->num_blocks)
                return invalid("row " + std::to_string(b) + " slot " + std::to_string(slot) + ": block id " +
                               std::to_string(row[slot]) + " is >= num_blocks (the sentinel included)");
    }
    uint64_t query_rows;
    if (!cmul(a->batch, a->num_heads, &query_rows) || !cmul(query_rows, a->l_new, &query_rows))
        return invalid("query row count overflows");
    if (query_rows > kI32Max) return invalid("query rows B * H * L_new exceed i32::MAX");
    if (s_max > kI32Max) return invalid("sequence length exceeds i32::MAX");
    uint64_t ws;
    if (!cmul(query_rows, s_max, &ws)) return invalid("workspace element count overflows");
    if (ws > kMaxWorkspaceElems)
        return invalid("workspace of " + std::to_string(ws) + " elements exceeds the limit " + std::to_string(kMaxWorkspaceElems));
    if (plan) {
        plan->out_numel = out_numel;
        plan->s_max = s_max;
        plan->query_rows = query_rows;
        plan->workspace_elems = ws;
    }
    return B200_OK;
}

int32_t shape_from_args(const b200_paged_attention_args* a, PagedAttnShape* sh) {
    if (a->layout.num_blocks > kI32Max) return fail(B200_UNSUPPORTED, "paged_attention: num_blocks above i32::MAX is not supported");
    if (head_dim(a) > 256) return fail(B200_UNSUPPORTED, "paged_attention: head_dim above 256 is not supported");
    sh->batch = int(a->batch);
    sh->l_new = int(a->l_new);
    sh->num_q_heads = int(a->num_heads);
    sh->num_kv_heads = int(a->num_kv_heads);
    sh->head_dim = int(head_dim(a));
    sh->block_size = int(a->layout.block_size);
    sh->num_blocks = int(a->layout.num_blocks);
    sh->max_blocks_per_seq = int(a->max_blocks_per_seq);
    sh->scale = a->scale;
    return B200_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int32_t run_attention(b200_ctx* ctx, const PagedAttnShape& sh, int kv_bf16, const float* q, const void* k_pool,
                      const void* v_pool, const uint32_t* tables_host, const uint32_t* seq_host,
                      const uint32_t* tables_dev, const uint32_t* seq_dev, int max_seq_len, float* out) {
    PagedAttnPlan plan;
    cudaError_t e = paged_attention_make_plan(&plan, sh, kv_bf16, k_pool, v_pool, max_seq_len, ctx->tune_attn_chunk_blocks);
    if (e != cudaSuccess) return fail(B200_KERNEL_LAUNCH_FAILED, "paged_attention: tensor map creation failed");
    const size_t tables_bytes = align_up(size_t(sh.batch) * sh.max_blocks_per_seq * 4, 256);
    const size_t seq_bytes = align_up(size_t(sh.batch) * 4, 256);
    const size_t scratch = paged_attention_scratch_bytes(plan);
    const size_t stage = tables_host ? tables_bytes + seq_bytes : 0;
    uint8_t* ws = nullptr;
    if (stage + scratch > 0) {
        ws = static_cast<uint8_t*>(ensure_ws(ctx, stage + scratch));
        if (!ws) return B200_DEVICE_ALLOCATION_FAILED;
    }
    if (tables_host) {
        // The reference uploads block tables and seq_lens on every call
        // (crates/backend-cuda/src/paged_kv.rs:222-310); so does this entry.
        e = cudaMemcpyAsync(ws, tables_host, size_t(sh.batch) * sh.max_blocks_per_seq * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(ws + tables_bytes, seq_host, size_t(sh.batch) * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) return fail_runtime(ctx, B200_TRANSFER_FAILED, std::string("paged_attention upload: ") + cudaGetErrorString(e));
        tables_dev = reinterpret_cast<const uint32_t*>(ws);
        seq_dev = reinterpret_cast<const uint32_t*>(ws + tables_bytes);
    }
    e = paged_attention_launch(plan, q, k_pool, v_pool, tables_dev, seq_dev, out, ws ? ws + stage : nullptr, ctx->attn_counter, ctx->sm_count, ctx->err_dev,
                               ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("paged_attention: ") + cudaGetErrorString(e));
    return B200_OK;
}

}  // namespace

extern "C" {

int32_t b200_validate_paged_kv_append(uint64_t k_new_numel, uint64_t v_new_numel, uint64_t k_pool_numel,
                                      uint64_t v_pool_numel, const uint32_t* slot_mapping, uint64_t n_slots,
                                      const b200_paged_kv_layout* layout, uint64_t* rows_out) {
    return validate_append(k_new_numel, v_new_numel, k_pool_numel, v_pool_numel, slot_mapping, n_slots, layout, rows_out);
}

int32_t b200_validate_paged_attention(uint64_t q_numel, uint64_t k_pool_numel, uint64_t v_pool_numel,
                                      const uint32_t* block_tables, uint64_t n_tables, const uint32_t* seq_lens,
                                      uint64_t n_seq_lens, const b200_paged_attention_args* args,
                                      b200_paged_attention_plan* plan_out) {
    return validate_attention(q_numel, k_pool_numel, v_pool_numel, block_tables, n_tables, seq_lens, n_seq_lens, args, plan_out);
}

int32_t b200_paged_attention_tuning(b200_ctx* ctx, int32_t chunk_blocks) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "paged_attention_tuning: context is null");
    if (chunk_blocks < 0 || chunk_blocks > 256) return fail(B200_INVALID_ARGUMENT, "paged_attention_tuning: chunk_blocks must be in 0..256");
    ctx->tune_attn_chunk_blocks = chunk_blocks;
    return B200_OK;
}

int32_t b200_paged_kv_append(b200_ctx* ctx, const b200_buf* k_new, size_t k_new_off, const b200_buf* v_new, size_t v_new_off,
                             b200_buf* k_pool, b200_buf* v_pool, const uint32_t* slot_mapping, uint64_t n_slots,
                             const b200_paged_kv_layout* layout) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (!k_new || !v_new || !k_pool || !v_pool) return fail(B200_INVALID_ARGUMENT, "paged_kv_append: null buffer");
    if (int32_t st = layout_recheck(layout)) return st;
    const size_t es = elem_size(layout->dtype);
    if (k_new_off > k_new->bytes || v_new_off > v_new->bytes) return fail(B200_SHAPE_MISMATCH, "paged_kv_append: offset beyond buffer");
    uint64_t rows = 0;
    if (int32_t st = validate_append((k_new->bytes - k_new_off) / 4, (v_new->bytes - v_new_off) / 4, k_pool->bytes / es,
                                     v_pool->bytes / es, slot_mapping, n_slots, layout, &rows))
        return st;
    if (int32_t st = check_buf(ctx, k_new, k_new_off, rows * layout->embed_dim * 4, "paged_kv_append k_new")) return st;
    if (int32_t st = check_buf(ctx, v_new, v_new_off, rows * layout->embed_dim * 4, "paged_kv_append v_new")) return st;
    if (int32_t st = check_buf(ctx, k_pool, 0, k_pool->bytes, "paged_kv_append k_pool")) return st;
    if (int32_t st = check_buf(ctx, v_pool, 0, v_pool->bytes, "paged_kv_append v_pool")) return st;
    if ((k_new_off & 15) || (v_new_off & 15)) return fail(B200_INVALID_ARGUMENT, "paged_kv_append: offsets must be multiples of 16 bytes");
    if (rows == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    uint32_t* slots_dev = static_cast<uint32_t*>(ensure_ws(ctx, rows * 4));
    if (!slots_dev) return B200_DEVICE_ALLOCATION_FAILED;
    cudaError_t e = cudaMemcpyAsync(slots_dev, slot_mapping, rows * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess)
        e = paged_kv_append(buf_ptr<const float>(k_new, k_new_off), buf_ptr<const float>(v_new, v_new_off), k_pool->ptr,
                            v_pool->ptr, slots_dev, int64_t(rows), int64_t(layout->embed_dim), int64_t(pool_rows(layout)),
                            layout->dtype == B200_BF16, ctx->err_dev, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("paged_kv_append: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_paged_attention_forward(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                     const b200_buf* v_pool, const uint32_t* block_tables, uint64_t n_tables,
                                     const uint32_t* seq_lens, uint64_t n_seq_lens, const b200_paged_attention_args* args,
                                     b200_buf* out, size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (!q || !k_pool || !v_pool || !out) return fail(B200_INVALID_ARGUMENT, "paged_attention_forward: null buffer");
    if (int32_t st = args_recheck(args)) return st;
    const size_t es = elem_size(args->layout.dtype);
    if (q_off > q->bytes) return fail(B200_SHAPE_MISMATCH, "paged_attention_forward: q offset beyond buffer");
    b200_paged_attention_plan plan;
    if (int32_t st = validate_attention((q->bytes - q_off) / 4, k_pool->bytes / es, v_pool->bytes / es, block_tables, n_tables,
                                        seq_lens, n_seq_lens, args, &plan))
        return st;
    if (int32_t st = check_buf(ctx, q, q_off, plan.out_numel * 4, "paged_attention_forward q")) return st;
    if (int32_t st = check_buf(ctx, k_pool, 0, k_pool->bytes, "paged_attention_forward k_pool")) return st;
    if (int32_t st = check_buf(ctx, v_pool, 0, v_pool->bytes, "paged_attention_forward v_pool")) return st;
    if (int32_t st = check_buf(ctx, out, out_off, plan.out_numel * 4, "paged_attention_forward out")) return st;
    if ((q_off & 15) || (out_off & 15)) return fail(B200_INVALID_ARGUMENT, "paged_attention_forward: offsets must be multiples of 16 bytes");
    if (plan.out_numel == 0) return B200_OK;
    PagedAttnShape sh;
    if (int32_t st = shape_from_args(args, &sh)) return st;
    if (int32_t st = set_device(ctx)) return st;
    return run_attention(ctx, sh, args->layout.dtype == B200_BF16, buf_ptr<const float>(q, q_off), k_pool->ptr, v_pool->ptr,
                         block_tables, seq_lens, nullptr, nullptr, int(plan.s_max), buf_ptr<float>(out, out_off));
}

int32_t b200_paged_attention_forward_resident(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                              const b200_buf* v_pool, const b200_buf* block_tables, const b200_buf* seq_lens,
                                              uint64_t max_seq_len, const b200_paged_attention_args* args, b200_buf* out,
                                              size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = args_recheck(args)) return st;
    const size_t es = elem_size(args->layout.dtype);
    const uint64_t eq = args->num_heads * head_dim(args);
    uint64_t out_numel;
    if (!cmul(args->batch, args->l_new, &out_numel) || !cmul(out_numel, eq, &out_numel)) return invalid("output element count overflows");
    uint64_t max_seq;
    if (!cmul(args->max_blocks_per_seq, args->layout.block_size, &max_seq)) return invalid("max_blocks_per_seq * block_size overflows");
    if (max_seq_len > max_seq || max_seq_len > kI32Max) return invalid("max_seq_len exceeds max_blocks_per_seq * block_size");
    if (int32_t st = check_buf(ctx, q, q_off, out_numel * 4, "paged_attention_forward_resident q")) return st;
    if (int32_t st = check_buf(ctx, out, out_off, out_numel * 4, "paged_attention_forward_resident out")) return st;
    if (int32_t st = check_buf(ctx, k_pool, 0, pool_elems(&args->layout) * es, "paged_attention_forward_resident k_pool")) return st;
    if (int32_t st = check_buf(ctx, v_pool, 0, pool_elems(&args->layout) * es, "paged_attention_forward_resident v_pool")) return st;
    if (int32_t st = check_buf(ctx, block_tables, 0, args->batch * args->max_blocks_per_seq * 4, "paged_attention_forward_resident block_tables")) return st;
    if (int32_t st = check_buf(ctx, seq_lens, 0, args->batch * 4, "paged_attention_forward_resident seq_lens")) return st;
    if ((q_off & 15) || (out_off & 15)) return fail(B200_INVALID_ARGUMENT, "paged_attention_forward_resident: offsets must be multiples of 16 bytes");
    if (out_numel == 0) return B200_OK;
    PagedAttnShape sh;
    if (int32_t st = shape_from_args(args, &sh)) return st;
    if (int32_t st = set_device(ctx)) return st;
    return run_attention(ctx, sh, args->layout.dtype == B200_BF16, buf_ptr<const float>(q, q_off), k_pool->ptr, v_pool->ptr,
                         nullptr, nullptr, buf_ptr<const uint32_t>(block_tables, 0), buf_ptr<const uint32_t>(seq_lens, 0),
                         int(max_seq_len), buf_ptr<float>(out, out_off));
}

// Decode attention for callers that cannot allocate device memory at call time - a host thread that
// drives the GPU from inside a latency-critical serving loop or a callback where cudaMalloc (which may
// synchronise the whole device and take a driver lock) is forbidden, or a process whose memory budget was
// handed out in full at start-up.  Same computation and same arguments as
// b200_paged_attention_forward_resident; the split partials go to a fixed 32 MiB array that is part of
// the library image on every GPU that loads it, instead of the context's growable scratch.
//  - Sizes whose partials would not fit (query rows * heads * splits * 520 bytes > 32 MiB) are refused
//    with B200_UNSUPPORTED; nothing is launched.
//  - The first call on a device looks up the array's device address; make that call before any stream
//    capture begins on the device.
//  - The array is shared by every context of the process on that GPU and keeps the previous call's
//    contents; each launch overwrites every partial it later reads, so nothing needs clearing, but two
//    calls whose kernels overlap on the GPU (different streams or contexts) race on it.
int32_t b200_paged_attention_forward_noalloc(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                             const b200_buf* v_pool, const b200_buf* block_tables,
                                             const b200_buf* seq_lens, uint64_t max_seq_len,
                                             const b200_paged_attention_args* args, b200_buf* out, size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = args_recheck(args)) return st;
    const size_t es = elem_size(args->layout.dtype);
    const uint64_t eq = args->num_heads * head_dim(args);
    uint64_t out_numel;
    if (!cmul(args->batch, args->l_new, &out_numel) || !cmul(out_numel, eq, &out_numel)) return invalid("output element count overflows");
    uint64_t max_seq;
    if (!cmul(args->max_blocks_per_seq, args->layout.block_size, &max_seq)) return invalid("max_blocks_per_seq * block_size overflows");
    if (max_seq_len > max_seq || max_seq_len > kI32Max) return invalid("max_seq_len exceeds max_blocks_per_seq * block_size");
    if (int32_t st = check_buf(ctx, q, q_off, out_numel * 4, "paged_attention_forward_noalloc q")) return st;
    if (int32_t st = check_buf(ctx, out, out_off, out_numel * 4, "paged_attention_forward_noalloc out")) return st;
    if (int32_t st = check_buf(ctx, k_pool, 0, pool_elems(&args->layout) * es, "paged_attention_forward_noalloc k_pool")) return st;
    if (int32_t st = check_buf(ctx, v_pool, 0, pool_elems(&args->layout) * es, "paged_attention_forward_noalloc v_pool")) return st;
    if (int32_t st = check_buf(ctx, block_tables, 0, args->batch * args->max_blocks_per_seq * 4, "paged_attention_forward_noalloc block_tables")) return st;
    if (int32_t st = check_buf(ctx, seq_lens, 0, args->batch * 4, "paged_attention_forward_noalloc seq_lens")) return st;
    if ((q_off & 15) || (out_off & 15)) return fail(B200_INVALID_ARGUMENT, "paged_attention_forward_noalloc: offsets must be multiples of 16 bytes");
    if (out_numel == 0) return B200_OK;
    PagedAttnShape sh;
    if (int32_t st = shape_from_args(args, &sh)) return st;
    if (int32_t st = set_device(ctx)) return st;
    PagedAttnPlan plan;
    cudaError_t e = paged_attention_make_plan(&plan, sh, args->layout.dtype == B200_BF16, k_pool->ptr, v_pool->ptr,
                                              int(max_seq_len), ctx->tune_attn_chunk_blocks);
    if (e != cudaSuccess) return fail(B200_KERNEL_LAUNCH_FAILED, "paged_attention_forward_noalloc: tensor map creation failed");
    const size_t need = paged_attention_scratch_bytes(plan);
    if (need > paged_attention_static_scratch_capacity()) {
        char msg[200];
        std::snprintf(msg, sizeof msg,
                      "paged_attention_forward_noalloc: the split partials need %zu bytes, the static scratch holds %zu; "
                      "use b200_paged_attention_forward_resident for this size",
                      need, paged_attention_static_scratch_capacity());
        return fail(B200_UNSUPPORTED, msg);
    }
    void* scratch = nullptr;
    e = paged_attention_static_scratch(ctx->ordinal, &scratch);
    if (e != cudaSuccess)
        return fail(B200_KERNEL_LAUNCH_FAILED, std::string("paged_attention_forward_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    e = paged_attention_launch(plan, buf_ptr<const float>(q, q_off), k_pool->ptr, v_pool->ptr,
                               buf_ptr<const uint32_t>(block_tables, 0), buf_ptr<const uint32_t>(seq_lens, 0),
                               buf_ptr<float>(out, out_off), scratch, ctx->attn_counter, ctx->sm_count, ctx->err_dev, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("paged_attention_forward_noalloc: ") + cudaGetErrorString(e));
    return B200_OK;
}

}  // extern "C"
