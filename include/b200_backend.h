/*
 * b200_backend.h - C ABI of the B200 (sm_100a) quantized transformer-decode backend.
 *
 * Drop-in boundary for the hot path of Fandhe-AI/fandhe-ai: every entry point below
 * is what an `extern "C"` block inside the reference's crates/backend-cuda would
 * bind in order to serve the corresponding `BackendOps` / `MemoryOps` trait method
 * (crates/tensor-core/src/backend_ops.rs:1275, crates/tensor-core/src/buffer.rs:389).
 * Plain pointers and sizes only; no C++ or torch types cross this boundary.
 *
 * Conventions (they restate the reference's contracts):
 *  - Every function returns a b200_status.  0 is success.  The codes carry the
 *    names of the reference's BackendError variants
 *    (crates/tensor-core/src/device.rs:225-371).  b200_last_error() returns a
 *    thread-local message for the last non-zero status on this thread.
 *  - All validation happens before the first driver call.  A failure that happens
 *    after work was enqueued poisons the context: later calls return
 *    B200_DEVICE_CONTEXT_POISONED until the context is destroyed and re-created.
 *  - Everything is enqueue-only on the context's single stream, except
 *    b200_download and b200_synchronize, which are the synchronisation points
 *    (crates/tensor-core/src/buffer.rs:61-69).
 *  - Buffers are created only by the backend and carry the generation of the
 *    context that made them; handing in a buffer of another context or generation
 *    is an error (B200_DEVICE_MISMATCH / B200_STALE_DEVICE_GENERATION), never UB.
 *  - There is no CPU fallback.  An unsupported request is B200_UNSUPPORTED.
 */
#ifndef B200_BACKEND_H
#define B200_BACKEND_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_ctx b200_ctx;   /* one per CUDA ordinal: stream, error word, generation, poison flag */
typedef struct b200_buf b200_buf;   /* device buffer handle: pointer, size in bytes, owner, generation */

typedef enum b200_status {
    B200_OK = 0,
    B200_SHAPE_MISMATCH = 1,
    B200_DEVICE_MISMATCH = 2,
    B200_DEVICE_ALLOCATION_FAILED = 3,
    B200_KERNEL_LAUNCH_FAILED = 4,
    B200_DEVICE_UNAVAILABLE = 5,
    B200_TRANSFER_FAILED = 6,
    B200_UNSUPPORTED = 7,
    B200_STORE_POISONED = 8,
    B200_INVALID_ARGUMENT = 9,
    B200_DEVICE_CONTEXT_POISONED = 10,
    B200_STALE_DEVICE_GENERATION = 11,
    B200_DEVICE_CONTEXT_RETIRING = 12,             /* transient: the context is being recovered by another call */
    B200_DEVICE_CONTEXT_UNRECOVERABLE = 13,        /* recovery failed for good: restart the process */
    B200_DEVICE_CONTEXT_CAPTURE_IN_PROGRESS = 14   /* transient: another thread is capturing a CUDA graph on the context */
} b200_status;

/* Activation selector of the fused epilogue.  NONE and RELU are the reference's
 * `Activation` (crates/tensor-core/src/backend_ops.rs:631-636); SILU and SILU_GATE
 * are the additions the quantized decoder needs (SiLU formula:
 * crates/tensor-core/src/scalar_op.rs:355,666-673). */
typedef enum b200_activation {
    B200_ACT_NONE = 0,
    B200_ACT_RELU = 1,
    B200_ACT_SILU = 2,
    B200_ACT_SILU_GATE = 3   /* weight rows [0, n/2) = gate, [n/2, n) = up; output has n/2 columns */
} b200_activation;

typedef enum b200_dtype {
    B200_F32 = 0,
    B200_BF16 = 1,
    B200_I8 = 2,
    B200_FP8_E4M3 = 3,
    B200_I32 = 4,
    B200_U32 = 5
} b200_dtype;

/* ------------------------------------------------------------------ context */

const char* b200_last_error(void);
const char* b200_status_name(int32_t status);

/* Opens CUDA ordinal `ordinal` (Device::Cuda(ordinal), crates/tensor-core/src/device.rs:58-80):
 * one stream, one device error word.  Fails with B200_DEVICE_UNAVAILABLE when no
 * sm_100 device is there. */
int32_t b200_ctx_create(int32_t ordinal, b200_ctx** out);
int32_t b200_ctx_destroy(b200_ctx* ctx);
/* BackendOps::synchronize_device (crates/tensor-core/src/backend_ops.rs:4897): waits for
 * the stream without a transfer; reports (and poisons on) a device-side error word. */
int32_t b200_synchronize(b200_ctx* ctx);
int32_t b200_ctx_is_poisoned(const b200_ctx* ctx);
/* Recovery of a poisoned context without re-creating it: `invalidate` of the reference's per-ordinal state machine
 * (crates/backend-cuda/src/context_cache.rs:1998-2560; error variants crates/tensor-core/src/device.rs:334-371).
 * Drains the stream, clears the device error word and runs the recovery probe (256-byte allocation, upload,
 * identity kernel, download, compare).  On success the context starts a new generation: every buffer, decoder and
 * scheduler made before is refused with B200_STALE_DEVICE_GENERATION / B200_STORE_POISONED and must be re-made.
 * While this runs, calls from other threads answer B200_DEVICE_CONTEXT_RETIRING.  A failed probe leaves the
 * context poisoned (retry allowed); the third consecutive failure, or a stream that cannot be drained, makes it
 * B200_DEVICE_CONTEXT_UNRECOVERABLE for the life of the process.  A healthy context is left untouched. */
int32_t b200_ctx_recover(b200_ctx* ctx);
/* Failure injection on the host, for tests of the state machine above (no device fault is ever provoked):
 * the next `count` recovery probes report a mismatch without touching the device; a context is marked poisoned. */
int32_t b200_test_inject_probe_failures(b200_ctx* ctx, int32_t count);
int32_t b200_test_poison(b200_ctx* ctx);
/* on != 0: the calling thread is treated as capturing a CUDA graph on the context (what the decode driver does
 * around its own capture), so calls from other threads answer B200_DEVICE_CONTEXT_CAPTURE_IN_PROGRESS; 0 ends it. */
int32_t b200_test_mark_capturing(b200_ctx* ctx, int32_t on);
/* Free and total device memory of the context's GPU in bytes (cudaMemGetInfo).  No counterpart in the reference;
 * lets a caller check that a call allocated nothing. */
int32_t b200_memory_info(b200_ctx* ctx, size_t* free_bytes, size_t* total_bytes);
uint64_t b200_ctx_generation(const b200_ctx* ctx);
/* The CUDA stream of the context as an opaque pointer (for event timing by callers). */
void* b200_ctx_stream(b200_ctx* ctx);

/* Overrides the GEMM tile width (64/128/224/256) and split-K count for later calls on this
 * context; 0 restores the heuristic.  The counterpart of the reference's per-shape kernel
 * selection (crates/backend-cuda/src/gemm_auto.rs:1829-1892), exposed for tests and tuning. */
int32_t b200_gemm_tuning(b200_ctx* ctx, int32_t tile_n, int32_t splits);

/* ------------------------------------------------------------------ MemoryOps
 * crates/tensor-core/src/buffer.rs:389-521.  Sizes are bytes.  A zero-sized request
 * returns a valid empty handle and never touches the driver. */
int32_t b200_alloc_zeroed(b200_ctx* ctx, size_t bytes, b200_buf** out);              /* MemoryOps::alloc_zeroed */
int32_t b200_upload(b200_ctx* ctx, const void* host, size_t bytes, b200_buf** out);  /* MemoryOps::upload */
int32_t b200_upload_into(b200_ctx* ctx, const void* host, size_t bytes, b200_buf* dst, size_t dst_offset);
                                                                                     /* MemoryOps::upload_into */
int32_t b200_download(b200_ctx* ctx, const b200_buf* src, size_t src_offset, void* host, size_t bytes);
                                                                                     /* MemoryOps::download (sync) */
int32_t b200_release(b200_ctx* ctx, b200_buf* buf);   /* Drop of DeviceBuffer (buffer.rs:40-48) */
size_t b200_buf_bytes(const b200_buf* buf);
void* b200_buf_device_ptr(const b200_buf* buf);

/* ------------------------------------------------------------------ quantisation API
 * Shaped after the reference's proposed QuantOps {quantize, dequantize, gemm_i8_s32_scaled}
 * (docs/backend-int8-quantization-decision.md:88-94); the numeric rule is symmetric
 * scale = amax / 127 with round-half-even, amax taken per output channel (weights)
 * or per token (activations); FP8 is per-tensor scale = amax / 448, E4M3, RNE,
 * saturating.  All arguments are device buffers with byte offsets. */
int32_t b200_quantize_i8_per_row(b200_ctx* ctx, const b200_buf* x_f32, size_t x_off, int64_t rows, int64_t cols,
                                 b200_buf* q_i8, size_t q_off, b200_buf* scale_f32, size_t scale_off);
int32_t b200_dequantize_i8_per_row(b200_ctx* ctx, const b200_buf* q_i8, size_t q_off, const b200_buf* scale_f32,
                                   size_t scale_off, int64_t rows, int64_t cols, b200_buf* x_f32, size_t x_off);
int32_t b200_quantize_fp8_e4m3_per_tensor(b200_ctx* ctx, const b200_buf* x_f32, size_t x_off, int64_t numel,
                                          b200_buf* q_fp8, size_t q_off, b200_buf* scale_f32, size_t scale_off);

/* acc[m, n] = sum_k a[m, k] * w[n, k] in exact int32.  a: [m, k] int8, w: [n, k] int8,
 * acc: [m, n] int32.  Exposed so accumulators can be compared bit for bit
 * (host model: crates/backend-cuda/tests/int8_mma_probe_real_device.rs:196-238). */
int32_t b200_gemm_i8_s32(b200_ctx* ctx, const b200_buf* a_i8, size_t a_off, const b200_buf* w_i8, size_t w_off,
                         int64_t m, int64_t n, int64_t k, b200_buf* acc_i32, size_t acc_off);

/* Scaled quantized GEMM with the fused epilogue
 *   y[m, j] = act(acc[m, j] * a_scale[m or 0] * w_scale[j or 0] + bias[j]) (+ residual[m, j])
 * (bias then activation, once after the full-K sum: crates/tensor-core/src/backend_ops.rs:4111-4127).
 * op_dtype: B200_I8 (s32 accumulate) or B200_FP8_E4M3 (f32 accumulate).
 * a_scale: per row ([m]) when a_scale_per_row != 0 else one value; w_scale likewise per
 * weight row.  bias, residual may be NULL.  out_dtype: B200_F32 or B200_BF16.
 * For B200_ACT_SILU_GATE the output has n/2 columns. */
int32_t b200_gemm_q8_scaled(b200_ctx* ctx, int32_t op_dtype, const b200_buf* a_q, size_t a_off,
                            const b200_buf* a_scale, size_t a_scale_off, int32_t a_scale_per_row,
                            const b200_buf* w_q, size_t w_off, const b200_buf* w_scale, size_t w_scale_off,
                            int32_t w_scale_per_row, const b200_buf* bias, size_t bias_off, int32_t activation,
                            const b200_buf* residual, size_t residual_off, int64_t m, int64_t n, int64_t k,
                            int32_t out_dtype, b200_buf* out, size_t out_off);

/* ------------------------------------------------------------------ block-scale INT8 contract
 * The variant the reference proposes for its own quantisation backend (QuantOps {quantize, dequantize,
 * gemm_i8_s32_scaled}, docs/backend-int8-quantization-decision.md:88-94; numeric contract
 * docs/int8-quant-grade-up-verification-plan.md:177-241):
 *   - one scale per `block_len` = 128 consecutive values of K, on both operands (per token x block for activations,
 *     per output channel x block for weights); delta = pow2ceil(max(amax_block, 1e-4) / 127), q = rne(x / delta),
 *     so |q| <= 127 without clamping and every scale is a power of two;
 *   - per block: s32 partial (exact) -> f32 (exact: |partial| <= 128 * 127^2 = 2 064 512 < 2^24) -> ONE multiplication
 *     by the composed scale delta_a * delta_b (exact) -> widened to f64; the blocks are added in ascending order in
 *     f64 and the sum is narrowed to f32 once.  The result is a pure function of the inputs: bit-identical to the
 *     CPU restatement (acceptance rule fail_count == 0).
 * The scale array of x [rows, cols] is [rows, nb] (scales_block_major = 0) or [nb, rows] (1), nb = ceil(cols / 128);
 * the GEMM takes the activation scales as [m, nb] and the weight scales as [nb, n].
 * Requests outside the contract are typed errors, never wrap-arounds or infinities: a block length above
 * K_safe = floor(i32::MAX / 127^2) = 133 144 is B200_INVALID_ARGUMENT (lengths other than 128 are B200_UNSUPPORTED);
 * a NaN / infinite input value and a result that overflows f32 at the final narrowing are recorded on the device and
 * reported by b200_quant_check as B200_INVALID_ARGUMENT (the context is not poisoned; the affected block is zeroed /
 * the affected output holds the infinity). */
int32_t b200_quantize_i8_block(b200_ctx* ctx, const b200_buf* x_f32, size_t x_off, int64_t rows, int64_t cols,
                               int64_t block_len, int32_t scales_block_major, b200_buf* q_i8, size_t q_off,
                               b200_buf* delta_f32, size_t delta_off);
int32_t b200_dequantize_i8_block(b200_ctx* ctx, const b200_buf* q_i8, size_t q_off, const b200_buf* delta_f32,
                                 size_t delta_off, int64_t rows, int64_t cols, int64_t block_len,
                                 int32_t scales_block_major, b200_buf* x_f32, size_t x_off);
int32_t b200_gemm_i8_block_scaled(b200_ctx* ctx, const b200_buf* a_i8, size_t a_off, const b200_buf* a_delta,
                                  size_t a_delta_off, const b200_buf* w_i8, size_t w_off, const b200_buf* w_delta,
                                  size_t w_delta_off, int64_t m, int64_t n, int64_t k, int64_t block_len, b200_buf* out_f32,
                                  size_t out_off);
/* Synchronises and reports what the three calls above flagged since the last check (then clears it). */
int32_t b200_quant_check(b200_ctx* ctx);

/* Which kernel form b200_gemm_i8_s32 (fused = 0) or b200_gemm_q8_scaled (fused = 1; gated = 1 for
 * B200_ACT_SILU_GATE) would use for a shape under the context's current tuning; nothing is launched.
 * out6 = {tile width, K splits, splits reduced inside a cluster (0/1), persistent kernel (0: no, 1: one CTA per tile,
 * 2: CTA pairs on 256-row tiles), resident CTAs of the persistent kernel, operand stages}.  The counterpart of asking the reference's kernel selection what it would run
 * (crates/backend-cuda/src/gemm_auto.rs:1829-1892); lets a test state which kernel it reached. */
int32_t b200_gemm_plan_info(b200_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t gated, int32_t fused, int32_t* out6);
/* Profiling aid for decode-shaped GEMMs (one-tile kernel): `iters` launches back to back between two CUDA events
 * (loop_us_per_launch), then one launch alone (alone_us) whose first CTA records %globaltimer at nine points;
 * stamps_ns9[i] = nanoseconds since the CTA's first instruction: 0 entry, 1 barriers + tensor memory set up, 2 the
 * launch before has completed, 3 first pass of TMA loads issued, 4 first operand stage has landed, 5 last MMA issued,
 * 6 accumulator complete, 7 the first epilogue warp has issued its stores, 8 tensor memory freed.  info6 as in b200_gemm_plan_info.
 * fused = 0: raw accumulators; 1: the dequantising epilogue.  Operands are zero-filled.  No reference counterpart. */
int32_t b200_gemm_phase_stamps(b200_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t fused, int32_t iters, uint64_t* stamps_ns9,
                               float* loop_us_per_launch, float* alone_us, int32_t* info6);

/* ------------------------------------------------------------------ quantized linear
 * BackendOps::linear_forward_device_into_tracked (crates/tensor-core/src/backend_ops.rs:4296-4366)
 * for INT8 per-output-channel weights: a [m, k] f32 device-resident, weight given as
 * views (buffer + byte offset) into flat parameter buffers (int8 payload [n, k], f32
 * scales [n], optional f32 bias [n]).  The activation is quantised on the device per
 * token to int8, multiplied on the tensor cores (s32 accumulators) and written, all
 * m*n (or m*n/2 for the gate form) elements, into `out` f32 without reading it. */
int32_t b200_linear_w8a8(b200_ctx* ctx, const b200_buf* a_f32, size_t a_off, int64_t m, int64_t k,
                         const b200_buf* w_i8, size_t w_off, const b200_buf* w_scale, size_t w_scale_off,
                         const b200_buf* bias, size_t bias_off, int64_t n, int32_t activation,
                         const b200_buf* residual, size_t residual_off, b200_buf* out, size_t out_off);

/* The same operator with FP8-E4M3 operands (the successor of the reference's f16 / bf16 low-precision linear,
 * crates/tensor-core/src/low_precision.rs:193-249): the weight view holds E4M3 codes [n, k] with ONE f32 scale
 * (per tensor, amax -> 448); the f32 activation [m, k] is quantised on the device per tensor the same way;
 * f32 accumulation; epilogue y = act(acc * sa * sw + bias) (+ residual); out_dtype B200_F32 or B200_BF16.
 * tcgen05 has no MMA that mixes int8 and E4M3 operands, so int8 weights cannot be used here: re-encode them. */
int32_t b200_linear_fp8(b200_ctx* ctx, const b200_buf* a_f32, size_t a_off, int64_t m, int64_t k,
                        const b200_buf* w_fp8, size_t w_off, const b200_buf* w_scale, size_t w_scale_off,
                        const b200_buf* bias, size_t bias_off, int64_t n, int32_t activation,
                        const b200_buf* residual, size_t residual_off, int32_t out_dtype, b200_buf* out, size_t out_off);

/* ------------------------------------------------------------------ paged KV cache
 * PagedKvLayout / PagedAttentionArgs / PagedAttentionPlan of the reference
 * (crates/tensor-core/src/paged_kv.rs:47-123, 130-200, 204-213), extended with the pool
 * element type and the number of KV heads.  K and V pools are [num_blocks, block_size,
 * embed_dim] row-major with embed_dim = num_kv_heads * head_dim; a token row is
 * block_id * block_size + pos % block_size.  q and out are f32 [batch, l_new, num_heads * head_dim]. */
typedef struct b200_paged_kv_layout {
    uint64_t num_blocks;   /* 1 .. u32::MAX - 1 */
    uint64_t block_size;   /* power of two, 1 .. 256 */
    uint64_t embed_dim;    /* E of the pools, 1 .. i32::MAX */
    int32_t dtype;         /* B200_BF16 or B200_F32 */
} b200_paged_kv_layout;

typedef struct b200_paged_attention_args {
    b200_paged_kv_layout layout;
    uint64_t batch;
    uint64_t l_new;
    uint64_t num_heads;            /* query heads; a multiple of num_kv_heads */
    uint64_t num_kv_heads;         /* divides embed_dim; equal to num_heads for the reference's MHA */
    uint64_t max_blocks_per_seq;
    float scale;                   /* multiplied into q before the dot product; finite */
} b200_paged_attention_args;

typedef struct b200_paged_attention_plan {
    uint64_t out_numel;        /* batch * l_new * num_heads * head_dim */
    uint64_t s_max;            /* max(seq_lens) */
    uint64_t query_rows;       /* batch * num_heads * l_new */
    uint64_t workspace_elems;  /* query_rows * s_max, capped at 2^30 as in the reference */
} b200_paged_attention_plan;

/* validate_paged_kv_append (crates/tensor-core/src/paged_kv.rs:220-267): element counts, slots
 * below num_blocks * block_size, no duplicate slot.  Pure host function, needs no device. */
int32_t b200_validate_paged_kv_append(uint64_t k_new_numel, uint64_t v_new_numel, uint64_t k_pool_numel,
                                      uint64_t v_pool_numel, const uint32_t* slot_mapping, uint64_t n_slots,
                                      const b200_paged_kv_layout* layout, uint64_t* rows_out);
/* validate_paged_attention (crates/tensor-core/src/paged_kv.rs:276-373): l_new <= seq_len <=
 * max_blocks_per_seq * block_size, used block ids < num_blocks (the sentinel 0xFFFFFFFF only in
 * unused slots), workspace cap.  Pure host function, needs no device. */
int32_t b200_validate_paged_attention(uint64_t q_numel, uint64_t k_pool_numel, uint64_t v_pool_numel,
                                      const uint32_t* block_tables, uint64_t n_tables, const uint32_t* seq_lens,
                                      uint64_t n_seq_lens, const b200_paged_attention_args* args,
                                      b200_paged_attention_plan* plan_out);

/* BackendOps::paged_kv_append (crates/tensor-core/src/backend_ops.rs:4709-4722): row r of k_new / v_new
 * (f32 [rows, embed_dim]) goes to pool row slot_mapping[r] (host array), rounded to the pool dtype.
 * Validates first, then enqueues; no sync. */
int32_t b200_paged_kv_append(b200_ctx* ctx, const b200_buf* k_new, size_t k_new_off, const b200_buf* v_new,
                             size_t v_new_off, b200_buf* k_pool, b200_buf* v_pool, const uint32_t* slot_mapping,
                             uint64_t n_slots, const b200_paged_kv_layout* layout);

/* BackendOps::paged_attention_forward (crates/tensor-core/src/backend_ops.rs:4755-4769):
 * out[b, i, h, :] = softmax_j((q * scale) . k_j) . v_j over j <= seq_len[b] - l_new + i.
 * block_tables is the host array [batch, max_blocks_per_seq] (unused slots 0xFFFFFFFF), seq_lens the
 * host array [batch]; both are validated and uploaded on every call, as the reference does. */
int32_t b200_paged_attention_forward(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                     const b200_buf* v_pool, const uint32_t* block_tables, uint64_t n_tables,
                                     const uint32_t* seq_lens, uint64_t n_seq_lens,
                                     const b200_paged_attention_args* args, b200_buf* out, size_t out_off);

/* Same computation with block tables and seq_lens already resident on the device (u32 buffers kept
 * and updated incrementally by the decode loop); `max_seq_len` is an upper bound of seq_lens that
 * sizes the split grid.  The host cannot check the table contents here: a used slot holding an id
 * >= num_blocks makes the kernel set the device error word (reported by the next download /
 * synchronize) instead of touching memory.  No counterpart in the reference, which re-uploads the
 * tables on each call (crates/backend-cuda/src/paged_kv.rs:222-310).  The lengths are guarded on the device in the
 * same way: a seq_lens entry above max_seq_len (or above max_blocks_per_seq * block_size) is clamped to it
 * and sets the error word (code 0x204), so neither the table row nor another row's partial results are read. */
int32_t b200_paged_attention_forward_resident(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                              const b200_buf* v_pool, const b200_buf* block_tables,
                                              const b200_buf* seq_lens, uint64_t max_seq_len,
                                              const b200_paged_attention_args* args, b200_buf* out, size_t out_off);

/* No counterpart in the reference.  b200_paged_attention_forward_resident for callers that may not
 * allocate device memory when they call: a serving loop or callback in which cudaMalloc is off limits
 * (it can stall the whole device behind a driver lock), or a process that gave away its whole memory
 * budget at start-up.  This entry point calls no cudaMalloc / cudaFree and no allocating library routine:
 * the per-split partial results go to a fixed 32 MiB array inside the library image (held by every GPU
 * that loads the library until the process exits).  Requests whose partials need more - query rows x
 * heads x splits x 520 bytes - are refused with B200_UNSUPPORTED before anything is launched.  The first
 * call on a device resolves the array's device address; issue it before starting any stream capture on
 * that device.  Where the CUDA runtime loads modules lazily and this is the process's first call into the
 * library on that device, the module load - which is when the driver sets the 32 MiB aside - also happens
 * inside this first call; call it (or anything else of the library) once during start-up if that matters.  All contexts of the process share the array on a given GPU, and it keeps whatever the
 * last call left; a call rewrites every partial it reads, so nothing has to be cleared, but calls whose
 * kernels overlap on the GPU race on it. */
int32_t b200_paged_attention_forward_noalloc(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* k_pool,
                                             const b200_buf* v_pool, const b200_buf* block_tables,
                                             const b200_buf* seq_lens, uint64_t max_seq_len,
                                             const b200_paged_attention_args* args, b200_buf* out, size_t out_off);

/* Blocks per split of the decode-attention kernel (1..256; 0 restores the default of 32), for tuning. */
int32_t b200_paged_attention_tuning(b200_ctx* ctx, int32_t chunk_blocks);

/* ------------------------------------------------------------------ host page table
 * BlockTable of the reference (crates/autodiff/src/nn/paged_kv.rs:158-364), host only: blocks are
 * taken from a LIFO stack of returned ids first, then from a counter starting at 0, so the order is
 * deterministic.  All rows have the same length (the reference's invariant). */
typedef struct b200_block_table b200_block_table;
int32_t b200_block_table_create(uint64_t max_blocks, uint64_t block_size, b200_block_table** out);
void b200_block_table_destroy(b200_block_table* table);
/* extend_for_append (paged_kv.rs:206-297): every one of the `batch` rows grows by l_new tokens; writes the
 * row-major slot mapping (row b, token i) into slots_out.  Fails without changing the table when the
 * batch differs from the cached one or the pool has too few free blocks. */
int32_t b200_block_table_extend_for_append(b200_block_table* table, uint64_t batch, uint64_t l_new,
                                           uint32_t* slots_out, uint64_t slots_capacity, uint64_t* n_slots);
/* flatten_tables (paged_kv.rs:299-322): [batch, max_blocks_per_seq], unused slots 0xFFFFFFFF. */
int32_t b200_block_table_flatten(const b200_block_table* table, uint64_t max_blocks_per_seq, uint32_t* out,
                                 uint64_t capacity);
/* rewind_to (paged_kv.rs:324-364): shrink to new_len, hand the tail blocks back; 0 resets the table. */
int32_t b200_block_table_rewind_to(b200_block_table* table, uint64_t new_len);
void b200_block_table_clear(b200_block_table* table);
uint64_t b200_block_table_seq_len(const b200_block_table* table);
uint64_t b200_block_table_free_blocks(const b200_block_table* table);
uint64_t b200_block_table_used_blocks(const b200_block_table* table);
int64_t b200_block_table_batch(const b200_block_table* table);   /* -1 while no batch is fixed */

/* ------------------------------------------------------------------ decode driver
 * The caller of the two kernels families above: a Llama-style decoder stack (RMSNorm eps, rotate-half
 * RoPE, grouped-query paged attention with a bf16 cache, SwiGLU) with INT8 per-output-channel
 * weights and per-token INT8 activations, resident in flat parameter buffers in the manner of
 * DeviceParamStore (crates/autodiff/src/optim/device_store.rs:27-52, 1288-1364), driven like the
 * reference's generate() (crates/autodiff/src/generate/mod.rs:500-613) but with sampling on the
 * device.  The reference has no such model; the wiring is defined here and in the CPU oracle. */
typedef struct b200_decoder b200_decoder;

typedef struct b200_decoder_config {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab;
    float rms_eps;
    float rope_theta;
    int32_t max_batch;      /* rows a step may hold */
    int32_t max_seq_len;    /* positions per row (rope table, block table width) */
    int32_t block_size;     /* tokens per KV block (16 selects the TMA attention path) */
    int32_t num_blocks;     /* blocks per K / V pool per layer */
    int32_t tp_rank, tp_size;   /* tensor parallel: this process's rank and the number of ranks */
    int32_t use_graph;      /* replay each step as a CUDA graph after the first (eager) one */
    int32_t tp_exact_int8;  /* tp_size > 1: quantise the rows that are split over the ranks under ONE per-token scale (the row
                             * maximum merged over the ranks with a max all-reduce) and all-reduce the int32 partial sums, so
                             * that logits and ids do not depend on tp_size (bit-identical to one GPU); costs two more
                             * collectives per layer and runs on ncclAllReduce.  0: every rank scales its slice of a row by
                             * itself and the ranks add dequantised f32 partials (the fast path). */
    int32_t act_fp8;        /* 1: the FP8 x FP8 form of the decoder.  Weights are kept as E4M3 codes with one scale per output
                             * row (amax / 448; f32 weights are encoded at load, int8 payloads are dequantised and re-encoded),
                             * activations are quantised per token to E4M3 (amax / 448), the GEMMs run on the kind::f8f6f4 MMA
                             * with f32 accumulation.  Everything else (RMSNorm, RoPE, attention, sampling) is unchanged.
                             * Row widths must fit the one-CTA row kernels (multiples of 4, at most 16384 columns per rank);
                             * not combinable with tp_exact_int8.  0: INT8 x INT8 (exact int32 accumulation). */
} b200_decoder_config;

typedef enum b200_weight {
    B200_W_EMBED = 0,       /* [vocab, d_model] f32, kept f32 */
    B200_W_ATTN_NORM = 1,   /* [1, d_model] per layer */
    B200_W_QKV = 2,         /* [(n_heads + 2 n_kv_heads) head_dim, d_model]: q rows, then k rows, then v rows */
    B200_W_O = 3,           /* [d_model, n_heads head_dim] */
    B200_W_MLP_NORM = 4,    /* [1, d_model] per layer */
    B200_W_GATE_UP = 5,     /* [2 d_ff, d_model]: gate rows then up rows */
    B200_W_DOWN = 6,        /* [d_model, d_ff] */
    B200_W_FINAL_NORM = 7,  /* [1, d_model] */
    B200_W_LM_HEAD = 8      /* [vocab, d_model] */
} b200_weight;

int32_t b200_decoder_create(b200_ctx* ctx, const b200_decoder_config* cfg, b200_decoder** out);
int32_t b200_decoder_destroy(b200_decoder* dec);
/* Loads one full (unsharded) f32 tensor [rows, cols] from the host; matrices are quantised on the
 * device (one scale per full row) and this rank's shard is kept. */
int32_t b200_decoder_load_tensor(b200_decoder* dec, int32_t which, int32_t layer, const float* host, int64_t rows,
                                 int64_t cols);
/* The same for a matrix that is already quantised (int8 [rows, cols] and one f32 scale per row, both on the host):
 * nothing is re-quantised, this rank's shard is kept. */
int32_t b200_decoder_load_tensor_i8(b200_decoder* dec, int32_t which, int32_t layer, const int8_t* q_host,
                                    const float* scale_host, int64_t rows, int64_t cols);
/* Weight wire format: a safetensors file (or byte buffer) holding every tensor of the decoder.  Extends the
 * reference's loader (crates/onnx-interop/src/st_load.rs:128-222, 433-562; crates/facade/src/interop/safetensors.rs:182),
 * which rejects the I8 dtype today (st_load.rs:624), with per-output-channel int8 weights: for each matrix M of
 * {"lm_head", "layers.<l>.wqkv", "layers.<l>.wo", "layers.<l>.wgu", "layers.<l>.wdown"} either "M.qweight" I8
 * [rows, cols] with "M.scale" F32 [rows], or "M.weight" F32 [rows, cols] (quantised on the device); plus
 * "embed.weight", "final_norm.weight", "layers.<l>.attn_norm.weight", "layers.<l>.mlp_norm.weight" in F32.
 * The reference's rules hold: layout validated first, no renaming or transposition, nothing skipped silently
 * (a wrong dtype or shape and an unknown tensor are errors), all missing names reported in one error. */
int32_t b200_decoder_load_safetensors(b200_decoder* dec, const char* path);
int32_t b200_decoder_load_safetensors_bytes(b200_decoder* dec, const uint8_t* bytes, size_t len);
/* validate_safetensors_layout_from_bytes (crates/onnx-interop/src/st_load.rs:128-132): header and layout only (header
 * length, JSON, offsets contiguous from 0 to the end of the buffer, byte length = shape x dtype width); any dtype of the
 * format; needs no device. */
int32_t b200_safetensors_validate(const uint8_t* bytes, size_t len, uint64_t* n_tensors);
/* Synthetic weights N(0, std^2) from a counter-based generator (norm weights 1), identical on every rank. */
int32_t b200_decoder_init_random(b200_decoder* dec, uint64_t seed, float std);
/* 128-byte NCCL unique id (rank 0 makes it, the launcher hands it to every rank) and communicator set-up. */
int32_t b200_nccl_unique_id(uint8_t* out128);
int32_t b200_decoder_init_tp(b200_decoder* dec, const uint8_t* unique_id128);
/* Non-zero when init_tp mapped the other ranks' exchange blocks (CUDA IPC), so that a row-parallel output is finished
 * by one kernel on the rank that owns the token row (rank-order sum of the ranks' partials, residual, RMSNorm, per-token
 * int8) which delivers the quantised row to every rank; the GEMM that consumes those rows waits for the peers'
 * delivered flags right before it loads its A operand.  2: the row-parallel GEMMs store their partial rows straight into
 * the owner's block and count themselves there, the finish kernel reads local memory only (the default; as planned
 * for the last enqueued step).  1: the GEMMs write local partials and the finish kernel loads them from the peers
 * (B200_TP_PUSH=0 in the environment, or a GEMM plan without a fused epilogue in the one-tile kernel).
 * 0: the step uses ncclAllReduce instead (mapping failed, batch not divisible by the rank count, or
 * B200_TP_EXCHANGE=0 in the environment).  No reference counterpart (the reference has no tensor parallelism). */
int32_t b200_decoder_tp_exchange(const b200_decoder* dec);
/* Failure-detection self-test on one GPU: runs the cross-GPU finish kernel as rank 0 of 2 with a peer whose flags
 * are never raised.  Its time-bounded wait (20 ms here, two seconds in a real run) runs out, the kernel records the
 * peer-wait code in the context's error word, poisons the flags it owns at the peer and returns; this call then
 * returns KernelLaunchFailed and the context is poisoned (recover or re-create it).  The device stays usable.
 * No reference counterpart. */
int32_t b200_selftest_peer_wait(b200_ctx* ctx);
/* Numerical self-test of the finish kernel on one GPU with nothing to wait for: `tp` exchange blocks on this device,
 * partials[tp][tp * rows][d] uploaded and every ready flag raised beforehand, the kernel run as rank `rank` with the
 * residual rows residual[tp * rows][d].  Outputs for the rows that rank owns: h_out[rows][d] (updated residual),
 * xq_out[tp][rows][d] and sx_out[tp][rows] (the int8 rows and scales found in EVERY block afterwards),
 * flags_out[tp][128] (each block's flag words: ready at 0.., delivered at 64..).  No reference counterpart. */
int32_t b200_selftest_tp_finish(b200_ctx* ctx, int32_t tp, int32_t rank, int32_t rows, int32_t d, const float* partials,
                                const float* residual, const float* norm_w, float eps, float* h_out, int8_t* xq_out,
                                float* sx_out, uint32_t* flags_out);
/* Numerical self-test on one GPU of the scattered form of a row-parallel output: for every rank s the int8 GEMM
 * a_q[s][tp * rows][k] x w_q[s][d][k]^T with scales a_scale[s][tp * rows], w_scale[s][d] is launched as rank s and
 * stores each dequantised row into the exchange block of the rank that owns it (`tp` blocks on this device) and counts
 * itself there when its last tile is stored; then the finish kernel runs as rank 0, 1, ... reading only its own block (rank-order sum, residual,
 * RMSNorm, per-token int8) and delivers into every block.  splits / tile as in b200_set_tuning (0: heuristic).
 * Outputs: h_out[tp * rows][d], xq_out[2][tp * rows][d] and sx_out[2][tp * rows] (first and last block),
 * counts_out[tp][tp] (launches counted in every block, per source rank: 1 each).  No reference counterpart. */
int32_t b200_selftest_tp_scatter(b200_ctx* ctx, int32_t tp, int32_t rows, int32_t d, int32_t k, int32_t splits, int32_t tile,
                                 const int8_t* a_q, const float* a_scale, const int8_t* w_q, const float* w_scale,
                                 const float* residual, const float* norm_w, float eps, float* h_out, int8_t* xq_out,
                                 float* sx_out, uint32_t* counts_out);
/* Starts a generation of `batch` rows: row b starts at start_lens[b] cached tokens (NULL: 0) and may grow
 * to max_total_lens[b]; blocks for the final length are reserved now and the tables uploaded once. */
int32_t b200_decoder_begin(b200_decoder* dec, int32_t batch, const int32_t* start_lens, const int32_t* max_total_lens);
/* Benchmark set-up: fills this rank's KV pools with synthetic bf16 values. */
int32_t b200_decoder_fill_cache_random(b200_decoder* dec, uint64_t seed, float std);
/* One decode step.  ids_host != NULL: input ids come from the host; else the previous step's samples.
 * next_ids_host != NULL: the greedy samples are copied back (this synchronises). */
int32_t b200_decoder_step(b200_decoder* dec, const int32_t* ids_host, int32_t* next_ids_host);
int32_t b200_decoder_logits(b200_decoder* dec, float* host, uint64_t capacity_elems);
/* One step in which only the rows with active[b] != 0 advance (NULL: all rows); the others keep their length and
 * contents, and their entries of next_ids mean nothing.  With b200_decoder_row_restart this is what continuous
 * batching over per-row lengths needs (the kernels already take seq_lens[B];
 * docs/device-resident-kv-paged-attention-design.md:51). */
int32_t b200_decoder_step_rows(b200_decoder* dec, const int32_t* ids, const uint8_t* active, int32_t* next_ids);
/* Multi-token prefill: the rows [row0, row0 + count) each consume l_new tokens (ids [count, l_new], host) in one
 * pass over count * l_new token rows: GEMMs at that many rows, every token's K / V appended, attention under the
 * reference's mask j <= seq_len - l_new + i (crates/backend-cpu/src/paged_kv.rs:137-140;
 * docs/device-resident-kv-paged-attention-design.md:149).  The rows' lengths grow by l_new; nothing is sampled (feed the
 * last prompt token through b200_decoder_step for that).  Long prompts are consumed in chunks internally.  The
 * counterpart of the prefill forward of generate() (crates/autodiff/src/generate/mod.rs:500-560). */
int32_t b200_decoder_prefill(b200_decoder* dec, int32_t row0, int32_t count, const int32_t* ids, int32_t l_new);
int32_t b200_decoder_vocab(const b200_decoder* dec);
/* Rows of the running generation (the batch given to b200_decoder_begin; 0 before). */
int32_t b200_decoder_batch(const b200_decoder* dec);

/* ---- sampling other than greedy ------------------------------------------------------------------------------
 * generate() of the reference samples on the host: sample_step (crates/autodiff/src/generate/mod.rs:382-427) builds,
 * per row, f32 weights from the logits in f64 - softmax_weights_f64 (:347-355), top_k_indices (:359-369, value
 * descending then index ascending), sampling_weights_f32 (:433-455) - and draws one index per row from them with its
 * own Generator::multinomial.  These entries produce exactly those weights; the draw stays with the caller's
 * generator, and the drawn ids go back through b200_decoder_step(ids).  The argument rules are those of
 * GenerateConfig::validate (:179-250): temperature finite and > 0; greedy with temperature 1 and k 0; temperature
 * strategy with k 0; top-k with 1 <= k <= vocab.  A non-finite logit is InvalidArgument, as in sample_step. */
enum b200_sampling_strategy {
    B200_SAMPLE_GREEDY = 0,        /* one-hot at the first maximum (never drawn from by the reference) */
    B200_SAMPLE_TEMPERATURE = 1,   /* softmax((x - max) / t) over the whole row */
    B200_SAMPLE_TOP_K = 2          /* the same softmax over the k largest logits, 0 elsewhere */
};
/* logits[rows][vocab] (host) -> weights_out[rows][vocab] (host). */
int32_t b200_sampling_weights(const float* logits, int64_t rows, int64_t vocab, int32_t strategy, int32_t k, float temperature,
                              float* weights_out);
/* The same for the logits of the decoder's last step: weights_out[batch][vocab] (host, capacity in elements). */
int32_t b200_decoder_sampling_weights(b200_decoder* dec, int32_t strategy, int32_t k, float temperature, float* weights_out,
                                      uint64_t capacity_elems);
/* Between steps: empties row `row` (its blocks return to the free stack) and reserves blocks for a new sequence
 * of up to max_total_len tokens (at most the largest length given to b200_decoder_begin). */
int32_t b200_decoder_row_restart(b200_decoder* dec, int32_t row, int32_t max_total_len);
/* generate() with greedy sampling: out is [batch, max_length] and begins with the prompt. */
int32_t b200_decoder_generate(b200_decoder* dec, const int32_t* prompt, int32_t batch, int32_t prompt_len,
                              int32_t max_length, int32_t* out);
/* Tensor-parallel shard arithmetic, pure host (no device needed): for rank cfg->tp_rank of cfg->tp_size,
 * the full shape of matrix `which`, the row ranges it keeps as (start, count) pairs (up to three: q / k / v
 * heads, or gate / up halves) and the column range it keeps (row-parallel O and down projections). */
int32_t b200_decoder_shard_plan(const b200_decoder_config* cfg, int32_t which, int64_t* rows, int64_t* cols,
                                int64_t* row_ranges6, int32_t* n_ranges, int64_t* col_start, int64_t* col_count);
uint64_t b200_decoder_launches_per_step(const b200_decoder* dec);
uint64_t b200_decoder_weight_bytes(const b200_decoder* dec);
int32_t b200_decoder_plan_info(const b200_decoder* dec, int32_t* out10);

/* ------------------------------------------------------------------ measurement aids
 * CUDA-event stopwatch on the context's stream: device time of everything enqueued between start and
 * stop (stop waits for it, without a transfer, like the completion wait of the reference's bench
 * harness, crates/bench-harness/src/lib.rs module doc). */
int32_t b200_timer_start(b200_ctx* ctx);
int32_t b200_timer_stop(b200_ctx* ctx, float* elapsed_ms);
/* Mean device time of one decode-attention launch on the decoder's current caches (cycling over the
 * layers so that each launch reads a different pool) and the algorithmic bytes of one launch. */
int32_t b200_decoder_time_attention(b200_decoder* dec, int32_t iters, float* ms_per_launch, uint64_t* bytes_per_launch);

/* ------------------------------------------------------------------ continuous batching
 * BatchScheduler of the reference (crates/autodiff/src/generate/scheduler.rs:395-): a FIFO queue of requests and
 * at most max_active requests in progress, one decoder row each; a step admits queued requests into free rows and
 * advances every request in progress by one token (an admitted prompt is prefilled up to its last token in one
 * multi-token pass; the last prompt token and then the greedy samples go through the batched decode step);
 * a request finishes when it holds max_length tokens.  Rows and requests are processed in ascending order, so a run
 * is reproducible.  With a decoder, create calls b200_decoder_begin(dec, max_active, ..., max_length per row). */
typedef struct b200_scheduler b200_scheduler;
int32_t b200_scheduler_create(b200_decoder* dec_or_null, int32_t max_active, int32_t max_queued, int32_t max_length,
                              b200_scheduler** out);
void b200_scheduler_destroy(b200_scheduler* s);
/* scheduler.rs:445-504: queues a copy of the prompt, no forward; errors (empty prompt, prompt longer than
 * max_length, max_length above the limit, queue full) leave the state unchanged.  Ids count up from 1. */
int32_t b200_scheduler_submit(b200_scheduler* s, const int32_t* prompt, int32_t prompt_len, int32_t max_length,
                              uint64_t* request_id);
int32_t b200_scheduler_queued_len(const b200_scheduler* s);
int32_t b200_scheduler_active_len(const b200_scheduler* s);
int32_t b200_scheduler_finished_len(const b200_scheduler* s);
/* scheduler.rs:571-589: one iteration; *completed = requests finished by this call. */
int32_t b200_scheduler_step(b200_scheduler* s, int32_t* completed);
/* The two host halves of a step (what b200_scheduler_step does around the decoder calls); arrays hold max_active
 * entries.  Usable without a device. */
int32_t b200_scheduler_plan_step(b200_scheduler* s, int32_t* ids, uint8_t* active, int32_t* restart_rows,
                                 int32_t* restart_lens, int32_t* n_restart, int32_t* completed_without_forward);
int32_t b200_scheduler_commit_step(b200_scheduler* s, const int32_t* sampled, int32_t* completed);
/* Requests set apart because they could not be served (a prompt token outside the vocabulary, no cache blocks for
 * the row): the reference keeps per-request failures out of step()'s error path in the same way
 * (crates/autodiff/src/generate/scheduler.rs:568-589, take_failed :718).  take_failed pops the oldest one: its id,
 * the status code and the message; *have = 0 when there is none. */
int32_t b200_scheduler_failed_len(const b200_scheduler* s);
int32_t b200_scheduler_take_failed(b200_scheduler* s, uint64_t* request_id, int32_t* status, char* message,
                                   int32_t capacity, int32_t* have);
/* For a scheduler without a decoder (host logic only): whether admitted prompts count as prefilled up to their last
 * token, and the vocabulary size that token ids are checked against on admission (0: no check).  With a decoder
 * both are set by create (prefill on, the decoder's vocabulary). */
int32_t b200_scheduler_configure(b200_scheduler* s, int32_t prefill, int32_t vocab);
/* Pops the oldest finished request (prompt + generated tokens); *len = -1 when there is none. */
int32_t b200_scheduler_take_finished(b200_scheduler* s, uint64_t* request_id, int32_t* tokens, int32_t capacity,
                                     int32_t* len);

#ifdef __cplusplus
}
#endif
#endif /* B200_BACKEND_H */
