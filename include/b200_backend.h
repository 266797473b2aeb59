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
    B200_STALE_DEVICE_GENERATION = 11
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
uint64_t b200_ctx_generation(const b200_ctx* ctx);
/* The CUDA stream of the context as an opaque pointer (for event timing by callers). */
void* b200_ctx_stream(b200_ctx* ctx);

/* Overrides the GEMM tile width (64/128/256) and split-K count for later calls on this
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

/* ------------------------------------------------------------------ quantized linear
 * BackendOps::linear_forward_device_into_tracked (crates/tensor-core/src/backend_ops.rs:4296-4366)
 * for INT8 per-output-channel weights: a [m, k] f32 device-resident, weight given as
 * views (buffer + byte offset) into flat parameter buffers (int8 payload [n, k], f32
 * scales [n], optional f32 bias [n]).  The activation is quantised on the device,
 * per token to int8 (act_dtype B200_I8) or per tensor to E4M3 (B200_FP8_E4M3, with the
 * int8 weights re-encoded as E4M3 is NOT done: that combination is B200_UNSUPPORTED),
 * multiplied on the tensor cores and written, all m*n (or m*n/2) elements, into `out`
 * f32 without reading it. */
int32_t b200_linear_w8a8(b200_ctx* ctx, const b200_buf* a_f32, size_t a_off, int64_t m, int64_t k,
                         const b200_buf* w_i8, size_t w_off, const b200_buf* w_scale, size_t w_scale_off,
                         const b200_buf* bias, size_t bias_off, int64_t n, int32_t activation,
                         const b200_buf* residual, size_t residual_off, b200_buf* out, size_t out_off);

#ifdef __cplusplus
}
#endif
#endif /* B200_BACKEND_H */
