// Internal C++ view of the C-ABI handles (b200_ctx, b200_buf) and helpers shared by
// the translation units that implement include/b200_backend.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../include/b200_backend.h"

struct b200_ctx {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    uint32_t* err_dev = nullptr;        // device error word written by kernels (0 = none)
    uint32_t* amax_scratch = nullptr;   // one word for tensor-wide amax
    unsigned int* attn_counter = nullptr;  // work counter of the persistent attention kernel (zero between launches)
    uint32_t* quant_status = nullptr;   // block-scale contract: bit 0 non-finite input met, bit 1 non-finite result
    uint32_t* err_host = nullptr;       // pinned mirror used when checking the word
    uint64_t generation = 0;
    bool poisoned = false;
    // Recovery state machine of an ordinal (crates/backend-cuda/src/context_cache.rs): Active -> poisoned ->
    // retiring (b200_ctx_recover drains and probes) -> Active with a new generation, or unrecoverable for good.
    std::atomic<bool> retiring{false};
    bool unrecoverable = false;
    std::string probe_error;            // why recovery failed (diagnostics of the unrecoverable state)
    int probe_failures = 0;             // consecutive failed recovery probes
    int inject_probe_failures = 0;      // host-side failure injection for tests: probes that report a mismatch
    std::atomic<uint64_t> capture_owner{0};   // hashed id of the thread that captures a CUDA graph on this context
    void* ws = nullptr;                 // grow-only scratch for the composite entry points
    size_t ws_bytes = 0;
    bool ws_locked = false;             // set while a composite call lends out part of the scratch
    int tune_bn = 0;                    // 0 = heuristic
    int tune_splits = 0;                // 0 = heuristic
    int tune_attn_chunk_blocks = 0;     // 0 = default
    int sm_count = 0;
    cudaEvent_t ev_start = nullptr;     // stopwatch of b200_timer_start / b200_timer_stop
    cudaEvent_t ev_stop = nullptr;
};

struct b200_buf {
    b200_ctx* owner = nullptr;
    uint64_t generation = 0;
    void* ptr = nullptr;
    size_t bytes = 0;
};

namespace b200 {

// Records `msg` as this thread's last error and returns `st`.
int32_t fail(int32_t st, const std::string& msg);
// Same, for a failure after work may have been enqueued: also poisons the context.
int32_t fail_runtime(b200_ctx* ctx, int32_t st, const std::string& msg);
int32_t check_ctx(const b200_ctx* ctx);
// Marks the calling thread as the one capturing a CUDA graph on `ctx` (entry points called from other threads
// answer B200_DEVICE_CONTEXT_CAPTURE_IN_PROGRESS until the guard is destroyed).
struct CaptureGuard {
    b200_ctx* ctx;
    explicit CaptureGuard(b200_ctx* c);
    ~CaptureGuard();
};
// Validates that `buf` belongs to `ctx`, is of its generation and holds [off, off + need).
// A null `buf` is accepted only when `optional`.
int32_t check_buf(const b200_ctx* ctx, const b200_buf* buf, size_t off, size_t need, const char* name,
                  bool optional = false);
template <typename T>
inline T* buf_ptr(const b200_buf* b, size_t off) {
    return b ? reinterpret_cast<T*>(static_cast<uint8_t*>(b->ptr) + off) : nullptr;
}
// Grow-only scratch of the context (contents undefined).  Returns nullptr after recording an error.
void* ensure_ws(b200_ctx* ctx, size_t bytes);
int32_t set_device(const b200_ctx* ctx);
// Checked multiply for element counts; false on overflow or negative input.
bool mul_size(int64_t a, int64_t b, size_t elem, size_t* out);

}  // namespace b200
