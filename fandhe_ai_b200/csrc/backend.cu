// C-ABI implementation, part 1: context, MemoryOps, quantisation API, quantized GEMM and
// the quantized linear.  Validation first, then enqueue; runtime failures poison the context
// (the reference's ordinal poison state machine, crates/backend-cuda/src/context_cache.rs:1-40).
#include "backend.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <new>
#include <thread>

#include "gemm_tc5.cuh"
#include "kernels.cuh"
#include "launch.cuh"

namespace b200 {

namespace {
thread_local std::string g_last_error;
std::atomic<uint64_t> g_generation{0};
}  // namespace

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int current_sm_count() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 1;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 1;
    }
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

int32_t fail(int32_t st, const std::string& msg) {
    g_last_error = msg;
    return st;
}
int32_t fail_runtime(b200_ctx* ctx, int32_t st, const std::string& msg) {
    if (ctx) ctx->poisoned = true;
    g_last_error = msg;
    return st;
}
namespace {
uint64_t this_thread_token() {
    const uint64_t h = static_cast<uint64_t>(std::hash<std::thread::id>()(std::this_thread::get_id()));
    return h | 1ull;      // never 0, which means "nobody"
}
}  // namespace

CaptureGuard::CaptureGuard(b200_ctx* c) : ctx(c) { ctx->capture_owner.store(this_thread_token()); }
CaptureGuard::~CaptureGuard() { ctx->capture_owner.store(0); }

// Entry gate of every call (begin_driver_call of the reference, crates/backend-cuda/src/context_cache.rs:1998):
// permanent states first, then the two transient ones, which do not poison anything.
int32_t check_ctx(const b200_ctx* ctx) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "context is null");
    if (ctx->unrecoverable)
        return fail(B200_DEVICE_CONTEXT_UNRECOVERABLE, "device context of ordinal " + std::to_string(ctx->ordinal) +
                                                           " could not be recovered (" + ctx->probe_error + "); restart the process");
    if (ctx->retiring.load())
        return fail(B200_DEVICE_CONTEXT_RETIRING, "device context of ordinal " + std::to_string(ctx->ordinal) +
                                                      " is being recovered; retry shortly");
    if (ctx->poisoned)
        return fail(B200_DEVICE_CONTEXT_POISONED,
                    "device context is poisoned by an earlier runtime failure; recover it (b200_ctx_recover) or re-create it");
    const uint64_t owner = ctx->capture_owner.load();
    if (owner != 0 && owner != this_thread_token())
        return fail(B200_DEVICE_CONTEXT_CAPTURE_IN_PROGRESS, "another thread is capturing a CUDA graph on ordinal " +
                                                                 std::to_string(ctx->ordinal) + "; retry shortly");
    return B200_OK;
}
int32_t check_buf(const b200_ctx* ctx, const b200_buf* buf, size_t off, size_t need, const char* name, bool optional) {
    if (!buf) {
        if (optional) return B200_OK;
        return fail(B200_INVALID_ARGUMENT, std::string(name) + ": buffer is null");
    }
    if (buf->owner != ctx) return fail(B200_DEVICE_MISMATCH, std::string(name) + ": buffer belongs to another context");
    if (buf->generation != ctx->generation) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "%s: stale buffer (ordinal %d, resource generation %llu, current %llu)", name,
                      ctx->ordinal, (unsigned long long)buf->generation, (unsigned long long)ctx->generation);
        return fail(B200_STALE_DEVICE_GENERATION, msg);
    }
    if (off > buf->bytes || need > buf->bytes - off) {
        char msg[200];
        std::snprintf(msg, sizeof msg, "%s: range [%zu, %zu + %zu) exceeds the buffer of %zu bytes", name, off, off, need,
                      buf->bytes);
        return fail(B200_SHAPE_MISMATCH, msg);
    }
    return B200_OK;
}
int32_t set_device(const b200_ctx* ctx) {
    cudaError_t e = cudaSetDevice(ctx->ordinal);
    if (e != cudaSuccess) return fail(B200_DEVICE_UNAVAILABLE, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    return B200_OK;
}
void* ensure_ws(b200_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->ws_bytes && ctx->ws) return ctx->ws;
    if (ctx->ws_locked) {
        fail(B200_UNSUPPORTED, "scratch cannot grow inside a composite call (split count too large for the reserved planes)");
        return nullptr;
    }
    size_t want = bytes + (bytes >> 2) + 4096;
    if (ctx->ws) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        fail(B200_DEVICE_ALLOCATION_FAILED, std::string("scratch allocation failed: ") + cudaGetErrorString(e));
        cudaGetLastError();
        return nullptr;
    }
    ctx->ws = p;
    ctx->ws_bytes = want;
    return p;
}
bool mul_size(int64_t a, int64_t b, size_t elem, size_t* out) {
    if (a < 0 || b < 0) return false;
    unsigned __int128 v = static_cast<unsigned __int128>(a) * static_cast<unsigned __int128>(b) * elem;
    if (v > static_cast<unsigned __int128>(SIZE_MAX / 2)) return false;
    *out = static_cast<size_t>(v);
    return true;
}

namespace {

int32_t check_error_word(b200_ctx* ctx, const char* where) {
    cudaError_t e = cudaMemcpyAsync(ctx->err_host, ctx->err_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess)
        return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string(where) + ": " + cudaGetErrorString(e));
    if (*ctx->err_host != 0) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "%s: a kernel reported device error 0x%x (bounded wait ran out or an index was out of range)",
                      where, *ctx->err_host);
        return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, msg);
    }
    return B200_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_last_error(void) { return g_last_error.c_str(); }

const char* b200_status_name(int32_t st) {
    switch (st) {
        case B200_OK: return "Ok";
        case B200_SHAPE_MISMATCH: return "ShapeMismatch";
        case B200_DEVICE_MISMATCH: return "DeviceMismatch";
        case B200_DEVICE_ALLOCATION_FAILED: return "DeviceAllocationFailed";
        case B200_KERNEL_LAUNCH_FAILED: return "KernelLaunchFailed";
        case B200_DEVICE_UNAVAILABLE: return "DeviceUnavailable";
        case B200_TRANSFER_FAILED: return "TransferFailed";
        case B200_UNSUPPORTED: return "Unsupported";
        case B200_STORE_POISONED: return "StorePoisoned";
        case B200_INVALID_ARGUMENT: return "InvalidArgument";
        case B200_DEVICE_CONTEXT_POISONED: return "DeviceContextPoisoned";
        case B200_STALE_DEVICE_GENERATION: return "StaleDeviceGeneration";
        case B200_DEVICE_CONTEXT_RETIRING: return "DeviceContextRetiring";
        case B200_DEVICE_CONTEXT_UNRECOVERABLE: return "DeviceContextUnrecoverable";
        case B200_DEVICE_CONTEXT_CAPTURE_IN_PROGRESS: return "DeviceContextCaptureInProgress";
        default: return "Unknown";
    }
}

int32_t b200_ctx_create(int32_t ordinal, b200_ctx** out) {
    if (!out) return fail(B200_INVALID_ARGUMENT, "ctx_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return fail(B200_DEVICE_UNAVAILABLE, "ctx_create: no CUDA device is visible (this backend has no CPU fallback)");
    }
    if (ordinal < 0 || ordinal >= count) return fail(B200_INVALID_ARGUMENT, "ctx_create: ordinal out of range");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, ordinal);
    if (e != cudaSuccess) return fail(B200_DEVICE_UNAVAILABLE, std::string("ctx_create: ") + cudaGetErrorString(e));
    if (prop.major != 10) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "ctx_create: device %d is sm_%d%d; the embedded kernels are sm_100a only", ordinal,
                      prop.major, prop.minor);
        return fail(B200_DEVICE_UNAVAILABLE, msg);
    }
    b200_ctx* ctx = new (std::nothrow) b200_ctx();
    if (!ctx) return fail(B200_DEVICE_ALLOCATION_FAILED, "ctx_create: host allocation failed");
    ctx->ordinal = ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->generation = ++g_generation;
    e = cudaSetDevice(ordinal);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->err_dev, 4 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->err_dev, 0, 4 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMallocHost(&ctx->err_host, sizeof(uint32_t));
    if (e != cudaSuccess) {
        std::string msg = std::string("ctx_create: ") + cudaGetErrorString(e);
        b200_ctx_destroy(ctx);
        return fail(B200_DEVICE_UNAVAILABLE, msg);
    }
    ctx->amax_scratch = ctx->err_dev + 1;
    ctx->attn_counter = ctx->err_dev + 2;
    ctx->quant_status = ctx->err_dev + 3;
    *ctx->err_host = 0;
    *out = ctx;
    return B200_OK;
}

int32_t b200_ctx_destroy(b200_ctx* ctx) {
    if (!ctx) return B200_OK;
    cudaSetDevice(ctx->ordinal);
    if (ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->err_dev) cudaFree(ctx->err_dev);
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    cudaGetLastError();
    delete ctx;
    return B200_OK;
}

int32_t b200_synchronize(b200_ctx* ctx) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = set_device(ctx)) return st;
    return check_error_word(ctx, "synchronize");
}

static __global__ void probe_identity_kernel(const uint32_t* in, uint32_t* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i];
}

// The recovery probe of the reference (256-byte allocation -> upload -> identity kernel -> download -> compare,
// crates/backend-cuda/src/context_cache.rs:2519).  Returns an empty string on success.
static std::string run_recovery_probe(b200_ctx* ctx) {
    if (ctx->inject_probe_failures > 0) {
        --ctx->inject_probe_failures;
        return "injected probe mismatch";
    }
    uint32_t host_in[64], host_out[64];
    for (int i = 0; i < 64; ++i) { host_in[i] = 0x9E3779B9u * (i + 1); host_out[i] = 0; }
    uint32_t* dev = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&dev), 512);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dev, host_in, 256, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        probe_identity_kernel<<<1, 64, 0, ctx->stream>>>(dev, dev + 64, 64);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_out, dev + 64, 256, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (dev) cudaFree(dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return std::string("probe failed: ") + cudaGetErrorString(e);
    }
    return std::memcmp(host_in, host_out, 256) == 0 ? std::string() : std::string("probe data mismatch");
}

// Recovery of a poisoned context in place (invalidate of the reference): drain, clear the device error word,
// probe, and start a new generation so that every buffer of the old one is refused as stale.
int32_t b200_ctx_recover(b200_ctx* ctx) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "ctx_recover: context is null");
    if (ctx->unrecoverable) return check_ctx(ctx);
    if (!ctx->poisoned) return B200_OK;
    if (ctx->retiring.exchange(true)) return fail(B200_DEVICE_CONTEXT_RETIRING, "ctx_recover: another thread is recovering this context");
    constexpr int kLimitProbeRetries = 3;
    std::string why;
    cudaError_t e = cudaSetDevice(ctx->ordinal);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->err_dev, 0, 4 * sizeof(uint32_t), ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        why = std::string("drain failed: ") + cudaGetErrorString(e);
        ctx->probe_failures = kLimitProbeRetries;          // a stream that cannot be drained is final
    } else {
        why = run_recovery_probe(ctx);
        ctx->probe_failures = why.empty() ? 0 : ctx->probe_failures + 1;
    }
    int32_t st = B200_OK;
    if (why.empty()) {
        ctx->generation = ++g_generation;
        ctx->poisoned = false;
        if (ctx->ws) { cudaFree(ctx->ws); ctx->ws = nullptr; ctx->ws_bytes = 0; }
        ctx->ws_locked = false;
    } else if (ctx->probe_failures >= kLimitProbeRetries) {
        ctx->unrecoverable = true;
        ctx->probe_error = why;
    } else {
        st = B200_DEVICE_CONTEXT_POISONED;
    }
    ctx->retiring.store(false);
    if (ctx->unrecoverable) return check_ctx(ctx);
    if (st != B200_OK) return fail(st, "ctx_recover: " + why + "; the context stays poisoned, recovery may be retried");
    return B200_OK;
}

int32_t b200_test_inject_probe_failures(b200_ctx* ctx, int32_t count) {
    if (!ctx || count < 0) return fail(B200_INVALID_ARGUMENT, "test_inject_probe_failures: bad argument");
    ctx->inject_probe_failures = count;
    return B200_OK;
}

int32_t b200_test_mark_capturing(b200_ctx* ctx, int32_t on) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "test_mark_capturing: context is null");
    ctx->capture_owner.store(on ? this_thread_token() : 0);
    return B200_OK;
}

int32_t b200_memory_info(b200_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
    if (!ctx || !free_bytes || !total_bytes) return fail(B200_INVALID_ARGUMENT, "memory_info: null pointer");
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = cudaMemGetInfo(free_bytes, total_bytes);
    if (e != cudaSuccess) return fail(B200_DEVICE_UNAVAILABLE, std::string("memory_info: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_test_poison(b200_ctx* ctx) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "test_poison: context is null");
    ctx->poisoned = true;
    return B200_OK;
}

int32_t b200_ctx_is_poisoned(const b200_ctx* ctx) { return ctx && (ctx->poisoned || ctx->unrecoverable) ? 1 : 0; }
uint64_t b200_ctx_generation(const b200_ctx* ctx) { return ctx ? ctx->generation : 0; }
void* b200_ctx_stream(b200_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }

int32_t b200_gemm_tuning(b200_ctx* ctx, int32_t tile_n, int32_t splits) {
    if (!ctx) return fail(B200_INVALID_ARGUMENT, "gemm_tuning: context is null");
    if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 224 && tile_n != 256)
        return fail(B200_INVALID_ARGUMENT, "gemm_tuning: tile_n must be 0 (heuristic), 64, 128, 224 or 256");
    if (splits < 0 || splits > 64) return fail(B200_INVALID_ARGUMENT, "gemm_tuning: splits must be in 0..64");
    ctx->tune_bn = tile_n;
    ctx->tune_splits = splits;
    return B200_OK;
}

/* ------------------------------------------------------------------ MemoryOps */

static int32_t new_buf(b200_ctx* ctx, size_t bytes, bool zero, b200_buf** out) {
    b200_buf* b = new (std::nothrow) b200_buf();
    if (!b) return fail(B200_DEVICE_ALLOCATION_FAILED, "host allocation of the buffer handle failed");
    b->owner = ctx;
    b->generation = ctx->generation;
    b->bytes = bytes;
    if (bytes > 0) {
        cudaError_t e = cudaMalloc(&b->ptr, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            delete b;
            char msg[160];
            std::snprintf(msg, sizeof msg, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
            return fail(B200_DEVICE_ALLOCATION_FAILED, msg);
        }
        if (zero) {
            e = cudaMemsetAsync(b->ptr, 0, bytes, ctx->stream);
            if (e != cudaSuccess) {
                cudaFree(b->ptr);
                delete b;
                return fail_runtime(ctx, B200_DEVICE_ALLOCATION_FAILED, std::string("memset failed: ") + cudaGetErrorString(e));
            }
        }
    }
    *out = b;
    return B200_OK;
}

int32_t b200_alloc_zeroed(b200_ctx* ctx, size_t bytes, b200_buf** out) {
    if (!out) return fail(B200_INVALID_ARGUMENT, "alloc_zeroed: out is null");
    *out = nullptr;
    if (int32_t st = check_ctx(ctx)) return st;
    if (bytes > 0)
        if (int32_t st = set_device(ctx)) return st;
    return new_buf(ctx, bytes, true, out);
}

int32_t b200_upload(b200_ctx* ctx, const void* host, size_t bytes, b200_buf** out) {
    if (!out) return fail(B200_INVALID_ARGUMENT, "upload: out is null");
    *out = nullptr;
    if (int32_t st = check_ctx(ctx)) return st;
    if (bytes > 0 && !host) return fail(B200_INVALID_ARGUMENT, "upload: host pointer is null");
    if (bytes > 0)
        if (int32_t st = set_device(ctx)) return st;
    b200_buf* b = nullptr;
    if (int32_t st = new_buf(ctx, bytes, false, &b)) return st;
    if (bytes > 0) {
        // Pageable source: the call returns once the host range has been staged, so the caller may reuse it.
        cudaError_t e = cudaMemcpyAsync(b->ptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) {
            cudaFree(b->ptr);
            delete b;
            return fail_runtime(ctx, B200_TRANSFER_FAILED, std::string("upload: ") + cudaGetErrorString(e));
        }
    }
    *out = b;
    return B200_OK;
}

int32_t b200_upload_into(b200_ctx* ctx, const void* host, size_t bytes, b200_buf* dst, size_t dst_offset) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = check_buf(ctx, dst, dst_offset, bytes, "upload_into dst")) return st;
    if (bytes == 0) return B200_OK;
    if (!host) return fail(B200_INVALID_ARGUMENT, "upload_into: host pointer is null");
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(dst->ptr) + dst_offset, host, bytes, cudaMemcpyHostToDevice,
                                    ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_TRANSFER_FAILED, std::string("upload_into: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_download(b200_ctx* ctx, const b200_buf* src, size_t src_offset, void* host, size_t bytes) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = check_buf(ctx, src, src_offset, bytes, "download src")) return st;
    if (bytes > 0 && !host) return fail(B200_INVALID_ARGUMENT, "download: host pointer is null");
    if (int32_t st = set_device(ctx)) return st;
    if (bytes > 0) {
        cudaError_t e = cudaMemcpyAsync(host, static_cast<const uint8_t*>(src->ptr) + src_offset, bytes,
                                        cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) return fail_runtime(ctx, B200_TRANSFER_FAILED, std::string("download: ") + cudaGetErrorString(e));
    }
    // The synchronisation point of a step; a deferred device-side failure surfaces here.
    return check_error_word(ctx, "download");
}

int32_t b200_release(b200_ctx* ctx, b200_buf* buf) {
    if (!buf) return B200_OK;
    if (!ctx || buf->owner != ctx) return fail(B200_DEVICE_MISMATCH, "release: buffer belongs to another context");
    if (buf->ptr) {
        cudaSetDevice(ctx->ordinal);
        cudaStreamSynchronize(ctx->stream);
        cudaFree(buf->ptr);
        cudaGetLastError();
    }
    delete buf;
    return B200_OK;
}

size_t b200_buf_bytes(const b200_buf* buf) { return buf ? buf->bytes : 0; }
void* b200_buf_device_ptr(const b200_buf* buf) { return buf ? buf->ptr : nullptr; }

/* ------------------------------------------------------------------ quantisation API */

int32_t b200_quantize_i8_per_row(b200_ctx* ctx, const b200_buf* x, size_t x_off, int64_t rows, int64_t cols,
                                 b200_buf* q, size_t q_off, b200_buf* scale, size_t scale_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    size_t xb, qb, sb;
    if (!mul_size(rows, cols, 4, &xb) || !mul_size(rows, cols, 1, &qb) || !mul_size(rows, 1, 4, &sb))
        return fail(B200_INVALID_ARGUMENT, "quantize_i8_per_row: rows/cols negative or overflowing");
    if (rows > 0x7FFFFFFF) return fail(B200_INVALID_ARGUMENT, "quantize_i8_per_row: rows exceed i32::MAX");
    if (int32_t st = check_buf(ctx, x, x_off, xb, "quantize_i8_per_row x")) return st;
    if (int32_t st = check_buf(ctx, q, q_off, qb, "quantize_i8_per_row q")) return st;
    if (int32_t st = check_buf(ctx, scale, scale_off, sb, "quantize_i8_per_row scale")) return st;
    if ((x_off & 15) || (q_off & 3) || (scale_off & 3))
        return fail(B200_INVALID_ARGUMENT, "quantize_i8_per_row: offsets must keep x 16-byte and q/scale 4-byte aligned");
    if (rows == 0 || cols == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = quantize_i8_per_row(buf_ptr<const float>(x, x_off), rows, cols, buf_ptr<int8_t>(q, q_off),
                                        buf_ptr<float>(scale, scale_off), ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("quantize_i8_per_row: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_dequantize_i8_per_row(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* scale,
                                   size_t scale_off, int64_t rows, int64_t cols, b200_buf* x, size_t x_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    size_t xb, qb, sb;
    if (!mul_size(rows, cols, 4, &xb) || !mul_size(rows, cols, 1, &qb) || !mul_size(rows, 1, 4, &sb))
        return fail(B200_INVALID_ARGUMENT, "dequantize_i8_per_row: rows/cols negative or overflowing");
    if (int32_t st = check_buf(ctx, q, q_off, qb, "dequantize_i8_per_row q")) return st;
    if (int32_t st = check_buf(ctx, scale, scale_off, sb, "dequantize_i8_per_row scale")) return st;
    if (int32_t st = check_buf(ctx, x, x_off, xb, "dequantize_i8_per_row x")) return st;
    if ((x_off & 3) || (scale_off & 3)) return fail(B200_INVALID_ARGUMENT, "dequantize_i8_per_row: misaligned offset");
    if (rows == 0 || cols == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = dequantize_i8_per_row(buf_ptr<const int8_t>(q, q_off), buf_ptr<const float>(scale, scale_off), rows,
                                          cols, buf_ptr<float>(x, x_off), ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("dequantize_i8_per_row: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_quantize_fp8_e4m3_per_tensor(b200_ctx* ctx, const b200_buf* x, size_t x_off, int64_t numel, b200_buf* q,
                                          size_t q_off, b200_buf* scale, size_t scale_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    size_t xb;
    if (!mul_size(numel, 1, 4, &xb)) return fail(B200_INVALID_ARGUMENT, "quantize_fp8: numel negative or overflowing");
    if (int32_t st = check_buf(ctx, x, x_off, xb, "quantize_fp8 x")) return st;
    if (int32_t st = check_buf(ctx, q, q_off, static_cast<size_t>(numel), "quantize_fp8 q")) return st;
    if (int32_t st = check_buf(ctx, scale, scale_off, 4, "quantize_fp8 scale")) return st;
    if ((x_off & 3) || (scale_off & 3)) return fail(B200_INVALID_ARGUMENT, "quantize_fp8: misaligned offset");
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = quantize_fp8_per_tensor(buf_ptr<const float>(x, x_off), numel, buf_ptr<uint8_t>(q, q_off),
                                            buf_ptr<float>(scale, scale_off), ctx->amax_scratch, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("quantize_fp8: ") + cudaGetErrorString(e));
    return B200_OK;
}

/* ------------------------------------------------------------------ GEMM */

static int32_t check_gemm_dims(const char* who, int64_t m, int64_t n, int64_t k) {
    if (m < 0 || n < 0 || k < 0) return fail(B200_INVALID_ARGUMENT, std::string(who) + ": negative dimension");
    if (m > 0x7FFFFFFF || n > 0x7FFFFFFF || k > 0x7FFFFFFF)
        return fail(B200_INVALID_ARGUMENT, std::string(who) + ": dimension exceeds i32::MAX");
    if (k % 16 != 0 || n % 16 != 0)
        return fail(B200_UNSUPPORTED, std::string(who) + ": n and k must be multiples of 16 (TMA strides); no fallback exists");
    return B200_OK;
}

int32_t b200_gemm_i8_s32(b200_ctx* ctx, const b200_buf* a, size_t a_off, const b200_buf* w, size_t w_off, int64_t m,
                         int64_t n, int64_t k, b200_buf* acc, size_t acc_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = check_gemm_dims("gemm_i8_s32", m, n, k)) return st;
    size_t ab, wb, cb;
    if (!mul_size(m, k, 1, &ab) || !mul_size(n, k, 1, &wb) || !mul_size(m, n, 4, &cb))
        return fail(B200_INVALID_ARGUMENT, "gemm_i8_s32: size overflow");
    if (int32_t st = check_buf(ctx, a, a_off, ab, "gemm_i8_s32 a")) return st;
    if (int32_t st = check_buf(ctx, w, w_off, wb, "gemm_i8_s32 w")) return st;
    if (int32_t st = check_buf(ctx, acc, acc_off, cb, "gemm_i8_s32 acc")) return st;
    if ((a_off & 15) || (w_off & 15) || (acc_off & 15))
        return fail(B200_INVALID_ARGUMENT, "gemm_i8_s32: offsets must be multiples of 16 bytes");
    if (m == 0 || n == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    if (k == 0) {
        cudaError_t e = cudaMemsetAsync(buf_ptr<uint8_t>(acc, acc_off), 0, cb, ctx->stream);
        if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, cudaGetErrorString(e));
        return B200_OK;
    }
    GemmPlan plan;
    const char* why = "";
    cudaError_t e = gemm_make_plan(&plan, kGemmI8, buf_ptr<const void>(a, a_off), buf_ptr<const void>(w, w_off), int(m),
                                   int(n), int(k), 0, ctx->tune_splits, ctx->tune_bn, &why);
    if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
    if (ctx->tune_splits == 0) gemm_plan_make_persistent(&plan, ctx->sm_count, false);
    GemmEpilogue ep;
    if (plan.out_planes == 1) {      // one pass over K, or split-K reduced inside a cluster
        ep.raw = buf_ptr<void>(acc, acc_off);
        e = gemm_launch(plan, ep, ctx->err_dev, ctx->stream);
    } else {
        void* ws = ensure_ws(ctx, gemm_raw_elems(plan) * 4);
        if (!ws) return B200_DEVICE_ALLOCATION_FAILED;
        ep.raw = ws;
        e = gemm_launch(plan, ep, ctx->err_dev, ctx->stream);
        if (e == cudaSuccess)
            e = gemm_sum_planes_i32(static_cast<const int*>(ws), plan.splits, int64_t(m) * n, buf_ptr<int>(acc, acc_off),
                                    ctx->stream);
    }
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("gemm_i8_s32: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_gemm_q8_scaled(b200_ctx* ctx, int32_t op_dtype, const b200_buf* a, size_t a_off, const b200_buf* a_scale,
                            size_t a_scale_off, int32_t a_scale_per_row, const b200_buf* w, size_t w_off,
                            const b200_buf* w_scale, size_t w_scale_off, int32_t w_scale_per_row, const b200_buf* bias,
                            size_t bias_off, int32_t activation, const b200_buf* residual, size_t residual_off, int64_t m,
                            int64_t n, int64_t k, int32_t out_dtype, b200_buf* out, size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (op_dtype != B200_I8 && op_dtype != B200_FP8_E4M3)
        return fail(B200_UNSUPPORTED, "gemm_q8_scaled: operand dtype must be I8 or FP8_E4M3");
    if (out_dtype != B200_F32 && out_dtype != B200_BF16)
        return fail(B200_UNSUPPORTED, "gemm_q8_scaled: output dtype must be F32 or BF16");
    if (activation < B200_ACT_NONE || activation > B200_ACT_SILU_GATE)
        return fail(B200_UNSUPPORTED, "gemm_q8_scaled: unknown activation");
    if (int32_t st = check_gemm_dims("gemm_q8_scaled", m, n, k)) return st;
    const bool gate = activation == B200_ACT_SILU_GATE;
    if (gate && (n % 32 != 0)) return fail(B200_UNSUPPORTED, "gemm_q8_scaled: gated n must be a multiple of 32");
    const int64_t n_out = gate ? n / 2 : n;
    const size_t osz = out_dtype == B200_F32 ? 4 : 2;
    size_t ab, wb, ob, rb, asb, wsb, bb;
    if (!mul_size(m, k, 1, &ab) || !mul_size(n, k, 1, &wb) || !mul_size(m, n_out, osz, &ob) ||
        !mul_size(m, n_out, 4, &rb) || !mul_size(a_scale_per_row ? m : 1, 1, 4, &asb) ||
        !mul_size(w_scale_per_row ? n : 1, 1, 4, &wsb) || !mul_size(n, 1, 4, &bb))
        return fail(B200_INVALID_ARGUMENT, "gemm_q8_scaled: size overflow");
    if (int32_t st = check_buf(ctx, a, a_off, ab, "gemm_q8_scaled a")) return st;
    if (int32_t st = check_buf(ctx, w, w_off, wb, "gemm_q8_scaled w")) return st;
    if (int32_t st = check_buf(ctx, a_scale, a_scale_off, asb, "gemm_q8_scaled a_scale")) return st;
    if (int32_t st = check_buf(ctx, w_scale, w_scale_off, wsb, "gemm_q8_scaled w_scale")) return st;
    if (int32_t st = check_buf(ctx, bias, bias_off, bias ? bb : 0, "gemm_q8_scaled bias", true)) return st;
    if (int32_t st = check_buf(ctx, residual, residual_off, residual ? rb : 0, "gemm_q8_scaled residual", true)) return st;
    if (int32_t st = check_buf(ctx, out, out_off, ob, "gemm_q8_scaled out")) return st;
    if ((a_off & 15) || (w_off & 15) || (out_off & 15) || (residual_off & 15) || (a_scale_off & 3) || (w_scale_off & 3) ||
        (bias_off & 3))
        return fail(B200_INVALID_ARGUMENT, "gemm_q8_scaled: misaligned offset (operands/out 16 bytes, scales/bias 4 bytes)");
    if (m == 0 || n == 0) return B200_OK;
    if (k == 0) return fail(B200_UNSUPPORTED, "gemm_q8_scaled: k == 0");
    if (int32_t st = set_device(ctx)) return st;

    const int kind = op_dtype == B200_I8 ? kGemmI8 : kGemmFp8;
    GemmEpilogue ep;
    ep.fused = 1;
    ep.a_scale = buf_ptr<const float>(a_scale, a_scale_off);
    ep.a_per_row = a_scale_per_row ? 1 : 0;
    ep.b_scale = buf_ptr<const float>(w_scale, w_scale_off);
    ep.b_per_col = w_scale_per_row ? 1 : 0;
    ep.bias = bias ? buf_ptr<const float>(bias, bias_off) : nullptr;
    ep.residual = residual ? buf_ptr<const float>(residual, residual_off) : nullptr;
    ep.out = buf_ptr<void>(out, out_off);
    ep.out_bf16 = out_dtype == B200_BF16;
    ep.act = activation;

    // First ask what a plain (ungated) plan would do: if the tile grid is too small it splits K,
    // and the row-wise finish applies the epilogue; otherwise the epilogue is fused into the GEMM.
    GemmPlan plan;
    const char* why = "";
    cudaError_t e;
    if (ctx->tune_splits == 0) {
        // default: the persistent kernel produces every epilogue (gated too) inside the GEMM launch
        e = gemm_make_plan(&plan, kind, buf_ptr<const void>(a, a_off), buf_ptr<const void>(w, w_off), int(m), int(n),
                           int(k), gate ? 1 : 0, 1, ctx->tune_bn, &why);
        if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
        gemm_plan_make_persistent(&plan, ctx->sm_count, true);
        if (plan.persist) {
            e = gemm_launch(plan, ep, ctx->err_dev, ctx->stream);
            if (e != cudaSuccess)
                return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("gemm_q8_scaled: ") + cudaGetErrorString(e));
            return B200_OK;
        }
    }
    e = gemm_make_plan(&plan, kind, buf_ptr<const void>(a, a_off), buf_ptr<const void>(w, w_off), int(m),
                       int(n), int(k), 0, ctx->tune_splits, ctx->tune_bn, &why);
    if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
    if (plan.splits > 1 && plan.cluster && !gate) {
        // split-K reduced inside a cluster: the epilogue runs on the reduced values in the same kernel
        e = gemm_launch(plan, ep, ctx->err_dev, ctx->stream);
    } else if (plan.splits > 1) {
        void* ws = ensure_ws(ctx, gemm_raw_elems(plan) * 4);
        if (!ws) return B200_DEVICE_ALLOCATION_FAILED;
        GemmEpilogue raw_ep;
        raw_ep.raw = ws;
        e = gemm_launch(plan, raw_ep, ctx->err_dev, ctx->stream);
        if (e == cudaSuccess)
            e = gemm_splitk_epilogue(kind, plan.out_planes, int(m), int(n), gate ? 1 : 0, ws, ep, ctx->stream);
    } else {
        if (gate) {
            e = gemm_make_plan(&plan, kind, buf_ptr<const void>(a, a_off), buf_ptr<const void>(w, w_off), int(m), int(n),
                               int(k), 1, 1, ctx->tune_bn, &why);
            if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
        }
        e = gemm_launch(plan, ep, ctx->err_dev, ctx->stream);
    }
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("gemm_q8_scaled: ") + cudaGetErrorString(e));
    return B200_OK;
}

// Which kernel form the two GEMM entry points above would use for a shape (nothing is launched).
int32_t b200_gemm_plan_info(b200_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t gated, int32_t fused, int32_t* out6) {
    if (!ctx || !out6) return fail(B200_INVALID_ARGUMENT, "gemm_plan_info: null pointer");
    if (int32_t st = check_gemm_dims("gemm_plan_info", m, n, k)) return st;
    if (m <= 0 || n <= 0 || k <= 0) return fail(B200_INVALID_ARGUMENT, "gemm_plan_info: m, n, k must be positive");
    if (int32_t st = set_device(ctx)) return st;
    GemmPlan plan;
    const char* why = "";
    const void* aligned = reinterpret_cast<const void*>(uintptr_t(256));     // never dereferenced, never encoded
    cudaError_t e;
    if (fused && ctx->tune_splits == 0) {
        e = gemm_make_plan(&plan, kGemmI8, aligned, aligned, int(m), int(n), int(k), gated ? 1 : 0, 1, ctx->tune_bn, &why, false);
        if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
        gemm_plan_make_persistent(&plan, ctx->sm_count, true);
    }
    if (!fused || !plan.persist) {
        e = gemm_make_plan(&plan, kGemmI8, aligned, aligned, int(m), int(n), int(k), 0, ctx->tune_splits, ctx->tune_bn, &why, false);
        if (e != cudaSuccess) return fail(B200_INVALID_ARGUMENT, why);
        if (!fused && ctx->tune_splits == 0) gemm_plan_make_persistent(&plan, ctx->sm_count, false);
    }
    const int v[6] = {plan.bn, plan.splits, plan.cluster, plan.persist ? (plan.pair ? 2 : 1) : 0, plan.persist ? plan.grid : 0, plan.stages};
    for (int i = 0; i < 6; ++i) out6[i] = v[i];
    return B200_OK;
}

// Where the time of one decode-shaped GEMM launch goes: runs the int8 GEMM of the shape the way b200_gemm_i8_s32
// (fused = 0) or the dequantising epilogue (fused = 1) would on the one-tile kernel, first `iters` launches back to
// back between two events (what a launch costs inside a stream of dependent launches), then ONE launch alone whose
// first CTA stamps %globaltimer at nine points of its life.  Operands are zero-filled device buffers.
int32_t b200_gemm_phase_stamps(b200_ctx* ctx, int64_t m, int64_t n, int64_t k, int32_t fused, int32_t iters, uint64_t* stamps_ns9,
                               float* loop_us_per_launch, float* alone_us, int32_t* info6) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (!stamps_ns9 || !loop_us_per_launch || !alone_us || !info6 || iters <= 0)
        return fail(B200_INVALID_ARGUMENT, "gemm_phase_stamps: bad argument");
    if (int32_t st = check_gemm_dims("gemm_phase_stamps", m, n, k)) return st;
    if (m <= 0 || n <= 0 || k <= 0) return fail(B200_INVALID_ARGUMENT, "gemm_phase_stamps: m, n, k must be positive");
    if (int32_t st = set_device(ctx)) return st;
    cudaStream_t s = ctx->stream;
    int8_t *a = nullptr, *b = nullptr;
    float* scales = nullptr;
    void* out = nullptr;
    unsigned long long* stamps = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    GemmPlan plan;
    const char* why = "";
    int32_t st = B200_OK;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&a), size_t(m) * k);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b), size_t(n) * k);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&scales), size_t(m + n) * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&stamps), kGemmStampCount * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemsetAsync(a, 0, size_t(m) * k, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(b, 0, size_t(n) * k, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(scales, 0, size_t(m + n) * sizeof(float), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(stamps, 0, kGemmStampCount * sizeof(unsigned long long), s);
    if (e == cudaSuccess) e = gemm_make_plan(&plan, kGemmI8, a, b, int(m), int(n), int(k), 0, ctx->tune_splits, ctx->tune_bn, &why);
    if (e == cudaSuccess && fused && !(plan.splits == 1 || plan.cluster)) {
        st = fail(B200_UNSUPPORTED, "gemm_phase_stamps: this shape has no fused epilogue in the one-tile kernel");
    } else if (e == cudaSuccess) {
        e = cudaMalloc(&out, gemm_raw_elems(plan) * 4);
        GemmEpilogue ep;
        ep.raw = out;
        if (fused) {
            ep.fused = 1;
            ep.a_scale = scales;
            ep.a_per_row = 1;
            ep.b_scale = scales + m;
            ep.b_per_col = 1;
            ep.out = out;
        }
        if (e == cudaSuccess) e = cudaEventCreate(&e0);
        if (e == cudaSuccess) e = cudaEventCreate(&e1);
        for (int i = 0; i < 3 && e == cudaSuccess; ++i) e = gemm_launch(plan, ep, ctx->err_dev, s);
        if (e == cudaSuccess) e = cudaEventRecord(e0, s);
        for (int i = 0; i < iters && e == cudaSuccess; ++i) e = gemm_launch(plan, ep, ctx->err_dev, s);
        if (e == cudaSuccess) e = cudaEventRecord(e1, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        float ms = 0.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        *loop_us_per_launch = ms * 1000.0f / float(iters);
        ep.stamps = stamps;
        if (e == cudaSuccess) e = cudaEventRecord(e0, s);
        if (e == cudaSuccess) e = gemm_launch(plan, ep, ctx->err_dev, s);
        if (e == cudaSuccess) e = cudaEventRecord(e1, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        *alone_us = ms * 1000.0f;
        unsigned long long host[kGemmStampCount] = {};
        if (e == cudaSuccess) e = cudaMemcpy(host, stamps, sizeof(host), cudaMemcpyDeviceToHost);
        for (int i = 0; i < kGemmStampCount; ++i) stamps_ns9[i] = host[i] >= host[0] ? host[i] - host[0] : 0;
        const int v[6] = {plan.bn, plan.splits, plan.cluster, 0, 0, plan.stages};
        for (int i = 0; i < 6; ++i) info6[i] = v[i];
    }
    if (e != cudaSuccess && st == B200_OK)
        st = fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("gemm_phase_stamps: ") + why + " " + cudaGetErrorString(e));
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(a);
    cudaFree(b);
    cudaFree(scales);
    cudaFree(out);
    cudaFree(stamps);
    if (st == B200_OK) st = b200_synchronize(ctx);
    return st;
}

/* ------------------------------------------------------------------ block-scale contract (QuantOps of the reference) */

static constexpr int64_t kBlockLen = 128;
static constexpr int64_t kKSafe = 133144;      // floor(i32::MAX / 127^2): longest chain of same-sign products that cannot wrap

int32_t b200_quantize_i8_block(b200_ctx* ctx, const b200_buf* x, size_t x_off, int64_t rows, int64_t cols, int64_t block_len,
                               int32_t scales_block_major, b200_buf* q, size_t q_off, b200_buf* delta, size_t delta_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (block_len <= 0) return fail(B200_INVALID_ARGUMENT, "quantize_i8_block: block length must be positive");
    if (block_len > kKSafe)
        return fail(B200_INVALID_ARGUMENT, "quantize_i8_block: block length " + std::to_string(block_len) +
                                               " exceeds K_safe = 133144 (an s32 accumulator over one block could wrap)");
    if (block_len != kBlockLen) return fail(B200_UNSUPPORTED, "quantize_i8_block: only blocks of 128 values are implemented");
    size_t xb, qb, db;
    const int64_t nb = cols > 0 ? (cols + kBlockLen - 1) / kBlockLen : 0;
    if (!mul_size(rows, cols, 4, &xb) || !mul_size(rows, cols, 1, &qb) || !mul_size(rows, nb, 4, &db))
        return fail(B200_INVALID_ARGUMENT, "quantize_i8_block: rows/cols negative or overflowing");
    if (int32_t st = check_buf(ctx, x, x_off, xb, "quantize_i8_block x")) return st;
    if (int32_t st = check_buf(ctx, q, q_off, qb, "quantize_i8_block q")) return st;
    if (int32_t st = check_buf(ctx, delta, delta_off, db, "quantize_i8_block delta")) return st;
    if ((x_off & 3) || (delta_off & 3)) return fail(B200_INVALID_ARGUMENT, "quantize_i8_block: misaligned offset");
    if (rows == 0 || cols == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = quantize_i8_block_pow2(buf_ptr<const float>(x, x_off), rows, cols, buf_ptr<int8_t>(q, q_off),
                                           buf_ptr<float>(delta, delta_off), scales_block_major ? 1 : 0, ctx->quant_status, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("quantize_i8_block: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_dequantize_i8_block(b200_ctx* ctx, const b200_buf* q, size_t q_off, const b200_buf* delta, size_t delta_off,
                                 int64_t rows, int64_t cols, int64_t block_len, int32_t scales_block_major, b200_buf* x,
                                 size_t x_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (block_len != kBlockLen) return fail(B200_UNSUPPORTED, "dequantize_i8_block: only blocks of 128 values are implemented");
    size_t xb, qb, db;
    const int64_t nb = cols > 0 ? (cols + kBlockLen - 1) / kBlockLen : 0;
    if (!mul_size(rows, cols, 4, &xb) || !mul_size(rows, cols, 1, &qb) || !mul_size(rows, nb, 4, &db))
        return fail(B200_INVALID_ARGUMENT, "dequantize_i8_block: rows/cols negative or overflowing");
    if (int32_t st = check_buf(ctx, q, q_off, qb, "dequantize_i8_block q")) return st;
    if (int32_t st = check_buf(ctx, delta, delta_off, db, "dequantize_i8_block delta")) return st;
    if (int32_t st = check_buf(ctx, x, x_off, xb, "dequantize_i8_block x")) return st;
    if ((x_off & 3) || (delta_off & 3)) return fail(B200_INVALID_ARGUMENT, "dequantize_i8_block: misaligned offset");
    if (rows == 0 || cols == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    cudaError_t e = dequantize_i8_block(buf_ptr<const int8_t>(q, q_off), buf_ptr<const float>(delta, delta_off), rows, cols,
                                        scales_block_major ? 1 : 0, buf_ptr<float>(x, x_off), ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("dequantize_i8_block: ") + cudaGetErrorString(e));
    return B200_OK;
}

int32_t b200_gemm_i8_block_scaled(b200_ctx* ctx, const b200_buf* a, size_t a_off, const b200_buf* a_delta, size_t a_delta_off,
                                  const b200_buf* w, size_t w_off, const b200_buf* w_delta, size_t w_delta_off, int64_t m,
                                  int64_t n, int64_t k, int64_t block_len, b200_buf* out, size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (block_len <= 0) return fail(B200_INVALID_ARGUMENT, "gemm_i8_block_scaled: block length must be positive");
    if (block_len > kKSafe)
        return fail(B200_INVALID_ARGUMENT, "gemm_i8_block_scaled: block length " + std::to_string(block_len) +
                                               " exceeds K_safe = 133144 (the s32 accumulator of one block could wrap)");
    if (block_len != kBlockLen) return fail(B200_UNSUPPORTED, "gemm_i8_block_scaled: only blocks of 128 values are implemented");
    if (int32_t st = check_gemm_dims("gemm_i8_block_scaled", m, n, k)) return st;
    const int64_t nb = k > 0 ? (k + kBlockLen - 1) / kBlockLen : 0;
    size_t ab, wb, cb, adb, wdb;
    if (!mul_size(m, k, 1, &ab) || !mul_size(n, k, 1, &wb) || !mul_size(m, n, 4, &cb) || !mul_size(m, nb, 4, &adb) ||
        !mul_size(n, nb, 4, &wdb))
        return fail(B200_INVALID_ARGUMENT, "gemm_i8_block_scaled: size overflow");
    if (int32_t st = check_buf(ctx, a, a_off, ab, "gemm_i8_block_scaled a")) return st;
    if (int32_t st = check_buf(ctx, a_delta, a_delta_off, adb, "gemm_i8_block_scaled a_delta")) return st;
    if (int32_t st = check_buf(ctx, w, w_off, wb, "gemm_i8_block_scaled w")) return st;
    if (int32_t st = check_buf(ctx, w_delta, w_delta_off, wdb, "gemm_i8_block_scaled w_delta")) return st;
    if (int32_t st = check_buf(ctx, out, out_off, cb, "gemm_i8_block_scaled out")) return st;
    if ((a_off & 15) || (w_off & 15) || (out_off & 15) || (a_delta_off & 3) || (w_delta_off & 3))
        return fail(B200_INVALID_ARGUMENT, "gemm_i8_block_scaled: misaligned offset (operands/out 16 bytes, scales 4 bytes)");
    if (m == 0 || n == 0) return B200_OK;
    if (int32_t st = set_device(ctx)) return st;
    if (k == 0) {
        cudaError_t e = cudaMemsetAsync(buf_ptr<uint8_t>(out, out_off), 0, cb, ctx->stream);
        if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, cudaGetErrorString(e));
        return B200_OK;
    }
    const char* why = "";
    cudaError_t e = gemm_i8_block_scaled(buf_ptr<const void>(a, a_off), buf_ptr<const float>(a_delta, a_delta_off),
                                         buf_ptr<const void>(w, w_off), buf_ptr<const float>(w_delta, w_delta_off), int(m), int(n),
                                         int(k), buf_ptr<float>(out, out_off), ctx->quant_status, ctx->err_dev, ctx->stream, &why);
    if (e == cudaErrorInvalidValue && why[0]) return fail(B200_INVALID_ARGUMENT, why);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("gemm_i8_block_scaled: ") + cudaGetErrorString(e));
    return B200_OK;
}

// Waits for the stream and reports (and clears) what the block-scale kernels flagged since the last check.  A flagged
// request was outside the contract, not a device failure: nothing is poisoned.
int32_t b200_quant_check(b200_ctx* ctx) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = set_device(ctx)) return st;
    uint32_t word = 0;
    cudaError_t e = cudaMemcpyAsync(ctx->err_host, ctx->quant_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) {
        word = *ctx->err_host;
        *ctx->err_host = 0;
        e = cudaMemsetAsync(ctx->quant_status, 0, sizeof(uint32_t), ctx->stream);
    }
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("quant_check: ") + cudaGetErrorString(e));
    if (int32_t st = check_error_word(ctx, "quant_check")) return st;
    if (word & 1u) return fail(B200_INVALID_ARGUMENT, "quant_check: an input of the block quantiser was not finite (NaN or infinity); its block was zeroed");
    if (word & 2u) return fail(B200_INVALID_ARGUMENT, "quant_check: a result of the block-scaled GEMM overflowed f32 when the f64 sum over the blocks was narrowed");
    return B200_OK;
}

/* ------------------------------------------------------------------ quantized linear */

int32_t b200_linear_w8a8(b200_ctx* ctx, const b200_buf* a, size_t a_off, int64_t m, int64_t k, const b200_buf* w,
                         size_t w_off, const b200_buf* w_scale, size_t w_scale_off, const b200_buf* bias, size_t bias_off,
                         int64_t n, int32_t activation, const b200_buf* residual, size_t residual_off, b200_buf* out,
                         size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    // Shape checks come before any capability answer (crates/tensor-core/src/low_precision.rs:201-224).
    if (int32_t st = check_gemm_dims("linear_w8a8", m, n, k)) return st;
    if (activation < B200_ACT_NONE || activation > B200_ACT_SILU_GATE)
        return fail(B200_UNSUPPORTED, "linear_w8a8: unknown activation");
    size_t ab;
    if (!mul_size(m, k, 4, &ab)) return fail(B200_INVALID_ARGUMENT, "linear_w8a8: size overflow");
    if (int32_t st = check_buf(ctx, a, a_off, ab, "linear_w8a8 a")) return st;
    if (a_off & 15) return fail(B200_INVALID_ARGUMENT, "linear_w8a8: a offset must be a multiple of 16 bytes");
    if (m == 0 || n == 0) return B200_OK;
    if (k == 0) return fail(B200_UNSUPPORTED, "linear_w8a8: k == 0");
    if (int32_t st = set_device(ctx)) return st;
    // Scratch: [xq m*k int8][sx m f32][split planes].  The GEMM entry may grow the scratch, so size it for
    // the worst case up front and hand out sub-ranges through a temporary handle.
    const size_t xq_bytes = align_up(size_t(m) * size_t(k), 256);
    const size_t sx_bytes = align_up(size_t(m) * 4, 256);
    const size_t max_planes = ctx->tune_splits > 16 ? size_t(ctx->tune_splits) : 16;
    const size_t plane_bytes = align_up(size_t(m) * size_t(n) * 4 * max_planes, 256);
    uint8_t* ws = static_cast<uint8_t*>(ensure_ws(ctx, xq_bytes + sx_bytes + plane_bytes));
    if (!ws) return B200_DEVICE_ALLOCATION_FAILED;
    cudaError_t e = quantize_i8_per_row(buf_ptr<const float>(a, a_off), m, k, reinterpret_cast<int8_t*>(ws),
                                        reinterpret_cast<float*>(ws + xq_bytes), ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("linear_w8a8 quantize: ") + cudaGetErrorString(e));
    // View the scratch as a buffer of this context so the GEMM entry can validate it like any other.
    b200_buf scratch;
    scratch.owner = ctx;
    scratch.generation = ctx->generation;
    scratch.ptr = ws;
    scratch.bytes = xq_bytes + sx_bytes;
    // Keep the GEMM's own scratch (split planes) behind the activations: temporarily offset ctx->ws.
    void* saved_ws = ctx->ws;
    size_t saved_bytes = ctx->ws_bytes;
    ctx->ws = ws + xq_bytes + sx_bytes;
    ctx->ws_bytes = saved_bytes - (xq_bytes + sx_bytes);
    ctx->ws_locked = true;
    int32_t st = b200_gemm_q8_scaled(ctx, B200_I8, &scratch, 0, &scratch, xq_bytes, 1, w, w_off, w_scale, w_scale_off, 1, bias,
                                     bias_off, activation, residual, residual_off, m, n, k, B200_F32, out, out_off);
    ctx->ws = saved_ws;
    ctx->ws_bytes = saved_bytes;
    ctx->ws_locked = false;
    return st;
}


int32_t b200_linear_fp8(b200_ctx* ctx, const b200_buf* a, size_t a_off, int64_t m, int64_t k, const b200_buf* w,
                        size_t w_off, const b200_buf* w_scale, size_t w_scale_off, const b200_buf* bias, size_t bias_off,
                        int64_t n, int32_t activation, const b200_buf* residual, size_t residual_off, int32_t out_dtype,
                        b200_buf* out, size_t out_off) {
    if (int32_t st = check_ctx(ctx)) return st;
    if (int32_t st = check_gemm_dims("linear_fp8", m, n, k)) return st;
    if (activation < B200_ACT_NONE || activation > B200_ACT_SILU_GATE)
        return fail(B200_UNSUPPORTED, "linear_fp8: unknown activation");
    size_t ab;
    if (!mul_size(m, k, 4, &ab)) return fail(B200_INVALID_ARGUMENT, "linear_fp8: size overflow");
    if (int32_t st = check_buf(ctx, a, a_off, ab, "linear_fp8 a")) return st;
    if (a_off & 15) return fail(B200_INVALID_ARGUMENT, "linear_fp8: a offset must be a multiple of 16 bytes");
    if (m == 0 || n == 0) return B200_OK;
    if (k == 0) return fail(B200_UNSUPPORTED, "linear_fp8: k == 0");
    if (int32_t st = set_device(ctx)) return st;
    // Scratch: [a as E4M3, m*k bytes][its scale, one f32][split planes of the GEMM entry behind them].
    const size_t aq_bytes = align_up(size_t(m) * size_t(k), 256);
    const size_t sa_bytes = 256;
    const size_t max_planes = ctx->tune_splits > 16 ? size_t(ctx->tune_splits) : 16;
    const size_t plane_bytes = align_up(size_t(m) * size_t(n) * 4 * max_planes, 256);
    uint8_t* ws = static_cast<uint8_t*>(ensure_ws(ctx, aq_bytes + sa_bytes + plane_bytes));
    if (!ws) return B200_DEVICE_ALLOCATION_FAILED;
    cudaError_t e = quantize_fp8_per_tensor(buf_ptr<const float>(a, a_off), m * k, ws, reinterpret_cast<float*>(ws + aq_bytes),
                                            ctx->amax_scratch, ctx->stream);
    if (e != cudaSuccess) return fail_runtime(ctx, B200_KERNEL_LAUNCH_FAILED, std::string("linear_fp8 quantize: ") + cudaGetErrorString(e));
    b200_buf scratch;
    scratch.owner = ctx;
    scratch.generation = ctx->generation;
    scratch.ptr = ws;
    scratch.bytes = aq_bytes + sa_bytes;
    void* saved_ws = ctx->ws;
    size_t saved_bytes = ctx->ws_bytes;
    ctx->ws = ws + aq_bytes + sa_bytes;
    ctx->ws_bytes = saved_bytes - (aq_bytes + sa_bytes);
    ctx->ws_locked = true;
    int32_t st = b200_gemm_q8_scaled(ctx, B200_FP8_E4M3, &scratch, 0, &scratch, aq_bytes, 0, w, w_off, w_scale, w_scale_off, 0,
                                     bias, bias_off, activation, residual, residual_off, m, n, k, out_dtype, out, out_off);
    ctx->ws = saved_ws;
    ctx->ws_bytes = saved_bytes;
    ctx->ws_locked = false;
    return st;
}

}  // extern "C"
