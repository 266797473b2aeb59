// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, every
// copy lands in the issuing CTA only), tcgen05 (TMEM alloc / MMA / commit / ld) and a few
// memory-ordering helpers.  Every wait in this file is bounded: a wait that runs
// out records a code in a device error word and returns false so the kernel can
// unwind (free TMEM, leave) instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Number of failed polls after which a wait gives up.  One failed
// mbarrier.try_wait already blocks for a hardware-defined slice, so this is on
// the order of a second, far above any healthy wait in these kernels.
constexpr uint32_t kSpinLimit = 1u << 22;

// Error codes written to the context's device error word by kernels.
enum DeviceErr : uint32_t {
    kErrNone = 0,
    kErrProducerWait = 0x101,   // TMA producer waited too long for a free stage
    kErrMmaWait = 0x102,        // MMA issuer waited too long for a filled stage
    kErrEpilogueWait = 0x103,   // epilogue waited too long for the accumulator
    kErrAttnLoadWait = 0x201,   // attention consumer waited too long for a KV tile
    kErrAttnBlockId = 0x202,    // attention met a block id >= num_blocks in a used slot
    kErrAppendSlot = 0x203,     // append met a slot >= pool rows
    kErrAttnSeqLen = 0x204,     // attention met a sequence length beyond the table width or the planned maximum
    kErrPeerWait = 0x301,       // cross-GPU flag wait ran out
    kErrPeerFailed = 0x302,     // a peer GPU reported that its own wait ran out (poisoned flag)
    kErrTokenId = 0x401,        // embedding gather met an id outside the vocabulary
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in the
// stream still runs.  pdl_wait() returns once the predecessor has completed and its writes are visible;
// everything before it must touch neither the predecessor's outputs nor buffers the predecessor still reads.
// pdl_launch_dependents() lets the successor's CTAs be scheduled from here on.  Both are no-ops for a
// kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Orders earlier generic-proxy accesses (here: the acquire of a flag another GPU raised) before later
// asynchronous-proxy accesses (TMA loads of the rows that flag announces), for global memory too.
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}
// TMA store of one box from shared memory (written by ordinary stores, then fence_proxy_async) to the tensor at
// (x, y); parts of the box outside the tensor are dropped.  Stores are tracked in bulk groups of the issuing thread.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src_smem, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tmap), "r"(src_smem), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every earlier bulk group of this thread has finished READING its shared memory (the buffer may be rewritten)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// every earlier bulk group of this thread is complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after recording `code`) when the limit is hit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t* err, uint32_t code) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (err) atomicCAS(err, 0u, code);
    return false;
}

// ---------------------------------------------------------------- TMA (tile mode, one CTA)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// The innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Asks L2 for a tile without bringing it into shared memory (same coordinate rules as the loads).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int x, int y, int z) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc5_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc5_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when all tcgen05.mma issued so far by this thread are done.
__device__ __forceinline__ void tc5_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2k and 2k + 1) work on one 256-row accumulator tile: each holds 128 rows of A, half of
// the B rows and, in its own tensor memory, the accumulator rows of its A rows.  The even CTA (the leader) issues the
// MMAs for both.  None of the loads below is a multicast load: every CTA fetches its own operand halves.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrival on an mbarrier of another CTA of the cluster (`bar` is a shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// TMA tile load whose completion is counted on an mbarrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives once, on the mbarrier at the same shared-memory offset in every CTA of `cta_mask`, when all tcgen05.mma
// issued so far by this thread are done.
__device__ __forceinline__ void tc5_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}
template <bool kInt8>
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kInt8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128
// bytes wide and stored with the 128-byte swizzle (the layout TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                       // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
    return d;
}

// Instruction descriptor, dense, both operands K-major, M x N tile.
//   kind::i8      : a/b format 1 = signed 8-bit, accumulator format 2 = s32
//   kind::f8f6f4  : a/b format 0 = e4m3,         accumulator format 1 = f32
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t ab_format, uint32_t c_format, uint32_t m, uint32_t n) {
    return (c_format << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

template <bool kInt8>
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    if constexpr (kInt8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row
// (lane base + i), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- numerics shared by kernels
// e^x from correctly rounded operations only (multiply, fused multiply-add, add, round-to-integer, exponent
// bit arithmetic), so that a CPU restatement written with the same operations returns the same bits; the libm
// and CUDA expf differ from each other in the last place.  Argument reduction x = n ln2 + r with ln2 split in
// two constants, a degree-5 polynomial in r on top of 1 + r (the classic single-precision minimax set), and
// the scaling by 2^n as two exact-or-once-rounded multiplications (covers denormal results).  About 1 ulp.
__device__ __forceinline__ float exp_det(float x) {
    if (!(x > -104.0f)) return x != x ? x : 0.0f;
    if (x > 88.8f) return __int_as_float(0x7F800000);
    const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693359375f, x);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float y = __fadd_rn(__fmaf_rn(p, __fmul_rn(r, r), r), 1.0f);
    const int ni = static_cast<int>(n);
    const int a = (ni - (ni & 1)) / 2, b = ni - a;
    y = __fmul_rn(y, __int_as_float((a + 127) << 23));
    return __fmul_rn(y, __int_as_float((b + 127) << 23));
}

// Two-branch sigmoid (never exponentiates a positive argument): 1 / (1 + e^-x) for x >= 0, e^x / (1 + e^x) below.
// Written without a branch - both forms exponentiate -|x| - so that a warp whose lanes differ in sign evaluates one
// exponential and one division per value instead of both paths; the results are those of the two-branch form bit for bit.
__device__ __forceinline__ float sigmoid_stable(float x) {
    const float e = exp_det(-fabsf(x));
    return __fdiv_rn(x >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
}
__device__ __forceinline__ float silu(float x) { return __fmul_rn(x, sigmoid_stable(x)); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// Round-to-nearest-even f32 -> bf16 bits; NaN stays NaN (quiet), overflow goes to inf.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x40u;
    u += 0x7FFFu + ((u >> 16) & 1u);
    return u >> 16;
}

// ---------------------------------------------------------------- system-scope accesses (memory of another GPU)
__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
// 16-byte load that is not served from this SM's L1 (the line may have been rewritten by its owner GPU)
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* addr) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(addr) : "memory");
    return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");      // not to be moved across barriers or memory accesses
    return t;
}

// Flags that one GPU raises in another GPU's memory are epoch counters: the waiting side polls its own memory
// until the flag has reached `epoch` (difference taken modulo 2^32).  Every such wait is bounded by time; a
// rank that gives up writes kPeerPoison into the flags it owns at its peers, so that they stop at once with
// an error of their own instead of consuming rows that were never delivered.
constexpr uint32_t kPeerPoison = 0xFFFFFFFFu;
constexpr uint64_t kPeerWaitNs = 2000000000ull;      // default bound of a cross-GPU wait: two seconds

__device__ __forceinline__ bool wait_peer_flag(const uint32_t* flag, uint32_t epoch, uint32_t* err, uint64_t timeout_ns) {
    if (timeout_ns == 0) timeout_ns = kPeerWaitNs;      // "no bound given" means the default bound, never "no patience"
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        const uint32_t v = ld_acquire_sys(flag);
        if (v == kPeerPoison) {
            atomicCAS(err, 0u, static_cast<uint32_t>(kErrPeerFailed));
            return false;
        }
        if (static_cast<int32_t>(v - epoch) >= 0) return true;
        if ((it & 63u) == 63u && global_timer_ns() - t0 > timeout_ns) break;
    }
    atomicCAS(err, 0u, static_cast<uint32_t>(kErrPeerWait));
    return false;
}

// A count that other GPUs raise in this GPU's memory with red_release_sys_add (one per finished piece of work): the
// wait ends when it has reached `target` (difference modulo 2^32, so the count may wrap).  A count passes through
// every value, so the poison travels in a word of its own: `poison` is a flag word of the same sender.
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ bool wait_peer_count(const uint32_t* count, uint32_t target, const uint32_t* poison, uint32_t* err,
                                                uint64_t timeout_ns) {
    if (timeout_ns == 0) timeout_ns = kPeerWaitNs;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        const uint32_t v = ld_acquire_sys(count);
        if (static_cast<int32_t>(v - target) >= 0) return true;
        if ((it & 15u) == 15u && ld_acquire_sys(poison) == kPeerPoison) {
            atomicCAS(err, 0u, static_cast<uint32_t>(kErrPeerFailed));
            return false;
        }
        if ((it & 63u) == 63u && global_timer_ns() - t0 > timeout_ns) break;
    }
    atomicCAS(err, 0u, static_cast<uint32_t>(kErrPeerWait));
    return false;
}

// Symmetric int8 quantisation of one value: round-to-nearest-even of x / scale, clamped to [-127, 127];
// scale 0 (an all-zero row) gives 0.
__device__ __forceinline__ int quant_i8(float x, float scale) {
    if (scale == 0.0f) return 0;
    float r = rintf(x / scale);
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return static_cast<int>(r);
}

// ---- FP8 (E4M3) activations: per-token scale amax / 448, codes = e4m3(x / scale) rounded to nearest even, saturating.
constexpr float kE4m3Max = 448.0f;
// Two f32 -> two e4m3 codes (first value in the low byte).
__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t quant4_e4m3(float x0, float x1, float x2, float x3, float scale) {
    if (scale == 0.0f) return 0u;
    return e4m3x2(x0 / scale, x1 / scale) | (e4m3x2(x2 / scale, x3 / scale) << 16);
}
// A finished accumulator word as f32: an int32 sum (INT8 operands) or the bits of an f32 sum (FP8 operands).
__device__ __forceinline__ float acc_word_f32(int v, int fp8) { return fp8 ? __int_as_float(v) : static_cast<float>(v); }

}  // namespace b200
