// Shared definitions for libtsb's translation units: the context object,
// status/error plumbing, and thin wrappers over the sm_100a PTX this backend
// leans on (mbarrier, cp.async.bulk, programmatic dependent launch, mma.sync).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/tsb.h"

struct tsb_ctx {
    int device = 0;
    int sm_count = 148;
    std::string last_error;
    uint64_t launches = 0;
    // A small device area every kernel gets a pointer to (TsbDevState below).  Word 0 is the error word any kernel
    // may set instead of trapping: 0 = fine.  Read back by tsb_stream_sync.
    uint32_t* dev_error = nullptr;
    uint32_t* host_error = nullptr;  // pinned mirror
    uint32_t wait_limit_us = 1000000;
    // diagnostics of the fused matmul chain (tsb_debug_chain_trace): device buffer of nanosecond stamps
    unsigned long long* chain_trace = nullptr;
    size_t chain_trace_cap = 0, chain_trace_used = 0;  // in stamps / in launches  // bound of every device-side wait (mirrored in word 1 of the device area)
    bool pdl = true;                 // programmatic dependent launch between this ctx's kernels
};

// Layout of the device area behind tsb_ctx::dev_error (64 bytes, zeroed at creation).
//   word 0        error word (first writer wins)
//   word 1        bound of a device-side wait, in microseconds
constexpr size_t TSB_DEV_STATE_BYTES = 64;

// Error words kernels may write (first writer wins).
enum : uint32_t {
    TSB_DEV_OK = 0,
    TSB_DEV_BARRIER_TIMEOUT = 1,  // a bounded mbarrier wait gave up
    TSB_DEV_BAD_INDEX = 2,        // an index outside its table was skipped
    TSB_DEV_NONFINITE = 3,
};

inline int32_t tsb_fail(tsb_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        ctx->last_error = buf;
    }
    return code;
}

#define TSB_CUDA(ctx, expr)                                                                        \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return tsb_fail((ctx), TSB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                            __FILE__, __LINE__);                                                   \
    } while (0)

#define TSB_REQUIRE(ctx, cond, ...)                                   \
    do {                                                              \
        if (!(cond)) return tsb_fail((ctx), TSB_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// Binds the calling thread to the ctx's device for the scope of an entry point.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(const tsb_ctx* ctx) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != ctx->device) ok = cudaSetDevice(ctx->device) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// A kernel's opt-in to more than 48 KB of dynamic shared memory is a property of the (device, function) pair:
// `done` is the call site's table of devices already configured (one per kernel instantiation).  Two host
// threads racing here both set the same value, which is harmless.
constexpr int TSB_MAX_DEVICES = 64;
struct SmemOptIn {
    bool done[TSB_MAX_DEVICES] = {};
};
template <typename Kern>
inline cudaError_t tsb_opt_in_smem(const tsb_ctx* ctx, Kern kern, size_t bytes, SmemOptIn& table) {
    const int dev = ctx->device;
    if (dev >= 0 && dev < TSB_MAX_DEVICES && table.done[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && dev >= 0 && dev < TSB_MAX_DEVICES) table.done[dev] = true;
    return e;
}

// Launch helper: every kernel of this library goes through here so launches are
// counted and may carry the programmatic-dependent-launch attribute, which lets
// a kernel's weight prefetch overlap the tail of the kernel before it.  Kernels
// launched this way must execute griddepcontrol.wait before touching anything a
// predecessor wrote.
template <typename... KArgs, typename... Args>
inline cudaError_t tsb_launch_cluster(tsb_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, bool pdl, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl && ctx->pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {  // thread-block cluster: the CTAs of one cluster share distributed shared memory
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    ctx->launches++;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t tsb_launch(tsb_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, bool pdl, Args... args) {
    return tsb_launch_cluster(ctx, kernel, grid, block, smem, stream, pdl, 1u, args...);
}

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same with a suspend-time hint (nanoseconds): the thread sleeps in hardware until the phase completes or the
// hint runs out, instead of coming back after the short default limit and polling again.  A waiting warp then takes
// no issue slots from the warps it shares a scheduler with.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: bounded by time, not by polls.  The limit (microseconds) sits in the word after the error word;
// when it runs out the wait records why and returns false, so the caller can drain and leave and the context
// stays usable.  A failed poll sleeps up to 20 us in hardware; the clock is read only every 8 failed polls, so a
// wait that succeeds quickly never touches it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* err_word) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0, limit_ns = 0;
    for (uint32_t i = 1;; i++) {
#ifndef TSB_WAIT_HINT_NS
#define TSB_WAIT_HINT_NS 20000
#endif
        if (TSB_WAIT_HINT_NS ? mbar_try_wait_sleep(bar, parity, (uint32_t)TSB_WAIT_HINT_NS) : mbar_try_wait(bar, parity)) return true;
        if ((i & 7u) == 0) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                const uint32_t us = err_word ? *reinterpret_cast<volatile uint32_t*>(err_word + 1) : 0u;
                limit_ns = (unsigned long long)(us ? us : 1000000u) * 1000ull;
            } else if (now - t0 > limit_ns) {
                break;
            }
        }
    }
    if (err_word) atomicCAS(err_word, 0u, (uint32_t)TSB_DEV_BARRIER_TIMEOUT);
    return false;
}
// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// D(16x8,f32) += A(16x8,f16,row) * B(8x8,f16,col)
__device__ __forceinline__ void mma_1688(float (&d)[4], const uint32_t (&a)[2], uint32_t b) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(b));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

#endif  // __CUDACC__
