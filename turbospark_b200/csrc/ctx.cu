// Context, memory and stream entry points of the C ABI.
#include <cstring>
#include <new>

#include "common.cuh"

extern "C" {

int32_t tsb_ctx_create(int32_t device_ordinal, tsb_ctx** out) {
    if (!out) return TSB_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return TSB_ERR_CUDA;  // no CPU fallback: fail loudly
    if (device_ordinal < 0 || device_ordinal >= count) return TSB_ERR_INVALID;
    tsb_ctx* ctx = new (std::nothrow) tsb_ctx();
    if (!ctx) return TSB_ERR_OOM;
    ctx->device = device_ordinal;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device_ordinal);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device_ordinal);
    if (e == cudaSuccess && prop.major < 10) {
        delete ctx;
        if (prev >= 0) cudaSetDevice(prev);
        return TSB_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
    }
    if (e == cudaSuccess) {
        ctx->sm_count = prop.multiProcessorCount;
        e = cudaMalloc((void**)&ctx->dev_error, TSB_DEV_STATE_BYTES);
    }
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_error, 0, TSB_DEV_STATE_BYTES);
    if (e == cudaSuccess) e = cudaMemcpy(ctx->dev_error + 1, &ctx->wait_limit_us, sizeof(uint32_t), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMallocHost((void**)&ctx->host_error, sizeof(uint32_t));
    if (prev >= 0) cudaSetDevice(prev);
    if (e != cudaSuccess) {
        delete ctx;
        return TSB_ERR_CUDA;
    }
    const char* env = getenv("TSB_PDL");
    if (env && env[0] == '0') ctx->pdl = false;
    *out = ctx;
    return TSB_OK;
}

void tsb_ctx_destroy(tsb_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard g(ctx);
    cudaDeviceSynchronize();
    if (ctx->dev_error) cudaFree(ctx->dev_error);
    if (ctx->host_error) cudaFreeHost(ctx->host_error);
    delete ctx;
}

const char* tsb_last_error(const tsb_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null ctx"; }
int32_t tsb_device_ordinal(const tsb_ctx* ctx) { return ctx ? ctx->device : -1; }
uint64_t tsb_launch_count(const tsb_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t tsb_alloc(tsb_ctx* ctx, size_t bytes, void** out_dev) {
    if (!ctx || !out_dev) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    *out_dev = nullptr;
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMalloc(out_dev, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return tsb_fail(ctx, TSB_ERR_OOM, "device allocation of %zu bytes failed", bytes);
    }
    TSB_CUDA(ctx, e);
    return TSB_OK;
}

int32_t tsb_free(tsb_ctx* ctx, void* dev) {
    if (!ctx) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaFree(dev));
    return TSB_OK;
}

int32_t tsb_weights_upload(tsb_ctx* ctx, const void* host_bytes, size_t bytes, void** out_dev_region) {
    if (!ctx || !host_bytes || !out_dev_region) return TSB_ERR_INVALID;
    // 256 spare bytes: the bulk-copy path may over-fetch up to one 16-byte
    // granule past an unaligned row run, which must stay inside the allocation.
    int32_t rc = tsb_alloc(ctx, bytes + 256, out_dev_region);
    if (rc) return rc;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaMemcpy(*out_dev_region, host_bytes, bytes, cudaMemcpyHostToDevice));
    TSB_CUDA(ctx, cudaMemset((char*)*out_dev_region + bytes, 0, 256));
    return TSB_OK;
}

int32_t tsb_memcpy_h2d(tsb_ctx* ctx, tsb_stream s, void* dev, const void* host, size_t bytes) {
    if (!ctx || (!dev && bytes) || (!host && bytes)) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)s));
    return TSB_OK;
}

int32_t tsb_memcpy_d2h(tsb_ctx* ctx, tsb_stream s, void* host, const void* dev, size_t bytes) {
    if (!ctx || (!dev && bytes) || (!host && bytes)) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    return TSB_OK;
}

int32_t tsb_stream_sync(tsb_ctx* ctx, tsb_stream s) {
    if (!ctx) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaMemcpyAsync(ctx->host_error, ctx->dev_error, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)s));
    TSB_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)s));
    uint32_t w = *ctx->host_error;
    if (w != TSB_DEV_OK) {
        cudaMemsetAsync(ctx->dev_error, 0, sizeof(uint32_t), (cudaStream_t)s);
        return tsb_fail(ctx, TSB_ERR_DEVICE, "a kernel reported error word %u (%s)", w,
                        w == TSB_DEV_BARRIER_TIMEOUT ? "bounded barrier wait gave up"
                        : w == TSB_DEV_BAD_INDEX     ? "index outside its table"
                                                     : "non-finite value");
    }
    return TSB_OK;
}

int32_t tsb_ctx_set_wait_limit_us(tsb_ctx* ctx, uint32_t microseconds) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, microseconds >= 1, "the limit must be at least one microsecond");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, cudaDeviceSynchronize());
    ctx->wait_limit_us = microseconds;
    TSB_CUDA(ctx, cudaMemcpy(ctx->dev_error + 1, &ctx->wait_limit_us, sizeof(uint32_t), cudaMemcpyHostToDevice));
    return TSB_OK;
}

namespace {
// One CTA waits on an mbarrier nobody arrives on; the bounded wait must give up, record why and return.
__global__ void wait_nobody_kernel(uint32_t* err, uint32_t* waited_ok) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) *waited_ok = mbar_wait(&bar, 0, err) ? 1u : 0u;
}
}  // namespace

int32_t tsb_debug_wait_nobody(tsb_ctx* ctx, tsb_stream s, void* out_u32_dev) {
    if (!ctx || !out_u32_dev) return TSB_ERR_INVALID;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, tsb_launch(ctx, wait_nobody_kernel, dim3(1), dim3(32), 0, (cudaStream_t)s, false, ctx->dev_error, (uint32_t*)out_u32_dev));
    return TSB_OK;
}

int64_t tsb_row_bytes(int32_t qtype, int64_t cols) {
    switch (qtype) {
        case TSB_Q4_K: return cols / 256 * 144;
        case TSB_Q6_K: return cols / 256 * 210;
        case TSB_MXFP4: return (cols + 31) / 32 * 17;
        case TSB_Q5_K: return cols / 256 * 176;
        case TSB_Q8_0: return cols / 32 * 34;
        default: return -1;
    }
}

static inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c[0] = n0, c[1] = n1, c[2] = n2, c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

uint64_t tsb_uniform_u64(int32_t mode, uint64_t seed, uint64_t step) {
    if (mode == 0) {
        uint64_t x = seed ^ (step * 0x9E3779B97F4A7C15ull);
        x += 0x9E3779B97F4A7C15ull;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        return x ^ (x >> 31);
    }
    uint32_t c[4] = {(uint32_t)step, (uint32_t)(step >> 32), 0u, 0u};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    return ((uint64_t)c[1] << 32) | c[0];
}

}  // extern "C"
