// Paged K/V cache: page bookkeeping on the host, and the kernels that write it —
// RoPE + K/V store for a batch of rows, accepted-path compaction, seeded fill.
#include <algorithm>
#include <cstring>
#include <new>

#include "kv.cuh"

namespace {

// ---- RoPE on q and k, then k and v into the cache --------------------------
// One CTA per row.  cos/sin of the row's position are computed once in shared
// memory (double precision exp/sin/cos rounded once, which reproduces a correctly
// rounded f32 libm: crates/compute/src/rope.rs:208-255), then every head is
// rotated with NeoX pairing (i, head_dim/2 + i).
__global__ void rope_store_kv_kernel(KvView kv, int layer, __half* __restrict__ qkv, const tsb_row_desc* __restrict__ rows,
                                     int n_q_heads, float log_theta, uint32_t* __restrict__ err) {
    extern __shared__ float cs[];  // cos[half], sin[half]
    pdl_wait();
    const int r = blockIdx.x;
    const tsb_row_desc rd = rows[r];
    const int hd = kv.head_dim, half = hd >> 1;
    const float pos = (float)rd.position;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float exponent = -((float)(2 * i)) / (float)hd;
        const float freq = (float)exp((double)__fmul_rn(exponent, log_theta));
        const float angle = __fmul_rn(pos, freq);
        cs[i] = (float)cos((double)angle);
        cs[half + i] = (float)sin((double)angle);
    }
    __syncthreads();
    pdl_launch_dependents();
    const int nkv = kv.kv_heads;
    __half* row = qkv + (size_t)r * (size_t)(n_q_heads + 2 * nkv) * hd;
    __half* krow = kv_row(kv, layer, 0, rd.seq, rd.base + rd.slot);
    __half* vrow = kv_row(kv, layer, 1, rd.seq, rd.base + rd.slot);
    if (!krow || !vrow || rd.seq < 0 || rd.seq >= kv.max_seqs) {
        if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
        return;
    }
    // q heads in place, k heads into the cache
    for (int idx = threadIdx.x; idx < (n_q_heads + nkv) * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const __half* src = row + (size_t)h * hd;
        const float x0 = __half2float(src[i]), x1 = __half2float(src[half + i]);
        const float c = cs[i], s = cs[half + i];
        const __half o0 = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        const __half o1 = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
        __half* dst = h < n_q_heads ? row + (size_t)h * hd : krow + (size_t)(h - n_q_heads) * hd;
        dst[i] = o0;
        dst[half + i] = o1;
    }
    // v heads: straight copy
    const uint4* vsrc = reinterpret_cast<const uint4*>(row + (size_t)(n_q_heads + nkv) * hd);
    uint4* vdst = reinterpret_cast<uint4*>(vrow);
    for (int idx = threadIdx.x; idx < nkv * hd / 8; idx += blockDim.x) vdst[idx] = vsrc[idx];
}

// ---- accepted-path compaction ---------------------------------------------
// dst row base+r <- src row base+path[r], every layer, K and V.  path is strictly increasing with
// path[0] == 0, so path[r] >= r and a row is never read after it has been overwritten provided rows
// are moved in increasing r; each (layer, K|V) pair is handled by one CTA, which moves the rows one
// after another with a barrier between them.
__global__ void kv_commit_path_kernel(KvView kv, int seq, int base, const uint32_t* __restrict__ path, int keep,
                                      uint32_t* __restrict__ err) {
    pdl_wait();
    const int layer = blockIdx.x >> 1, which = blockIdx.x & 1;
    const int row16 = kv.kv_heads * kv.head_dim / 8;
    for (int r = 1; r < keep; r++) {
        const int src_slot = (int)path[r];
        if (src_slot != r) {
            const uint4* src = reinterpret_cast<const uint4*>(kv_row(kv, layer, which, seq, base + src_slot));
            uint4* dst = reinterpret_cast<uint4*>(kv_row(kv, layer, which, seq, base + r));
            if (!src || !dst) {
                if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
                return;
            }
            for (int i = threadIdx.x; i < row16; i += blockDim.x) dst[i] = src[i];
        }
        __syncthreads();
    }
    pdl_launch_dependents();
}

// ---- seeded fill (benchmark set-up) ----------------------------------------
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}
__global__ void kv_fill_random_kernel(KvView kv, int seq, int tokens, uint64_t seed) {
    const int row = kv.kv_heads * kv.head_dim;
    const int64_t per_layer = (int64_t)tokens * row;
    const int64_t total = per_layer * kv.layers * 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int lw = (int)(i / per_layer);
        const int64_t rem = i - (int64_t)lw * per_layer;
        const int pos = (int)(rem / row), e = (int)(rem - (int64_t)pos * row);
        __half* p = kv_row(kv, lw >> 1, lw & 1, seq, pos);
        if (!p) continue;
        // sum of four uniforms, centred: roughly normal with unit variance
        uint32_t h = hash32((uint32_t)i ^ (uint32_t)(seed * 0x9E3779B9u)) ^ hash32((uint32_t)(i >> 32) + (uint32_t)(seed >> 32));
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            h = hash32(h + 0x9E3779B9u * (k + 1));
            acc += (float)(h >> 8) * (1.0f / 16777216.0f);
        }
        p[e] = __float2half_rn((acc - 2.0f) * 1.7320508f);
    }
}

int32_t kv_check(tsb_kv* kv, int32_t seq) {
    if (!kv) return TSB_ERR_INVALID;
    if (seq < 0 || seq >= kv->view.max_seqs) return tsb_fail(kv->ctx, TSB_ERR_INVALID, "stream %d outside 0..%d", seq, kv->view.max_seqs);
    return TSB_OK;
}

}  // namespace

cudaError_t launch_rope_store_kv(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, __half* qkv,
                                 const tsb_row_desc* rows_dev, int rows, int n_q_heads, float theta) {
    return tsb_launch(ctx, rope_store_kv_kernel, dim3((unsigned)rows), dim3(256), (size_t)kv->view.head_dim * sizeof(float),
                      st, true, kv->view, layer, qkv, rows_dev, n_q_heads, logf(theta), ctx->dev_error);
}

extern "C" {

int32_t tsb_kv_create(tsb_ctx* ctx, int32_t layers, int32_t kv_heads, int32_t head_dim, int32_t page_tokens,
                      int32_t num_pages, int32_t max_seqs, int32_t max_pages_per_seq, tsb_kv** out) {
    if (!ctx || !out) return TSB_ERR_INVALID;
    *out = nullptr;
    TSB_REQUIRE(ctx, layers > 0 && kv_heads > 0 && num_pages > 0 && max_seqs > 0 && max_pages_per_seq > 0, "bad sizes");
    TSB_REQUIRE(ctx, head_dim == 64 || head_dim == 128, "head_dim must be 64 or 128, got %d", head_dim);
    TSB_REQUIRE(ctx, page_tokens >= 16 && (page_tokens & (page_tokens - 1)) == 0, "page_tokens must be a power of two >= 16");
    DeviceGuard g(ctx);
    tsb_kv* kv = new (std::nothrow) tsb_kv();
    if (!kv) return TSB_ERR_OOM;
    kv->ctx = ctx;
    KvView& v = kv->view;
    v.layers = layers, v.kv_heads = kv_heads, v.head_dim = head_dim;
    v.page_tokens = page_tokens;
    v.page_shift = 0;
    while ((1 << v.page_shift) < page_tokens) v.page_shift++;
    v.num_pages = num_pages, v.max_seqs = max_seqs, v.max_pages_per_seq = max_pages_per_seq;
    v.kv_stride = (int64_t)num_pages * page_tokens * kv_heads * head_dim;
    v.layer_stride = 2 * v.kv_stride;
    const size_t pool_bytes = (size_t)layers * v.layer_stride * sizeof(__half);
    cudaError_t e = cudaMalloc((void**)&v.pool, pool_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete kv;
        return tsb_fail(ctx, TSB_ERR_OOM, "K/V pool of %zu bytes: %s", pool_bytes, cudaGetErrorString(e));
    }
    // rows nobody has written yet are read by kernels that fetch whole pages (and mask them): they must hold finite values
    e = cudaMemset(v.pool, 0, pool_bytes);
    if (e != cudaSuccess) {
        cudaFree(v.pool);
        delete kv;
        return tsb_fail(ctx, TSB_ERR_CUDA, "clearing the K/V pool: %s", cudaGetErrorString(e));
    }
    const size_t pt = (size_t)max_seqs * max_pages_per_seq;
    kv->page_table_host.assign(pt, -1);
    e = cudaMalloc((void**)&kv->page_table_dev, pt * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemset(kv->page_table_dev, 0xFF, pt * sizeof(int32_t));
    if (e != cudaSuccess) {
        cudaFree(v.pool);
        delete kv;
        return tsb_fail(ctx, TSB_ERR_CUDA, "page table: %s", cudaGetErrorString(e));
    }
    v.page_table = kv->page_table_dev;
    kv->free_pages.resize(num_pages);
    for (int i = 0; i < num_pages; i++) kv->free_pages[i] = num_pages - 1 - i;  // pop_back hands out page 0 first
    kv->pages_of_seq.assign(max_seqs, 0);
    kv->cursor.assign(max_seqs, 0);
    *out = kv;
    return TSB_OK;
}

void tsb_kv_destroy(tsb_kv* kv) {
    if (!kv) return;
    DeviceGuard g(kv->ctx);
    cudaDeviceSynchronize();
    cudaFree(kv->view.pool);
    cudaFree(kv->page_table_dev);
    delete kv;
}

int32_t tsb_kv_reserve(tsb_kv* kv, int32_t seq, int64_t tokens) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    tsb_ctx* ctx = kv->ctx;
    const KvView& v = kv->view;
    const int64_t need = (tokens + v.page_tokens - 1) >> v.page_shift;
    if (need > v.max_pages_per_seq)
        return tsb_fail(ctx, TSB_ERR_OOM, "stream %d needs %lld pages, table holds %d", seq, (long long)need, v.max_pages_per_seq);
    const int have = kv->pages_of_seq[seq];
    if (need <= have) return TSB_OK;
    if ((int64_t)kv->free_pages.size() < need - have)
        return tsb_fail(ctx, TSB_ERR_OOM, "out of K/V pages (%zu free, %lld wanted)", kv->free_pages.size(), (long long)(need - have));
    DeviceGuard g(ctx);
    int32_t* row = &kv->page_table_host[(size_t)seq * v.max_pages_per_seq];
    for (int64_t p = have; p < need; p++) {
        row[p] = kv->free_pages.back();
        kv->free_pages.pop_back();
    }
    kv->pages_of_seq[seq] = (int)need;
    TSB_CUDA(ctx, cudaMemcpy(kv->page_table_dev + (size_t)seq * v.max_pages_per_seq + have, row + have,
                             (size_t)(need - have) * sizeof(int32_t), cudaMemcpyHostToDevice));
    return TSB_OK;
}

int32_t tsb_kv_reset(tsb_kv* kv, int32_t seq) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    tsb_ctx* ctx = kv->ctx;
    const KvView& v = kv->view;
    DeviceGuard g(ctx);
    int32_t* row = &kv->page_table_host[(size_t)seq * v.max_pages_per_seq];
    const int have = kv->pages_of_seq[seq];
    for (int p = have - 1; p >= 0; p--) {
        kv->free_pages.push_back(row[p]);
        row[p] = -1;
    }
    kv->pages_of_seq[seq] = 0;
    kv->cursor[seq] = 0;
    if (have)
        TSB_CUDA(ctx, cudaMemcpy(kv->page_table_dev + (size_t)seq * v.max_pages_per_seq, row, (size_t)have * sizeof(int32_t),
                                 cudaMemcpyHostToDevice));
    return TSB_OK;
}

int64_t tsb_kv_cursor(const tsb_kv* kv, int32_t seq) {
    if (!kv || seq < 0 || seq >= kv->view.max_seqs) return -1;
    return kv->cursor[seq];
}

int32_t tsb_kv_set_cursor(tsb_kv* kv, int32_t seq, int64_t position) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    if (position < 0 || position > (int64_t)kv->pages_of_seq[seq] * kv->view.page_tokens)
        return tsb_fail(kv->ctx, TSB_ERR_STATE, "cursor %lld outside the reserved %lld positions", (long long)position,
                        (long long)kv->pages_of_seq[seq] * kv->view.page_tokens);
    kv->cursor[seq] = position;
    return TSB_OK;
}

int32_t tsb_kv_rewind_by(tsb_kv* kv, int32_t seq, int64_t count) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    if (count < 0 || count > kv->cursor[seq])
        return tsb_fail(kv->ctx, TSB_ERR_STATE, "cannot rewind %lld rows from cursor %lld", (long long)count, (long long)kv->cursor[seq]);
    kv->cursor[seq] -= count;
    return TSB_OK;
}

static int32_t kv_copy_rows(tsb_kv* kv, tsb_stream s, int32_t seq, int32_t layer, int64_t pos0, int32_t n, void* hk, void* hv,
                            bool to_device) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    tsb_ctx* ctx = kv->ctx;
    const KvView& v = kv->view;
    TSB_REQUIRE(ctx, layer >= 0 && layer < v.layers && n >= 0 && pos0 >= 0 && hk && hv, "bad arguments");
    if (pos0 + n > (int64_t)kv->pages_of_seq[seq] * v.page_tokens)
        return tsb_fail(ctx, TSB_ERR_STATE, "rows %lld..%lld are not reserved", (long long)pos0, (long long)(pos0 + n));
    DeviceGuard g(ctx);
    const size_t row = (size_t)v.kv_heads * v.head_dim;
    const int32_t* pt = &kv->page_table_host[(size_t)seq * v.max_pages_per_seq];
    int64_t p = pos0;
    while (p < pos0 + n) {  // one copy per page run
        const int64_t in_page = p & (v.page_tokens - 1);
        const int64_t run = std::min<int64_t>(v.page_tokens - in_page, pos0 + n - p);
        const int64_t slot = (int64_t)pt[p >> v.page_shift] * v.page_tokens + in_page;
        for (int which = 0; which < 2; which++) {
            __half* dev = v.pool + (int64_t)layer * v.layer_stride + (int64_t)which * v.kv_stride + slot * (int64_t)row;
            char* host = (char*)(which ? hv : hk) + (size_t)(p - pos0) * row * sizeof(__half);
            if (to_device)
                TSB_CUDA(ctx, cudaMemcpyAsync(dev, host, (size_t)run * row * sizeof(__half), cudaMemcpyHostToDevice, (cudaStream_t)s));
            else
                TSB_CUDA(ctx, cudaMemcpyAsync(host, dev, (size_t)run * row * sizeof(__half), cudaMemcpyDeviceToHost, (cudaStream_t)s));
        }
        p += run;
    }
    TSB_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)s));
    return TSB_OK;
}

int32_t tsb_kv_write_rows(tsb_kv* kv, tsb_stream s, int32_t seq, int32_t layer, int64_t pos0, int32_t n, const void* hk,
                          const void* hv) {
    return kv_copy_rows(kv, s, seq, layer, pos0, n, const_cast<void*>(hk), const_cast<void*>(hv), true);
}
int32_t tsb_kv_read_rows(tsb_kv* kv, tsb_stream s, int32_t seq, int32_t layer, int64_t pos0, int32_t n, void* hk, void* hv) {
    return kv_copy_rows(kv, s, seq, layer, pos0, n, hk, hv, false);
}

int32_t tsb_kv_fill_random(tsb_kv* kv, tsb_stream s, int32_t seq, int64_t tokens, uint64_t seed) {
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    rc = tsb_kv_reserve(kv, seq, tokens);
    if (rc) return rc;
    tsb_ctx* ctx = kv->ctx;
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, tsb_launch(ctx, kv_fill_random_kernel, dim3((unsigned)(ctx->sm_count * 8)), dim3(256), 0, (cudaStream_t)s,
                             false, kv->view, seq, (int)tokens, seed));
    return TSB_OK;
}

int32_t tsb_rope_store_kv(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, void* qkv_f16, const tsb_row_desc* rows_dev,
                          int32_t rows, int32_t n_q_heads, float theta) {
    if (!ctx || !kv) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, qkv_f16 && rows_dev && rows > 0 && n_q_heads > 0, "bad arguments");
    TSB_REQUIRE(ctx, layer >= 0 && layer < kv->view.layers, "layer %d outside 0..%d", layer, kv->view.layers);
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_rope_store_kv(ctx, (cudaStream_t)s, kv, layer, (__half*)qkv_f16, rows_dev, rows, n_q_heads, theta));
    return TSB_OK;
}

int32_t tsb_kv_commit_path(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t seq, int64_t base, const uint32_t* host_path,
                           int32_t keep) {
    if (!ctx || !kv) return TSB_ERR_INVALID;
    int32_t rc = kv_check(kv, seq);
    if (rc) return rc;
    TSB_REQUIRE(ctx, host_path && keep >= 1 && keep <= 128, "path of 1..128 slots expected, got %d", keep);
    // the only shape for which the in-place gather is race-free (crates/gpu/src/dflash_conv.rs:218-234)
    TSB_REQUIRE(ctx, host_path[0] == 0, "path must start at the anchor slot 0");
    for (int r = 1; r < keep; r++)
        TSB_REQUIRE(ctx, host_path[r] > host_path[r - 1], "path must be strictly increasing (slot %d)", r);
    const uint64_t top = (uint64_t)base + host_path[keep - 1];  // 64-bit so a wrapping sum cannot pass
    if (base < 0 || top >= (uint64_t)kv->pages_of_seq[seq] * kv->view.page_tokens)
        return tsb_fail(ctx, TSB_ERR_STATE, "path slot %llu is past the reserved rows", (unsigned long long)top);
    bool identity = true;
    for (int r = 0; r < keep; r++) identity &= host_path[r] == (uint32_t)r;
    if (identity) return TSB_OK;  // a chain: nothing to move
    DeviceGuard g(ctx);
    cudaStream_t st = (cudaStream_t)s;
    uint32_t* dpath = nullptr;
    TSB_CUDA(ctx, cudaMallocAsync((void**)&dpath, keep * sizeof(uint32_t), st));
    cudaError_t e = cudaMemcpyAsync(dpath, host_path, keep * sizeof(uint32_t), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess)
        e = tsb_launch(ctx, kv_commit_path_kernel, dim3((unsigned)(kv->view.layers * 2)), dim3(256), 0, st, true, kv->view,
                       (int)seq, (int)base, (const uint32_t*)dpath, (int)keep, ctx->dev_error);
    cudaError_t e2 = cudaFreeAsync(dpath, st);
    TSB_CUDA(ctx, e);
    TSB_CUDA(ctx, e2);
    return TSB_OK;
}

}  // extern "C"
