// The producer: a dense Llama-style decoder running on the kernels of this
// library, with the reference's rounding points (f16 storage between operators,
// fp32 accumulation, bf16 norm weights), plus the sessions that own K/V caches
// and work buffers for a set of independent request streams.
//
// Op order of one layer (crates/runtime/src/families/llama/mod.rs:205-291,
// dense.rs:48-120), fused where two reference dispatches are adjacent:
//   [residual add +] RMSNorm -> qkv matmul (one matmul over q|k|v rows) ->
//   RoPE + K/V store -> split-KV attention -> o_proj matmul ->
//   residual add + RMSNorm -> gate|up matmul -> SiLU*up -> down matmul
// Every producer of a matmul input writes the matmul's activation operand
// directly, so a layer is 9 launches.
#include <algorithm>
#include <cstring>
#include <memory>
#include <new>
#include <vector>

#include "accept.cuh"
#include "attention.cuh"
#include "model.cuh"

namespace {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

// Seeded synthetic blocks: every byte pseudo-random, then the scale fields are overwritten so the
// dequantised weights are finite, zero-mean and of standard deviation about 0.02.
__host__ __device__ inline int block_bytes_of(int qtype) {
    return qtype == TSB_Q4_K ? 144 : qtype == TSB_Q6_K ? 210 : qtype == TSB_Q5_K ? 176 : qtype == TSB_Q8_0 ? 34 : 17;
}

__global__ void fill_blocks_kernel(uint8_t* __restrict__ data, int64_t n_blocks, int qtype, uint32_t seed) {
    const int bb = block_bytes_of(qtype);
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (int64_t)gridDim.x * blockDim.x) {
        uint8_t* p = data + b * bb;
        uint32_t h = mix32((uint32_t)b * 0x9E3779B9u + seed) ^ mix32((uint32_t)(b >> 32) + seed * 31u);
        for (int i = 0; i < bb; i++) {
            if ((i & 3) == 0) h = mix32(h + 0x9E3779B9u);
            p[i] = (uint8_t)(h >> ((i & 3) * 8));
        }
        const float u = (float)(mix32(h) >> 8) * (1.0f / 16777216.0f);
        if (qtype == TSB_Q4_K) {
            // zero-mean weights of std ~0.02: E[sc*q] = 31.5*7.5 is cancelled by dmin*E[m] with dmin = 7.5 d
            const __half d = __float2half_rn(7.7e-5f * (0.5f + u)), dm = __float2half_rn(7.5f * 7.7e-5f * (0.5f + u));
            const unsigned short db = __half_as_ushort(d), mb = __half_as_ushort(dm);
            p[0] = db & 0xFF, p[1] = db >> 8, p[2] = mb & 0xFF, p[3] = mb >> 8;
        } else if (qtype == TSB_Q6_K) {
            const unsigned short db = __half_as_ushort(__float2half_rn(1.46e-5f * (0.5f + u)));
            p[208] = db & 0xFF, p[209] = db >> 8;
        } else if (qtype == TSB_Q5_K) {
            // E[sc*q] = 31.5*15.5 cancelled by dmin*E[m] with dmin = 15.5 d
            const __half d = __float2half_rn(3.7e-5f * (0.5f + u)), dm = __float2half_rn(15.5f * 3.7e-5f * (0.5f + u));
            const unsigned short db = __half_as_ushort(d), mb = __half_as_ushort(dm);
            p[0] = db & 0xFF, p[1] = db >> 8, p[2] = mb & 0xFF, p[3] = mb >> 8;
        } else if (qtype == TSB_Q8_0) {
            const unsigned short db = __half_as_ushort(__float2half_rn(2.7e-4f * (0.5f + u)));
            p[0] = db & 0xFF, p[1] = db >> 8;
        } else {
            p[0] = (uint8_t)(119 + (h & 1));
        }
    }
}

__global__ void fill_u16_kernel(uint16_t* p, int64_t n, uint16_t v) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

}  // namespace

// ------------------------------------------------------------------ model

static int64_t mat_bytes(const Mat& m) { return m.rows * tsb_row_bytes(m.qtype, m.cols); }

static int32_t mat_alloc(tsb_ctx* ctx, Mat& m, int qtype, int64_t rows, int64_t cols) {
    m.qtype = qtype, m.rows = rows, m.cols = cols;
    void* p = nullptr;
    // spare bytes: the bulk-copy path may over-fetch one 16-byte granule past an unaligned row run
    int32_t rc = tsb_alloc(ctx, (size_t)mat_bytes(m) + 256, &p);
    if (rc) return rc;
    m.data = (uint8_t*)p;
    m.owned = true;
    cudaMemset(m.data + mat_bytes(m), 0, 256);
    return TSB_OK;
}

static void mat_free(tsb_ctx* ctx, Mat& m) {
    if (m.owned && m.data) tsb_free(ctx, m.data);
    m = Mat();
}

static int local_experts(const tsb_model* m) { return m->n_local_experts > 0 ? m->n_local_experts : m->n_experts; }

static int64_t rows_of_v(const tsb_model_config& c) { return (int64_t)c.n_kv_heads * c.head_dim; }

static Mat* fused_slot(tsb_model* m, int layer, int which, int64_t* row_off, int64_t* total_rows, int64_t* want_rows,
                       int64_t* want_cols) {
    const tsb_model_config& c = m->cfg;
    const int64_t qd = (int64_t)c.n_q_heads * c.head_dim, kd = (int64_t)c.n_kv_heads * c.head_dim;
    *row_off = 0;
    if (which == TSB_W_EMBED) {
        *total_rows = *want_rows = c.vocab, *want_cols = c.d_model;
        return &m->embed;
    }
    if (which == TSB_W_LM_HEAD) {
        *total_rows = *want_rows = c.vocab, *want_cols = c.d_model;
        return &m->lm_head;
    }
    if (layer < 0 || layer >= c.n_layers) return nullptr;
    LayerW& l = m->layers[layer];
    switch (which) {
        case TSB_W_Q: *total_rows = qd + 2 * kd, *want_rows = qd, *want_cols = c.d_model; return &l.wqkv;
        case TSB_W_K: *total_rows = qd + 2 * kd, *want_rows = kd, *want_cols = c.d_model, *row_off = qd; return &l.wqkv;
        case TSB_W_V: *total_rows = qd + 2 * kd, *want_rows = kd, *want_cols = c.d_model, *row_off = qd + kd; return &l.wqkv;
        case TSB_W_O: *total_rows = *want_rows = c.d_model, *want_cols = qd; return &l.wo;
        case TSB_W_GATE: *total_rows = 2 * (int64_t)c.ffn, *want_rows = c.ffn, *want_cols = c.d_model; return &l.wgu;
        case TSB_W_UP: *total_rows = 2 * (int64_t)c.ffn, *want_rows = c.ffn, *want_cols = c.d_model, *row_off = c.ffn; return &l.wgu;
        case TSB_W_DOWN: *total_rows = *want_rows = c.d_model, *want_cols = c.ffn; return &l.wdown;
        default: return nullptr;
    }
}

extern "C" {

int32_t tsb_model_create(tsb_ctx* ctx, const tsb_model_config* cfg, tsb_model** out) {
    if (!ctx || !cfg || !out) return TSB_ERR_INVALID;
    *out = nullptr;
    TSB_REQUIRE(ctx, cfg->n_layers > 0 && cfg->d_model > 0 && cfg->n_q_heads > 0 && cfg->n_kv_heads > 0 && cfg->ffn > 0 &&
                         cfg->vocab > 0 && cfg->max_context > 0,
                "model dimensions must be positive");
    TSB_REQUIRE(ctx, cfg->head_dim == 64 || cfg->head_dim == 128, "head_dim must be 64 or 128");
    TSB_REQUIRE(ctx, cfg->n_q_heads % cfg->n_kv_heads == 0, "n_q_heads must be a multiple of n_kv_heads");
    if (cfg->d_model % 256 || cfg->ffn % 256 || (cfg->n_q_heads * cfg->head_dim) % 256)
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "d_model, ffn and n_q_heads*head_dim must be multiples of 256");
    tsb_model* m = new (std::nothrow) tsb_model();
    if (!m) return TSB_ERR_OOM;
    m->ctx = ctx;
    m->cfg = *cfg;
    m->layers.resize(cfg->n_layers);
    *out = m;
    return TSB_OK;
}

void tsb_model_destroy(tsb_model* m) {
    if (!m) return;
    DeviceGuard g(m->ctx);
    cudaDeviceSynchronize();
    for (auto& l : m->layers) {
        mat_free(m->ctx, l.wqkv), mat_free(m->ctx, l.wv), mat_free(m->ctx, l.wo), mat_free(m->ctx, l.wgu), mat_free(m->ctx, l.wdown);
        if (l.norms_owned) {
            if (l.attn_norm) tsb_free(m->ctx, l.attn_norm);
            if (l.ffn_norm) tsb_free(m->ctx, l.ffn_norm);
        }
        if (l.moe_owned)
            for (void* p : {(void*)l.router_q, (void*)l.router_scale, (void*)l.router_bias, (void*)l.experts_gate_up, (void*)l.experts_down})
                if (p) tsb_free(m->ctx, p);
    }
    mat_free(m->ctx, m->embed), mat_free(m->ctx, m->lm_head);
    if (m->out_norm_owned && m->out_norm) tsb_free(m->ctx, m->out_norm);
    delete m;
}

int32_t tsb_model_set_matrix(tsb_model* m, int32_t layer, int32_t which, int32_t qtype, const void* host_blocks,
                             int64_t rows, int64_t cols) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, host_blocks, "null data");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    int64_t off, total, wr, wc;
    Mat* slot = fused_slot(m, layer, which, &off, &total, &wr, &wc);
    TSB_REQUIRE(ctx, slot, "no such tensor (layer %d, which %d)", layer, which);
    TSB_REQUIRE(ctx, rows == wr && cols == wc, "tensor %d of layer %d must be %lld x %lld, got %lld x %lld", which, layer,
                (long long)wr, (long long)wc, (long long)rows, (long long)cols);
    DeviceGuard g(ctx);
    const int64_t rb = tsb_row_bytes(qtype, cols);
    if (which == TSB_W_Q || which == TSB_W_K || which == TSB_W_V) {
        // Files quantized with mixed recipes keep v in a wider format than q and k: v then lives in its own matrix
        // and the pass runs the q|k rows and the v rows as two launches.
        LayerW& l = m->layers[layer];
        const int64_t qk_rows = total - rows_of_v(m->cfg);
        if (which == TSB_W_V && (l.wv.data || (l.wqkv.data && l.wqkv.qtype != qtype))) {
            if (l.wv.data && l.wv.qtype != qtype) mat_free(ctx, l.wv);
            if (!l.wv.data) {
                int32_t rc = mat_alloc(ctx, l.wv, qtype, rows, cols);
                if (rc) return rc;
            }
            if (l.wqkv.data) l.wqkv.rows = qk_rows;
            TSB_CUDA(ctx, cudaMemcpy(l.wv.data, host_blocks, (size_t)(rows * rb), cudaMemcpyHostToDevice));
            l.qkv_set |= 4;
            return TSB_OK;
        }
        if (which != TSB_W_V && l.wqkv.data && l.wqkv.qtype != qtype) {
            if (l.qkv_set != 4 || l.wv.data || !l.wqkv.owned)
                return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "q and k of a layer must share one block format");
            // only v has arrived so far: it moves to its own matrix and q|k start over in the new format
            const int64_t vb = tsb_row_bytes(l.wqkv.qtype, cols);
            int32_t rc = mat_alloc(ctx, l.wv, l.wqkv.qtype, rows_of_v(m->cfg), cols);
            if (rc) return rc;
            TSB_CUDA(ctx, cudaMemcpy(l.wv.data, l.wqkv.data + qk_rows * vb, (size_t)(rows_of_v(m->cfg) * vb), cudaMemcpyDeviceToDevice));
            mat_free(ctx, l.wqkv);
            if ((rc = mat_alloc(ctx, l.wqkv, qtype, qk_rows, cols))) return rc;
        }
        l.qkv_set |= which == TSB_W_Q ? 1 : (which == TSB_W_K ? 2 : 4);
    }
    if (!slot->data) {
        int32_t rc = mat_alloc(ctx, *slot, qtype, total, cols);
        if (rc) return rc;
    } else if (slot->qtype != qtype) {
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "gate and up of a layer must share one block format");
    }
    TSB_CUDA(ctx, cudaMemcpy(slot->data + off * rb, host_blocks, (size_t)(rows * rb), cudaMemcpyHostToDevice));
    return TSB_OK;
}

int32_t tsb_model_set_moe(tsb_model* m, int32_t n_experts, int32_t top_k, int32_t moe_ffn) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, n_experts >= 1 && n_experts <= 512 && top_k >= 1 && top_k <= 8 && top_k <= n_experts, "need 1 <= top_k <= min(8, experts) and at most 512 experts");
    TSB_REQUIRE(ctx, moe_ffn > 0 && moe_ffn % 256 == 0, "the expert width must be a multiple of 256");
    for (const LayerW& l : m->layers) TSB_REQUIRE(ctx, !l.wgu.data && !l.wdown.data, "set_moe comes before the tensors");
    m->n_experts = n_experts, m->top_k = top_k, m->moe_ffn = moe_ffn;
    m->expert_lo = 0, m->n_local_experts = 0;
    return TSB_OK;
}

int32_t tsb_model_set_expert_shard(tsb_model* m, int32_t expert_lo, int32_t n_local) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, m->n_experts > 0, "the model has no experts (tsb_model_set_moe first)");
    TSB_REQUIRE(ctx, expert_lo >= 0 && n_local >= 1 && expert_lo + n_local <= m->n_experts, "experts %d..%d outside the model's %d", expert_lo,
                expert_lo + n_local, m->n_experts);
    for (const LayerW& l : m->layers) TSB_REQUIRE(ctx, !l.experts_gate_up && !l.experts_down, "the shard comes before the expert tensors");
    m->expert_lo = expert_lo, m->n_local_experts = n_local;
    return TSB_OK;
}

static int32_t upload(tsb_ctx* ctx, void** slot, const void* host, size_t bytes) {
    if (!*slot) {
        // spare bytes for the bulk-copy path's 16-byte granules, as for the dense matrices
        int32_t rc = tsb_alloc(ctx, bytes + 256, slot);
        if (rc) return rc;
        cudaMemset((uint8_t*)*slot + bytes, 0, 256);
    }
    TSB_CUDA(ctx, cudaMemcpy(*slot, host, bytes, cudaMemcpyHostToDevice));
    return TSB_OK;
}

int32_t tsb_model_set_router(tsb_model* m, int32_t layer, const void* q_u8, const void* scale_bf16, const void* bias_bf16) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, m->n_experts > 0, "the model has no experts (tsb_model_set_moe first)");
    TSB_REQUIRE(ctx, layer >= 0 && layer < m->cfg.n_layers && q_u8 && scale_bf16 && bias_bf16, "bad layer or null data");
    TSB_REQUIRE(ctx, m->cfg.d_model % 64 == 0, "d_model must be a multiple of the router's 64-column group");
    DeviceGuard g(ctx);
    LayerW& l = m->layers[layer];
    l.moe_owned = true;
    const size_t n = (size_t)m->n_experts * m->cfg.d_model;
    int32_t rc;
    if ((rc = upload(ctx, (void**)&l.router_q, q_u8, n)) || (rc = upload(ctx, (void**)&l.router_scale, scale_bf16, n / 64 * 2)) ||
        (rc = upload(ctx, (void**)&l.router_bias, bias_bf16, n / 64 * 2)))
        return rc;
    return TSB_OK;
}

int32_t tsb_model_set_experts(tsb_model* m, int32_t layer, int32_t qtype, const void* gate_up_blocks, const void* down_blocks) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, m->n_experts > 0, "the model has no experts (tsb_model_set_moe first)");
    TSB_REQUIRE(ctx, layer >= 0 && layer < m->cfg.n_layers && gate_up_blocks && down_blocks, "bad layer or null data");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    DeviceGuard g(ctx);
    LayerW& l = m->layers[layer];
    l.moe_owned = true;
    l.experts_qtype = qtype;
    const size_t gu = (size_t)local_experts(m) * 2 * m->moe_ffn * tsb_row_bytes(qtype, m->cfg.d_model);
    const size_t dn = (size_t)local_experts(m) * m->cfg.d_model * tsb_row_bytes(qtype, m->moe_ffn);
    int32_t rc;
    if ((rc = upload(ctx, (void**)&l.experts_gate_up, gate_up_blocks, gu)) || (rc = upload(ctx, (void**)&l.experts_down, down_blocks, dn))) return rc;
    return TSB_OK;
}

int32_t tsb_model_set_norm(tsb_model* m, int32_t layer, int32_t which, const void* host_bf16, int32_t n) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, host_bf16 && n == m->cfg.d_model, "a norm weight has d_model entries");
    uint16_t** slot;
    if (which == TSB_N_OUT) {
        slot = &m->out_norm;
        m->out_norm_owned = true;
    } else {
        TSB_REQUIRE(ctx, layer >= 0 && layer < m->cfg.n_layers, "layer %d outside the model", layer);
        slot = which == TSB_N_ATTN ? &m->layers[layer].attn_norm : &m->layers[layer].ffn_norm;
        m->layers[layer].norms_owned = true;
    }
    DeviceGuard g(ctx);
    if (!*slot) {
        void* p;
        int32_t rc = tsb_alloc(ctx, (size_t)n * 2, &p);
        if (rc) return rc;
        *slot = (uint16_t*)p;
    }
    TSB_CUDA(ctx, cudaMemcpy(*slot, host_bf16, (size_t)n * 2, cudaMemcpyHostToDevice));
    return TSB_OK;
}

int32_t tsb_model_share(tsb_model* dst, int32_t dst_layer, const tsb_model* src, int32_t src_layer) {
    if (!dst || !src) return TSB_ERR_INVALID;
    tsb_ctx* ctx = dst->ctx;
    TSB_REQUIRE(ctx, dst->cfg.d_model == src->cfg.d_model && dst->cfg.vocab == src->cfg.vocab, "models differ in width or vocabulary");
    auto borrow = [](Mat& d, const Mat& s) {
        d = s;
        d.owned = false;
    };
    if (dst_layer < 0) {
        borrow(dst->embed, src->embed), borrow(dst->lm_head, src->lm_head);
        dst->out_norm = src->out_norm, dst->out_norm_owned = false;
        return TSB_OK;
    }
    TSB_REQUIRE(ctx, dst_layer < dst->cfg.n_layers && src_layer >= 0 && src_layer < src->cfg.n_layers, "layer out of range");
    TSB_REQUIRE(ctx, dst->cfg.ffn == src->cfg.ffn && dst->cfg.n_q_heads == src->cfg.n_q_heads &&
                         dst->cfg.n_kv_heads == src->cfg.n_kv_heads && dst->cfg.head_dim == src->cfg.head_dim,
                "layer shapes differ");
    LayerW& d = dst->layers[dst_layer];
    const LayerW& s = src->layers[src_layer];
    borrow(d.wqkv, s.wqkv), borrow(d.wv, s.wv), borrow(d.wo, s.wo), borrow(d.wgu, s.wgu), borrow(d.wdown, s.wdown);
    d.qkv_set = s.qkv_set;
    d.router_q = s.router_q, d.router_scale = s.router_scale, d.router_bias = s.router_bias;
    d.experts_gate_up = s.experts_gate_up, d.experts_down = s.experts_down, d.experts_qtype = s.experts_qtype, d.moe_owned = false;
    d.attn_norm = s.attn_norm, d.ffn_norm = s.ffn_norm, d.norms_owned = false;
    return TSB_OK;
}

int32_t tsb_model_fill_synthetic(tsb_model* m, int32_t qtype, int32_t lm_head_qtype, uint64_t seed) {
    if (!m) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST && lm_head_qtype >= TSB_Q4_K && lm_head_qtype <= TSB_QTYPE_LAST, "bad format");
    DeviceGuard g(ctx);
    const tsb_model_config& c = m->cfg;
    const int64_t qd = (int64_t)c.n_q_heads * c.head_dim, kd = (int64_t)c.n_kv_heads * c.head_dim;
    uint32_t sd = (uint32_t)seed * 2654435761u + (uint32_t)(seed >> 32);
    auto fill = [&](Mat& t, int qt, int64_t rows, int64_t cols) -> int32_t {
        if (!t.data) {
            int32_t rc = mat_alloc(ctx, t, qt, rows, cols);
            if (rc) return rc;
        }
        const int64_t nb = mat_bytes(t) / block_bytes_of(qt);
        fill_blocks_kernel<<<1024, 256>>>(t.data, nb, qt, sd);
        sd = sd * 1664525u + 1013904223u;
        return TSB_OK;
    };
    auto ones = [&](uint16_t** p) -> int32_t {
        if (!*p) {
            void* q;
            int32_t rc = tsb_alloc(ctx, (size_t)c.d_model * 2, &q);
            if (rc) return rc;
            *p = (uint16_t*)q;
        }
        fill_u16_kernel<<<32, 256>>>(*p, c.d_model, (uint16_t)0x3F80);  // bf16 1.0
        return TSB_OK;
    };
    int32_t rc;
    for (auto& l : m->layers) {
        if ((rc = fill(l.wqkv, qtype, qd + 2 * kd, c.d_model))) return rc;
        if ((rc = fill(l.wo, qtype, c.d_model, qd))) return rc;
        if (m->n_experts > 0) {
            // routed layers: random 8-bit router with scale 0.004 / bias -0.5 (zero-mean weights), experts as blocks
            const size_t rn = (size_t)m->n_experts * c.d_model, rg = rn / 64;
            const int64_t gu_b = (int64_t)local_experts(m) * 2 * m->moe_ffn * tsb_row_bytes(qtype, c.d_model);
            const int64_t dn_b = (int64_t)local_experts(m) * c.d_model * tsb_row_bytes(qtype, m->moe_ffn);
            l.moe_owned = true, l.experts_qtype = qtype;
            void* p;
            if (!l.router_q) {
                if ((rc = tsb_alloc(ctx, rn + 256, &p))) return rc;
                l.router_q = (uint8_t*)p;
                if ((rc = tsb_alloc(ctx, rg * 2, &p))) return rc;
                l.router_scale = (uint16_t*)p;
                if ((rc = tsb_alloc(ctx, rg * 2, &p))) return rc;
                l.router_bias = (uint16_t*)p;
                if ((rc = tsb_alloc(ctx, (size_t)gu_b + 256, &p))) return rc;
                l.experts_gate_up = (uint8_t*)p;
                if ((rc = tsb_alloc(ctx, (size_t)dn_b + 256, &p))) return rc;
                l.experts_down = (uint8_t*)p;
                cudaMemset(l.experts_gate_up + gu_b, 0, 256), cudaMemset(l.experts_down + dn_b, 0, 256);
            }
            fill_blocks_kernel<<<64, 256>>>(l.router_q, (int64_t)(rn / 17), TSB_MXFP4, sd);  // any bytes do for the 8-bit weights
            fill_u16_kernel<<<32, 256>>>(l.router_scale, (int64_t)rg, (uint16_t)0x3B83);      // bf16 0.004
            fill_u16_kernel<<<32, 256>>>(l.router_bias, (int64_t)rg, (uint16_t)0xBF00);       // bf16 -0.5
            fill_blocks_kernel<<<1024, 256>>>(l.experts_gate_up, gu_b / block_bytes_of(qtype), qtype, sd + 1);
            fill_blocks_kernel<<<1024, 256>>>(l.experts_down, dn_b / block_bytes_of(qtype), qtype, sd + 2);
            sd = sd * 1664525u + 1013904223u;
        } else {
            if ((rc = fill(l.wgu, qtype, 2 * (int64_t)c.ffn, c.d_model))) return rc;
            if ((rc = fill(l.wdown, qtype, c.d_model, c.ffn))) return rc;
        }
        l.norms_owned = true;
        if ((rc = ones(&l.attn_norm)) || (rc = ones(&l.ffn_norm))) return rc;
    }
    if ((rc = fill(m->embed, qtype, c.vocab, c.d_model))) return rc;
    if ((rc = fill(m->lm_head, lm_head_qtype, c.vocab, c.d_model))) return rc;
    m->out_norm_owned = true;
    if ((rc = ones(&m->out_norm))) return rc;
    TSB_CUDA(ctx, cudaDeviceSynchronize());
    return TSB_OK;
}

int64_t tsb_model_weight_bytes(const tsb_model* m) {
    if (!m) return 0;
    int64_t t = mat_bytes(m->lm_head);
    for (auto& l : m->layers) t += mat_bytes(l.wqkv) + mat_bytes(l.wv) + mat_bytes(l.wo) + mat_bytes(l.wgu) + mat_bytes(l.wdown);
    if (m->n_experts > 0)  // every expert, although a pass reads only the routed ones
        for (auto& l : m->layers)
            t += (int64_t)local_experts(m) * (2 * m->moe_ffn * tsb_row_bytes(l.experts_qtype, m->cfg.d_model) +
                                          m->cfg.d_model * tsb_row_bytes(l.experts_qtype, m->moe_ffn)) +
                 (int64_t)m->n_experts * m->cfg.d_model;
    return t;
}

}  // extern "C"

constexpr int WIDE_MIN_ROWS = 24;  // a model whose largest pass has this many rows or more runs every pass on the tensor-memory matmul

static int32_t model_complete(const tsb_model* m) {
    tsb_ctx* ctx = m->ctx;
    for (size_t i = 0; i < m->layers.size(); i++) {
        const LayerW& l = m->layers[i];
        if (m->n_experts > 0)
            TSB_REQUIRE(ctx, l.wqkv.data && l.wo.data && l.attn_norm && l.ffn_norm && l.router_q && l.experts_gate_up && l.experts_down,
                        "layer %zu is missing a tensor (attention, norms, router or experts)", i);
        else
            TSB_REQUIRE(ctx, l.wqkv.data && l.wo.data && l.wgu.data && l.wdown.data && l.attn_norm && l.ffn_norm,
                        "layer %zu is missing a tensor", i);
        TSB_REQUIRE(ctx, l.qkv_set == 0 || l.qkv_set == 7, "layer %zu is missing one of q, k, v", i);
    }
    TSB_REQUIRE(ctx, m->embed.data && m->lm_head.data && m->out_norm, "embedding, head or final norm missing");
    return TSB_OK;
}

// ------------------------------------------------------------------ session

static int32_t dev_alloc(tsb_ctx* ctx, std::vector<void*>& owned, size_t bytes, void** out) {
    int32_t rc = tsb_alloc(ctx, bytes, out);
    if (rc == TSB_OK) owned.push_back(*out);
    return rc;
}

static int32_t runtime_init(tsb_session* s, ModelRt& rt, const tsb_model* model, int n_streams, int max_rows, int page_tokens, bool is_draft) {
    tsb_ctx* ctx = s->ctx;
    rt.model = model;
    const tsb_model_config& c = model->cfg;
    const int R = n_streams * max_rows;
    const int Rp = (R + 7) / 8 * 8;  // activation operands hold whole token tiles
    const int64_t qkv_dim = (int64_t)(c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim;
    const int pages_per_seq = (c.max_context + page_tokens - 1) / page_tokens;
    int32_t rc = tsb_kv_create(ctx, c.n_layers, c.n_kv_heads, c.head_dim, page_tokens, pages_per_seq * n_streams, n_streams,
                               pages_per_seq, &rt.kv);
    if (rc) return rc;
    auto A = [&](size_t bytes, void** p) { return dev_alloc(ctx, s->owned, bytes, p); };
    if ((rc = A((size_t)R * c.d_model * 2, (void**)&rt.h))) return rc;
    if ((rc = A((size_t)R * c.n_q_heads * c.head_dim * 2, (void**)&rt.q))) return rc;
    if ((rc = A((size_t)R * c.head_dim * sizeof(float), (void**)&rt.cs))) return rc;
    if ((rc = A((size_t)(2 * c.n_layers + 1) * R * (c.d_model / 16) * sizeof(float), (void**)&rt.ss))) return rc;
    const int64_t od = (int64_t)c.n_q_heads * c.head_dim;
    if ((rc = A(act_xp_bytes(Rp, c.d_model), (void**)&rt.act_d.xp)) || (rc = A(act_xs_bytes(Rp, c.d_model), (void**)&rt.act_d.xs))) return rc;
    if ((rc = A(act_xp_bytes(Rp, od), (void**)&rt.act_o.xp)) || (rc = A(act_xs_bytes(Rp, od), (void**)&rt.act_o.xs))) return rc;
    if ((rc = A(act_xp_bytes(Rp, c.ffn), (void**)&rt.act_f.xp)) || (rc = A(act_xs_bytes(Rp, c.ffn), (void**)&rt.act_f.xs))) return rc;
    cudaMemset(rt.act_d.xp, 0, act_xp_bytes(Rp, c.d_model));
    cudaMemset(rt.act_o.xp, 0, act_xp_bytes(Rp, od));
    cudaMemset(rt.act_f.xp, 0, act_xp_bytes(Rp, c.ffn));
    cudaMemset(rt.act_d.xs, 0, act_xs_bytes(Rp, c.d_model));
    cudaMemset(rt.act_o.xs, 0, act_xs_bytes(Rp, od));
    cudaMemset(rt.act_f.xs, 0, act_xs_bytes(Rp, c.ffn));
    rt.attn_scratch_bytes = attn_scratch_bytes(R, c.n_q_heads, c.head_dim);
    if ((rc = A(rt.attn_scratch_bytes, &rt.attn_scratch))) return rc;
    cudaMemset(rt.attn_scratch, 0, rt.attn_scratch_bytes);  // the ticket words start at zero
    rt.fed.assign(n_streams, std::vector<int32_t>());
    rt.pending.assign(n_streams, PendingVerify());
    // the many-row path: only when the session can hold that many rows and every matrix suits the kernel
    if (model->n_experts > 0) {
        // routed feed-forward: natural-layout rows around the router and the experts
        if ((rc = A((size_t)R * c.d_model * 2, (void**)&rt.w_xn)) || (rc = A((size_t)R * qkv_dim * 2, (void**)&rt.w_qkv)) ||
            (rc = A((size_t)R * c.d_model * 2, (void**)&rt.w_o)) || (rc = A((size_t)R * model->n_experts * sizeof(float), (void**)&rt.moe_logits)) ||
            (rc = A((size_t)R * model->top_k * sizeof(int32_t), (void**)&rt.moe_ids)) || (rc = A((size_t)R * model->top_k * 2, (void**)&rt.moe_w)) ||
            (rc = A((size_t)R * c.d_model * 2, (void**)&rt.moe_zero)) ||
            (rc = A(moe_ffn_workspace_bytes(R, model->top_k, model->n_experts, c.d_model, model->moe_ffn), &rt.moe_ws)))
            return rc;
        cudaMemset(rt.moe_zero, 0, (size_t)R * c.d_model * 2);
        if ((rc = A((size_t)R * sizeof(float), (void**)&rt.moe_unit_ss))) return rc;
        if ((rc = A((size_t)R * c.d_model * sizeof(float), (void**)&rt.tp_partial))) return rc;
        {
            std::vector<float> unit((size_t)R, (float)c.d_model);  // sum / d_model = 1 and eps = 0: 1/rms = 1 exactly
            TSB_CUDA(ctx, cudaMemcpy(rt.moe_unit_ss, unit.data(), unit.size() * sizeof(float), cudaMemcpyHostToDevice));
        }
        return TSB_OK;
    }
    // One matmul path per (session, model), whatever a pass's row count: the register path and the tensor-memory path
    // sum in different orders, so a model that switched between them by row count would not reproduce its own
    // single-row results in a batch (the reference's verify runs the decode path's arithmetic).  The tensor-memory path
    // is taken when the model's largest pass has WIDE_MIN_ROWS rows or more: the target's verify carries max_rows rows
    // of every stream; the drafter's largest pass is two rows per stream (a round's first step) or one stream's tree.
    const int largest_pass = is_draft ? std::max(2 * n_streams, max_rows) : R;
    bool wide = largest_pass >= WIDE_MIN_ROWS && gemm_wide_supported(model->lm_head.qtype, model->lm_head.rows, model->lm_head.cols, R);
    for (const LayerW& l : model->layers)
        wide = wide && !l.wv.data && gemm_wide_supported(l.wqkv.qtype, l.wqkv.rows, l.wqkv.cols, R) && gemm_wide_supported(l.wo.qtype, l.wo.rows, l.wo.cols, R) &&
               gemm_wide_supported(l.wgu.qtype, l.wgu.rows, l.wgu.cols, R) && gemm_wide_supported(l.wdown.qtype, l.wdown.rows, l.wdown.cols, R);
    {
        const char* env = getenv("TSB_WIDE_FORWARD");
        if (env && env[0] == '0') wide = false;
    }
    if (wide) {
        const int64_t widest = std::max<int64_t>(std::max<int64_t>(c.d_model, od), c.ffn);
        if ((rc = A((size_t)R * c.d_model * 2, (void**)&rt.w_xn)) || (rc = A((size_t)R * qkv_dim * 2, (void**)&rt.w_qkv)) ||
            (rc = A((size_t)R * od * 2, (void**)&rt.w_ao)) || (rc = A((size_t)R * c.d_model * 2, (void**)&rt.w_o)) ||
            (rc = A((size_t)R * 2 * c.ffn * 2, (void**)&rt.w_gu)) || (rc = A((size_t)R * c.ffn * 2, (void**)&rt.w_a)) ||
            (rc = A((size_t)R * c.vocab * 2, (void**)&rt.w_logits)) || (rc = A(gemm_wide_workspace_bytes(widest, R), &rt.w_ws)))
            return rc;
        size_t part = gemm_wide_partial_bytes(ctx, model->lm_head.rows, model->lm_head.cols);
        for (const LayerW& l : model->layers)
            for (const Mat* mt : {&l.wqkv, &l.wo, &l.wgu, &l.wdown}) part = std::max(part, gemm_wide_partial_bytes(ctx, mt->rows, mt->cols));
        if (part && (rc = A(part, &rt.w_part))) return rc;
        if (part) TSB_CUDA(ctx, cudaMemset(rt.w_part, 0, 4096));  // the ticket words of cut tiles
        rt.wide_ok = true;
    }
    return TSB_OK;
}

// The same pass for many rows: natural-layout f16 activations, the tensor-memory matmul, and the reference's own
// operator order and rounding points (rms_norm -> matmul -> rope/store -> attention -> o_proj -> residual + rms_norm ->
// gate|up -> silu*up -> down -> residual; crates/runtime/src/families/llama/mod.rs:205-291).
static cudaError_t forward_device_wide(tsb_session* s, ModelRt& rt, const int32_t* tokens_dev, int token_stride,
                                       const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int max_len, __half* logits,
                                       int64_t logits_stride, bool last_rows_only) {
    tsb_ctx* ctx = s->ctx;
    cudaStream_t st = s->stream;
    const tsb_model* m = rt.model;
    const tsb_model_config& c = m->cfg;
    const float scale = 1.0f / sqrtf((float)c.head_dim);
    const int64_t od = (int64_t)c.n_q_heads * c.head_dim, qkv_dim = (int64_t)(c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim;
    const ActOut none{nullptr, nullptr};
    cudaError_t e;
#define FW(x)                           \
    do {                                \
        e = (x);                        \
        if (e != cudaSuccess) return e; \
    } while (0)
    FW(launch_embed_rows(ctx, st, m->embed.qtype, m->embed.data, c.vocab, c.d_model, tokens_dev, token_stride, rows, rt.h, 1.0f));
    FW(launch_rmsnorm_rows(ctx, st, rt.h, nullptr, m->layers[0].attn_norm, rt.w_xn, none, rows, c.d_model, c.rms_eps));
    for (int L = 0; L < c.n_layers; L++) {
        const LayerW& l = m->layers[L];
        FW(launch_gemm_wide_q4k(ctx, st, l.wqkv.data, l.wqkv.rows, l.wqkv.cols, rt.w_xn, c.d_model, rows, rt.w_qkv, qkv_dim, false, rt.w_ws, rt.w_part));
        FW(launch_rope_store_kv(ctx, st, rt.kv, L, rt.w_qkv, rows_dev, rows, c.n_q_heads, c.rope_theta));
        FW(launch_attn_decode_rows(ctx, st, rt.kv, L, rt.w_qkv, qkv_dim, rt.w_ao, none, rows_dev, rows, rows_per_seq, c.n_q_heads, scale,
                                   max_len, rt.attn_scratch, s->n_streams * s->max_rows));
        FW(launch_gemm_wide_q4k(ctx, st, l.wo.data, l.wo.rows, l.wo.cols, rt.w_ao, od, rows, rt.w_o, c.d_model, false, rt.w_ws, rt.w_part));
        FW(launch_rmsnorm_rows(ctx, st, rt.h, rt.w_o, l.ffn_norm, rt.w_xn, none, rows, c.d_model, c.rms_eps));
        FW(launch_gemm_wide_q4k(ctx, st, l.wgu.data, l.wgu.rows, l.wgu.cols, rt.w_xn, c.d_model, rows, rt.w_gu, 2 * (int64_t)c.ffn, false, rt.w_ws, rt.w_part));
        FW(launch_silu_mul(ctx, st, rt.w_gu, rt.w_gu + c.ffn, rt.w_a, none, rows, c.ffn, 2 * (int64_t)c.ffn, c.ffn));
        FW(launch_gemm_wide_q4k(ctx, st, l.wdown.data, l.wdown.rows, l.wdown.cols, rt.w_a, c.ffn, rows, rt.w_o, c.d_model, false, rt.w_ws, rt.w_part));
        const void* g = L + 1 < c.n_layers ? (const void*)m->layers[L + 1].attn_norm : (const void*)m->out_norm;
        FW(launch_rmsnorm_rows(ctx, st, rt.h, rt.w_o, g, rt.w_xn, none, rows, c.d_model, c.rms_eps));
    }
    if (logits) {
        if (last_rows_only && rows_per_seq > 1) {
            // every row's logits into the staging buffer, then each stream's last row to its place
            FW(launch_gemm_wide_q4k(ctx, st, m->lm_head.data, m->lm_head.rows, m->lm_head.cols, rt.w_xn, c.d_model, rows, rt.w_logits, c.vocab,
                                    false, rt.w_ws, rt.w_part));
            FW(cudaMemcpy2DAsync(logits, (size_t)logits_stride * 2, rt.w_logits + (size_t)(rows_per_seq - 1) * c.vocab,
                                 (size_t)rows_per_seq * c.vocab * 2, (size_t)c.vocab * 2, (size_t)(rows / rows_per_seq),
                                 cudaMemcpyDeviceToDevice, st));
        } else {
            FW(launch_gemm_wide_q4k(ctx, st, m->lm_head.data, m->lm_head.rows, m->lm_head.cols, rt.w_xn, c.d_model, rows, logits, logits_stride,
                                    false, rt.w_ws, rt.w_part));
        }
    }
#undef FW
    return cudaSuccess;
}

// The pass of a model whose feed-forward is routed (crates/runtime/src/families/llama/mod.rs:205-291 with the
// feed-forward of families/llama/moe.rs:36-221): unfused operators on natural-layout f16 rows with the reference's
// rounding points; the routed sum is formed over a zero residual and added to the stream afterwards.
static cudaError_t forward_device_moe(tsb_session* s, ModelRt& rt, const int32_t* tokens_dev, int token_stride,
                                      const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int max_len, __half* logits,
                                      int64_t logits_stride, bool last_rows_only) {
    tsb_ctx* ctx = s->ctx;
    cudaStream_t st = s->stream;
    const tsb_model* m = rt.model;
    const tsb_model_config& c = m->cfg;
    const float scale = 1.0f / sqrtf((float)c.head_dim);
    const int64_t qd = (int64_t)c.n_q_heads * c.head_dim, kd = (int64_t)c.n_kv_heads * c.head_dim, qkv_dim = qd + 2 * kd;
    const ActOut none{nullptr, nullptr}, out_d{rt.act_d.xp, rt.act_d.xs}, out_o{rt.act_o.xp, rt.act_o.xs};
    const ActOperand in_d{rt.act_d.xp, rt.act_d.xs}, in_o{rt.act_o.xp, rt.act_o.xs};
    cudaError_t e;
#define FW(x)                           \
    do {                                \
        e = (x);                        \
        if (e != cudaSuccess) return e; \
    } while (0)
    // embedding rows into the residual stream plus the RoPE table of the rows' positions (the operand and the sums
    // this kernel also writes are replaced by the norm that follows)
    FW(launch_embed_norm(ctx, st, m->embed.qtype, m->embed.data, c.vocab, c.d_model, tokens_dev, token_stride, rows, rt.h,
                         m->layers[0].attn_norm, out_d, rt.ss, rt.cs, rows_dev, c.head_dim, c.rope_theta));
    FW(launch_rmsnorm_rows(ctx, st, rt.h, nullptr, m->layers[0].attn_norm, rt.w_xn, out_d, rows, c.d_model, c.rms_eps));
    for (int L = 0; L < c.n_layers; L++) {
        const LayerW& l = m->layers[L];
        {   // q|k|v over the normed operand; epilogue: f16 rounding, RoPE, q -> buffer, k and v -> cache slots
            EpiArgs a;
            a.ss_in = rt.moe_unit_ss, a.ss_parts = 1, a.d_in = c.d_model, a.eps = 0.f;
            a.kv = rt.kv->view, a.layer = L, a.row_desc = rows_dev, a.cs = rt.cs, a.q_out = rt.q;
            a.n_q_heads = c.n_q_heads, a.n_kv_heads = c.n_kv_heads, a.head_dim = c.head_dim;
            if (l.wv.data) a.n_v_heads = 0;
            FW(launch_gemm_fused(ctx, st, l.wqkv.qtype, l.wqkv.data, l.wqkv.rows, l.wqkv.cols, in_d, rows, EPI_ROPE_STORE, a));
            if (l.wv.data) {
                a.n_q_heads = 0, a.n_kv_heads = 0, a.n_v_heads = c.n_kv_heads;
                FW(launch_gemm_fused(ctx, st, l.wv.qtype, l.wv.data, l.wv.rows, l.wv.cols, in_d, rows, EPI_ROPE_STORE, a));
            }
        }
        FW(launch_attn_decode_rows(ctx, st, rt.kv, L, rt.q, qd, nullptr, out_o, rows_dev, rows, rows_per_seq, c.n_q_heads, scale,
                                   max_len, rt.attn_scratch, s->n_streams * s->max_rows));
        if (comm_world(s->comm) > 1) {
            // tensor-parallel attention: this rank's o_proj holds its heads' columns; the f32 shares are summed over the
            // ranks, then rounded to f16 once, as the single projection is
            FW(launch_gemm_quant(ctx, st, l.wo.qtype, l.wo.data, l.wo.rows, l.wo.cols, in_o, rt.tp_partial, c.d_model, rows, true));
            FW(comm_all_reduce_f32(s->comm, st, rt.tp_partial, (size_t)rows * c.d_model));
            FW(launch_f32_to_f16(ctx, st, rt.tp_partial, rt.w_o, (int64_t)rows * c.d_model));
        } else {
            FW(launch_gemm_quant(ctx, st, l.wo.qtype, l.wo.data, l.wo.rows, l.wo.cols, in_o, rt.w_o, c.d_model, rows, false));
        }
        FW(launch_rmsnorm_rows(ctx, st, rt.h, rt.w_o, l.ffn_norm, rt.w_xn, none, rows, c.d_model, c.rms_eps));
        FW(launch_router_logits(ctx, st, l.router_q, l.router_scale, l.router_bias, rt.w_xn, c.d_model, rows, m->n_experts, c.d_model, rt.moe_logits));
        FW(launch_moe_route(ctx, st, rt.moe_logits, rows, m->n_experts, m->top_k, rt.moe_ids, rt.moe_w));
        FW(launch_moe_ffn(ctx, st, l.experts_qtype, l.experts_gate_up, l.experts_down, m->n_experts, c.d_model, m->moe_ffn, rt.w_xn, c.d_model,
                          rt.moe_zero, rt.moe_ids, rt.moe_w, rows, m->top_k, nullptr, rt.moe_ws, m->expert_lo, m->n_local_experts));
        // sharded experts: every (row, slot) value was computed by exactly one rank, the others hold zero there - the
        // sum over the ranks is exact, and the slot-ordered combine below sees the values of a single GPU
        if (m->n_local_experts > 0)
            FW(comm_all_reduce_f32(s->comm, st, const_cast<float*>(moe_ffn_values(rt.moe_ws, rows, m->top_k, m->n_experts, c.d_model, m->moe_ffn)),
                                   (size_t)rows * m->top_k * c.d_model));
        // the slot-ordered weighted sum (over a zero residual, rounded to f16), its add onto the stream and the next norm
        const void* g = L + 1 < c.n_layers ? (const void*)m->layers[L + 1].attn_norm : (const void*)m->out_norm;
        FW(launch_combine_norm_rows(ctx, st, rt.h, moe_ffn_values(rt.moe_ws, rows, m->top_k, m->n_experts, c.d_model, m->moe_ffn), rt.moe_w,
                                    m->top_k, g, rt.w_xn, out_d, rows, c.d_model, c.rms_eps));
    }
    if (logits) {
        EpiArgs a;
        a.y = logits, a.y_stride = logits_stride, a.y_f32 = 0;
        a.y_every = last_rows_only ? rows_per_seq : 0;
        FW(launch_gemm_fused(ctx, st, m->lm_head.qtype, m->lm_head.data, m->lm_head.rows, m->lm_head.cols, in_d, rows, EPI_PLAIN, a));
    }
#undef FW
    return cudaSuccess;
}

// Which launches of a pass forward_device enqueues: all of them, or - for the two timing entry points - only the
// layer matmuls / everything but the layer matmuls.
enum { PASS_ALL = 0, PASS_MATMULS = 1, PASS_REST = 2 };

// One forward pass over `rows` rows (rows_per_seq per stream).  Row descriptors and token ids are
// already on the device.  Cursors are not touched here.
static cudaError_t forward_device(tsb_session* s, ModelRt& rt, const int32_t* tokens_dev, int token_stride,
                                  const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int max_len, __half* logits,
                                  int64_t logits_stride, bool last_rows_only = false, int only = PASS_ALL) {
    if (s->replay) return cudaSuccess;  // the captured graph already holds this work
    const bool matmuls_only = only == PASS_MATMULS, skip_matmuls = only == PASS_REST;
    if (rt.model->n_experts > 0)
        return forward_device_moe(s, rt, tokens_dev, token_stride, rows_dev, rows, rows_per_seq, (max_len + 511) / 512 * 512, logits,
                                  logits_stride, last_rows_only);
    if (rt.wide_ok && only == PASS_ALL)
        return forward_device_wide(s, rt, tokens_dev, token_stride, rows_dev, rows, rows_per_seq, (max_len + 511) / 512 * 512, logits,
                                   logits_stride, last_rows_only);
    tsb_ctx* ctx = s->ctx;
    cudaStream_t st = s->stream;
    const tsb_model* m = rt.model;
    const tsb_model_config& c = m->cfg;
    const float scale = 1.0f / sqrtf((float)c.head_dim);
    max_len = (max_len + 511) / 512 * 512;  // the split plan changes only every 512 positions (graph reuse)
    cudaError_t e;
#define FW(x)                         \
    do {                              \
        e = (x);                      \
        if (e != cudaSuccess) return e; \
    } while (0)
    const ActOut out_d{rt.act_d.xp, rt.act_d.xs}, out_o{rt.act_o.xp, rt.act_o.xs}, out_f{rt.act_f.xp, rt.act_f.xs};
    const ActOperand in_d{rt.act_d.xp, rt.act_d.xs}, in_o{rt.act_o.xp, rt.act_o.xs}, in_f{rt.act_f.xp, rt.act_f.xs};
    const int R = s->n_streams * s->max_rows;
    const int parts = c.d_model / 16;
    auto ss_slot = [&](int i) { return rt.ss + (size_t)i * R * parts; };
    // (PASS_MATMULS / PASS_REST: the measurement aids - only the layer matmuls with their real epilogues, or only the
    // other launches of the pass (embedding, attention, head), over whatever the buffers hold)
    // embedding: residual stream, layer 0's operand f16(h * g), sum of h^2 (one partial per row), RoPE table
    if (!matmuls_only) FW(launch_embed_norm(ctx, st, m->embed.qtype, m->embed.data, c.vocab, c.d_model, tokens_dev, token_stride, rows, rt.h,
                         m->layers[0].attn_norm, out_d, ss_slot(0), rt.cs, rows_dev, c.head_dim, c.rope_theta));
    for (int L = 0; L < c.n_layers; L++) {
        const LayerW& l = m->layers[L];
        if (!skip_matmuls) {   // q|k|v matmul; epilogue: 1/rms, RoPE, q -> buffer, k and v -> cache slots
            EpiArgs a;
            a.ss_in = ss_slot(2 * L), a.ss_parts = L == 0 ? 1 : parts, a.d_in = c.d_model, a.eps = c.rms_eps;
            a.kv = rt.kv->view, a.layer = L, a.row_desc = rows_dev, a.cs = rt.cs, a.q_out = rt.q;
            a.n_q_heads = c.n_q_heads, a.n_kv_heads = c.n_kv_heads, a.head_dim = c.head_dim;
            if (l.wv.data) a.n_v_heads = 0;
            FW(launch_gemm_fused(ctx, st, l.wqkv.qtype, l.wqkv.data, l.wqkv.rows, l.wqkv.cols, in_d, rows, EPI_ROPE_STORE, a));
            if (l.wv.data) {  // v in its own block format: the v rows as a second launch, every tile a v tile
                a.n_q_heads = 0, a.n_kv_heads = 0, a.n_v_heads = c.n_kv_heads;
                FW(launch_gemm_fused(ctx, st, l.wv.qtype, l.wv.data, l.wv.rows, l.wv.cols, in_d, rows, EPI_ROPE_STORE, a));
            }
        }
        if (!matmuls_only)
            FW(launch_attn_decode_rows(ctx, st, rt.kv, L, rt.q, (int64_t)c.n_q_heads * c.head_dim, nullptr, out_o, rows_dev, rows,
                                       rows_per_seq, c.n_q_heads, scale, max_len, rt.attn_scratch, s->n_streams * s->max_rows));
        if (skip_matmuls) continue;
        {   // o_proj; epilogue: residual add, next operand f16(h * g_ffn), partial sums of h^2
            EpiArgs a;
            a.h = rt.h, a.g = l.ffn_norm, a.out = out_d, a.ss_out = ss_slot(2 * L + 1);
            FW(launch_gemm_fused(ctx, st, l.wo.qtype, l.wo.data, l.wo.rows, l.wo.cols, in_o, rows, EPI_RESID_NORM, a));
        }
        {   // gate|up matmul; epilogue: 1/rms, SiLU(gate) * up -> operand of the down projection
            EpiArgs a;
            a.ss_in = ss_slot(2 * L + 1), a.ss_parts = parts, a.d_in = c.d_model, a.eps = c.rms_eps, a.out = out_f;
            FW(launch_gemm_fused(ctx, st, l.wgu.qtype, l.wgu.data, l.wgu.rows, l.wgu.cols, in_d, rows, EPI_SILU, a));
        }
        {   // down projection; epilogue: residual add, operand for the next layer's norm (or the final norm)
            EpiArgs a;
            a.h = rt.h, a.g = L + 1 < c.n_layers ? m->layers[L + 1].attn_norm : m->out_norm, a.out = out_d;
            a.ss_out = ss_slot(2 * L + 2);
            FW(launch_gemm_fused(ctx, st, l.wdown.qtype, l.wdown.data, l.wdown.rows, l.wdown.cols, in_f, rows, EPI_RESID_NORM, a));
        }
    }
    if (logits && !matmuls_only) {
        // head over the final-normed operand; row t of the logits sits at logits + t * logits_stride
        EpiArgs a;
        a.ss_in = ss_slot(2 * c.n_layers), a.ss_parts = parts, a.d_in = c.d_model, a.eps = c.rms_eps;
        a.y = logits, a.y_stride = logits_stride, a.y_f32 = 0;
        a.y_every = last_rows_only ? rows_per_seq : 0;  // logits of each stream's last row only, one output row per stream
        FW(launch_gemm_fused(ctx, st, m->lm_head.qtype, m->lm_head.data, m->lm_head.rows, m->lm_head.cols, in_d, rows, EPI_SCALE, a));
    }
#undef FW
    return cudaSuccess;
}

// Host side of a forward: descriptors for `n_active` streams x rows_per_seq rows, uploaded through the
// pinned staging ring.  parent == nullptr: a chain.  Returns the device pointers.
static int32_t stage_rows(tsb_session* s, ModelRt& rt, const int32_t* streams, int n_active, int rows_per_seq,
                          const int32_t* slot_parent, const int32_t* tokens_host /* may be null */,
                          const tsb_row_desc** rows_dev, const int32_t** tokens_dev, int* max_len) {
    tsb_ctx* ctx = s->ctx;
    const int rows = n_active * rows_per_seq;
    TSB_REQUIRE(ctx, rows <= s->n_streams * s->max_rows, "%d rows exceed the session's %d", rows, s->n_streams * s->max_rows);
    TSB_REQUIRE(ctx, rows_per_seq <= 128, "at most 128 in-flight rows per stream");
    if (s->stage_used + rows > s->stage_cap) {
        if (s->replay || s->capturing) return tsb_fail(ctx, TSB_ERR_STATE, "staging ring overflow inside a captured round");
        // the ring is reused only after the work that read it has finished
        TSB_CUDA(ctx, cudaStreamSynchronize(s->stream));
        s->stage_used = 0;
    }
    tsb_row_desc* hd = s->stage_rows_host + s->stage_used;
    int32_t* ht = s->stage_tok_host + s->stage_used;
    std::vector<int> depth(rows_per_seq, 0);
    std::vector<uint64_t> mlo(rows_per_seq, 0), mhi(rows_per_seq, 0);
    for (int j = 0; j < rows_per_seq; j++) {
        if (slot_parent) {
            if (j == 0) {
                TSB_REQUIRE(ctx, slot_parent[0] == -1, "a tree's slot 0 is the anchor (parent -1)");
            } else {
                const int p = slot_parent[j];
                TSB_REQUIRE(ctx, p >= 0 && p < j, "slot %d's parent %d must precede it", j, p);
                depth[j] = depth[p] + 1;
                mlo[j] = mlo[p], mhi[j] = mhi[p];
            }
        } else {
            depth[j] = j;
            if (j) mlo[j] = mlo[j - 1], mhi[j] = mhi[j - 1];
        }
        if (j < 64) mlo[j] |= 1ull << j; else mhi[j] |= 1ull << (j - 64);
    }
    int ml = 0;
    for (int a = 0; a < n_active; a++) {
        const int seq = streams[a];
        TSB_REQUIRE(ctx, seq >= 0 && seq < s->n_streams, "stream %d outside the session", seq);
        const int64_t base = tsb_kv_cursor(rt.kv, seq);
        if (base + rows_per_seq > rt.model->cfg.max_context)
            return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: %lld + %d rows exceed the context window %d", seq, (long long)base,
                            rows_per_seq, rt.model->cfg.max_context);
        int32_t rc = tsb_kv_reserve(rt.kv, seq, base + rows_per_seq);
        if (rc) return rc;
        for (int j = 0; j < rows_per_seq; j++) {
            tsb_row_desc& d = hd[a * rows_per_seq + j];
            d.seq = seq, d.base = (int32_t)base, d.slot = j, d.position = (int32_t)base + depth[j];
            d.mask[0] = mlo[j], d.mask[1] = mhi[j];
            if (tokens_host) ht[a * rows_per_seq + j] = tokens_host[a * rows_per_seq + j];
        }
        ml = ml > (int)base + rows_per_seq ? ml : (int)base + rows_per_seq;
    }
    tsb_row_desc* dd = s->stage_rows_dev + s->stage_used;
    int32_t* dt = s->stage_tok_dev + s->stage_used;
    if (!s->replay) {
        TSB_CUDA(ctx, cudaMemcpyAsync(dd, hd, rows * sizeof(tsb_row_desc), cudaMemcpyHostToDevice, s->stream));
        if (tokens_host) TSB_CUDA(ctx, cudaMemcpyAsync(dt, ht, rows * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    }
    s->stage_used += rows;
    *rows_dev = dd;
    if (tokens_dev) *tokens_dev = dt;
    *max_len = ml;
    return TSB_OK;
}

extern "C" {
static int32_t drafter_catch_up(tsb_session* s, int stream, int64_t upto);
}

// forward + cursor advance for one stream (the single-stream producer calls)
static int32_t forward_stream(tsb_session* s, ModelRt& rt, int stream, const int32_t* tokens, int n, const int32_t* slot_parent,
                              __half* logits_dev, void* logits_out_host) {
    tsb_ctx* ctx = s->ctx;
    const tsb_row_desc* rd;
    const int32_t* td;
    int max_len;
    int32_t rc = stage_rows(s, rt, &stream, 1, n, slot_parent, tokens, &rd, &td, &max_len);
    if (rc) return rc;
    const int vocab = rt.model->cfg.vocab;
    TSB_CUDA(ctx, forward_device(s, rt, td, 1, rd, n, n, max_len, logits_dev, vocab));
    tsb_kv_set_cursor(rt.kv, stream, tsb_kv_cursor(rt.kv, stream) + n);
    if (logits_dev && logits_out_host)
        TSB_CUDA(ctx, cudaMemcpyAsync(logits_out_host, logits_dev, (size_t)n * vocab * 2, cudaMemcpyDeviceToHost, s->stream));
    if (logits_out_host) return tsb_stream_sync(ctx, s->stream);
    return TSB_OK;
}

extern "C" {

int32_t tsb_session_create(tsb_ctx* ctx, const tsb_model* target, const tsb_model* draft, int32_t n_streams,
                           int32_t max_rows, int32_t page_tokens, tsb_session** out) {
    if (!ctx || !target || !out) return TSB_ERR_INVALID;
    *out = nullptr;
    TSB_REQUIRE(ctx, n_streams > 0 && max_rows > 0 && max_rows <= 128, "n_streams must be positive and max_rows in 1..128");
    int32_t rc = model_complete(target);
    if (rc) return rc;
    if (draft) {
        if ((rc = model_complete(draft))) return rc;
        TSB_REQUIRE(ctx, draft->cfg.vocab == target->cfg.vocab, "the drafter must share the target's vocabulary");
    }
    if (target->cfg.vocab > accept_max_vocab())
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "vocabulary %d exceeds the device sampler's %d", target->cfg.vocab, accept_max_vocab());
    DeviceGuard g(ctx);
    tsb_session* s = new (std::nothrow) tsb_session();
    if (!s) return TSB_ERR_OOM;
    s->ctx = ctx, s->n_streams = n_streams, s->max_rows = max_rows;
    s->generated.assign(n_streams, 0);
    auto fail = [&](int32_t code) {
        tsb_session_destroy(s);
        return code;
    };
    if (cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess) return fail(TSB_ERR_CUDA);
    for (auto& ev : s->ev)
        if (cudaEventCreate(&ev) != cudaSuccess) return fail(TSB_ERR_CUDA);
    if ((rc = runtime_init(s, s->target, target, n_streams, max_rows, page_tokens, false))) return fail(rc);
    if (draft && (rc = runtime_init(s, s->draft, draft, n_streams, max_rows, page_tokens, true))) return fail(rc);
    s->has_draft = draft != nullptr;
    {
        const char* env = getenv("TSB_GRAPH");
        if (env && env[0] == '0') s->use_graph = false;
    }
    const int R = n_streams * max_rows, V = target->cfg.vocab;
    auto A = [&](size_t bytes, void** p) { return dev_alloc(ctx, s->owned, bytes, p); };
    if ((rc = A((size_t)R * V * 2, (void**)&s->logits_target))) return fail(rc);
    if ((rc = A((size_t)R * V * 2, (void**)&s->logits_draft))) return fail(rc);
    if ((rc = A((size_t)(R + 2 * n_streams) * sizeof(int32_t), (void**)&s->feed_dev))) return fail(rc);
    s->pair_dev = s->feed_dev + R;
    if ((rc = A((size_t)n_streams * (3 * max_rows + 2) * sizeof(uint64_t), (void**)&s->uniforms_dev))) return fail(rc);
    if ((rc = A((size_t)n_streams * sizeof(tsb_accept_out), (void**)&s->accept_out_dev))) return fail(rc);
    s->accept_scratch_bytes = accept_scratch_bytes(n_streams, max_rows, V);
    if ((rc = A(s->accept_scratch_bytes, &s->accept_scratch))) return fail(rc);
    if ((rc = A((size_t)n_streams * sizeof(int32_t), (void**)&s->tok1_dev))) return fail(rc);
    if ((rc = A((size_t)128 * 9 * sizeof(int32_t), (void**)&s->tree_dev))) return fail(rc);
    // pinned staging: descriptors and tokens of several forwards in flight
    s->stage_cap = R * (2 * max_rows + 8);
    if (cudaMallocHost((void**)&s->stage_rows_host, (size_t)s->stage_cap * sizeof(tsb_row_desc)) != cudaSuccess) return fail(TSB_ERR_CUDA);
    if (cudaMallocHost((void**)&s->stage_tok_host, (size_t)s->stage_cap * sizeof(int32_t)) != cudaSuccess) return fail(TSB_ERR_CUDA);
    if ((rc = A((size_t)s->stage_cap * sizeof(tsb_row_desc), (void**)&s->stage_rows_dev))) return fail(rc);
    if ((rc = A((size_t)s->stage_cap * sizeof(int32_t), (void**)&s->stage_tok_dev))) return fail(rc);
    if (cudaMallocHost((void**)&s->accept_out_host, (size_t)n_streams * sizeof(tsb_accept_out)) != cudaSuccess) return fail(TSB_ERR_CUDA);
    if (cudaMallocHost((void**)&s->uniforms_host, (size_t)n_streams * (3 * max_rows + 2) * sizeof(uint64_t)) != cudaSuccess) return fail(TSB_ERR_CUDA);
    if (cudaMallocHost((void**)&s->feed_host, (size_t)(R + 2 * n_streams) * sizeof(int32_t)) != cudaSuccess) return fail(TSB_ERR_CUDA);
    s->pair_host = s->feed_host + R;
    if (cudaMallocHost((void**)&s->logits_host, (size_t)V * 2) != cudaSuccess) return fail(TSB_ERR_CUDA);
    *out = s;
    return TSB_OK;
}

void tsb_session_destroy(tsb_session* s) {
    if (!s) return;
    DeviceGuard g(s->ctx);
    cudaDeviceSynchronize();
    if (s->graph) cudaGraphExecDestroy(s->graph);
    for (void* p : s->owned) tsb_free(s->ctx, p);
    if (s->target.kv) tsb_kv_destroy(s->target.kv);
    if (s->draft.kv) tsb_kv_destroy(s->draft.kv);
    cudaFreeHost(s->stage_rows_host), cudaFreeHost(s->stage_tok_host), cudaFreeHost(s->accept_out_host);
    cudaFreeHost(s->uniforms_host), cudaFreeHost(s->feed_host), cudaFreeHost(s->logits_host);
    for (auto& ev : s->ev)
        if (ev) cudaEventDestroy(ev);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

int32_t tsb_session_set_comm(tsb_session* s, tsb_comm* c) {
    if (!s) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    TSB_CUDA(s->ctx, cudaStreamSynchronize(s->stream));
    if (s->graph) cudaGraphExecDestroy(s->graph), s->graph = nullptr;  // captured rounds hold the old exchange steps
    s->comm = c;
    return TSB_OK;
}

tsb_kv* tsb_session_kv(tsb_session* s, int32_t which) { return !s ? nullptr : (which == 0 ? s->target.kv : s->draft.kv); }

// ---- LogitProducer / SpeculativeProducer, one stream ----------------------

int32_t tsb_producer_reset(tsb_session* s, int32_t stream) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    DeviceGuard g(s->ctx);
    TSB_CUDA(s->ctx, cudaStreamSynchronize(s->stream));
    int32_t rc = tsb_kv_reset(s->target.kv, stream);
    if (rc) return rc;
    s->target.fed[stream].clear();
    s->target.pending[stream] = PendingVerify();
    s->generated[stream] = 0;
    if (s->has_draft) {
        if ((rc = tsb_kv_reset(s->draft.kv, stream))) return rc;
    }
    return TSB_OK;
}

int32_t tsb_session_set_generated(tsb_session* s, int32_t stream, int32_t generated) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams && generated >= 0, "bad stream or count");
    s->generated[stream] = generated;
    return TSB_OK;
}

static int32_t check_position(tsb_session* s, ModelRt& rt, int stream, int64_t position) {
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    const int64_t cur = tsb_kv_cursor(rt.kv, stream);
    if (position != cur)  // crates/runtime/src/families/qwen/batched.rs:150-160: start must equal the cursor
        return tsb_fail(s->ctx, TSB_ERR_STATE, "position %lld does not continue the cache (cursor %lld)", (long long)position,
                        (long long)cur);
    return TSB_OK;
}

static void record_fed(ModelRt& rt, int stream, int64_t position, const int32_t* tokens, int n) {
    auto& f = rt.fed[stream];
    f.resize((size_t)position);
    f.insert(f.end(), tokens, tokens + n);
}

int32_t tsb_producer_produce(tsb_session* s, int32_t stream, int32_t token, int64_t position, void* logits_out_host) {
    if (!s) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    int32_t rc = check_position(s, s->target, stream, position);
    if (rc) return rc;
    record_fed(s->target, stream, position, &token, 1);
    return forward_stream(s, s->target, stream, &token, 1, nullptr, s->logits_target, logits_out_host);
}

int32_t tsb_producer_produce_prefill(tsb_session* s, int32_t stream, int32_t token, int64_t position) {
    if (!s) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    int32_t rc = check_position(s, s->target, stream, position);
    if (rc) return rc;
    record_fed(s->target, stream, position, &token, 1);
    return forward_stream(s, s->target, stream, &token, 1, nullptr, nullptr, nullptr);
}

// the drafter is a stand-alone decoder: bring its cache up to `upto` from the record of fed tokens
static int32_t drafter_catch_up(tsb_session* s, int stream, int64_t upto) {
    ModelRt& d = s->draft;
    const auto& fed = s->target.fed[stream];
    while (tsb_kv_cursor(d.kv, stream) < upto) {
        const int64_t p = tsb_kv_cursor(d.kv, stream);
        if ((size_t)p >= fed.size()) return tsb_fail(s->ctx, TSB_ERR_STATE, "drafter position %lld was never fed to the target", (long long)p);
        int64_t n64 = upto - p;
        if (n64 > s->max_rows) n64 = s->max_rows;
        if (n64 > (int64_t)fed.size() - p) n64 = (int64_t)fed.size() - p;
        const int n = (int)n64;
        int32_t rc = forward_stream(s, d, stream, fed.data() + p, n, nullptr, nullptr, nullptr);
        if (rc) return rc;
    }
    return TSB_OK;
}

static int32_t drafter_step(tsb_session* s, int32_t stream, int32_t next, int64_t position, bool head, void* logits_out_host) {
    if (!s) return TSB_ERR_INVALID;
    if (!s->has_draft) return tsb_fail(s->ctx, TSB_ERR_STATE, "the session has no drafter");
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    DeviceGuard g(s->ctx);
    int32_t rc = drafter_catch_up(s, stream, position + 1);
    if (rc) return rc;
    if ((rc = check_position(s, s->draft, stream, position + 1))) return rc;
    return forward_stream(s, s->draft, stream, &next, 1, nullptr, head ? s->logits_draft : nullptr, logits_out_host);
}

int32_t tsb_producer_prime_drafter(tsb_session* s, int32_t stream, int32_t next, int64_t position) {
    return drafter_step(s, stream, next, position, false, nullptr);
}
int32_t tsb_producer_draft_step(tsb_session* s, int32_t stream, int32_t next, int64_t position, void* logits_out_host) {
    return drafter_step(s, stream, next, position, true, logits_out_host);
}

int32_t tsb_producer_verify(tsb_session* s, int32_t stream, const int32_t* feed, int32_t n, int64_t base, void* logits_out_host) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, feed && n > 0 && n <= s->max_rows, "verify takes 1..%d rows", s->max_rows);
    DeviceGuard g(s->ctx);
    int32_t rc = check_position(s, s->target, stream, base);
    if (rc) return rc;
    record_fed(s->target, stream, base, feed, n);
    PendingVerify& pv = s->target.pending[stream];
    pv.active = true, pv.tree = false, pv.base = base, pv.rows = n, pv.feed.clear(), pv.drafter_rows = 0;
    return forward_stream(s, s->target, stream, feed, n, nullptr, s->logits_target, logits_out_host);
}

int32_t tsb_producer_verify_tree(tsb_session* s, int32_t stream, const int32_t* feed, const int32_t* slot_parent, int32_t n,
                                 int64_t base, void* logits_out_host) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, feed && slot_parent && n > 0 && n <= s->max_rows, "verify_tree takes 1..%d rows", s->max_rows);
    DeviceGuard g(s->ctx);
    int32_t rc = check_position(s, s->target, stream, base);
    if (rc) return rc;
    // the slots' tokens are kept until compact_tree says which of them form the accepted path
    PendingVerify& pv = s->target.pending[stream];
    const int drafted = pv.active && pv.tree && pv.base == base && pv.rows == 0 ? pv.drafter_rows : 0;  // left by draft_tree
    pv.active = true, pv.tree = true, pv.base = base, pv.rows = n, pv.feed.assign(feed, feed + n), pv.drafter_rows = drafted;
    return forward_stream(s, s->target, stream, feed, n, slot_parent, s->logits_target, logits_out_host);
}

int32_t tsb_session_verify_tree(tsb_session* s, const int32_t* feed, const int32_t* slot_parent, int32_t n, void* logits_out_host) {
    if (!s) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, feed && slot_parent && n > 0 && n <= s->max_rows, "verify_tree takes 1..%d rows per stream", s->max_rows);
    DeviceGuard g(ctx);
    const int S = s->n_streams;
    std::vector<int32_t> streams(S);
    for (int b = 0; b < S; b++) streams[b] = b;
    const tsb_row_desc* rd;
    const int32_t* td;
    int max_len;
    int32_t rc = stage_rows(s, s->target, streams.data(), S, n, slot_parent, feed, &rd, &td, &max_len);
    if (rc) return rc;
    const int vocab = s->target.model->cfg.vocab;
    TSB_CUDA(ctx, forward_device(s, s->target, td, 1, rd, S * n, n, max_len, s->logits_target, vocab));
    for (int b = 0; b < S; b++) {
        const int64_t base = tsb_kv_cursor(s->target.kv, b);
        PendingVerify& pv = s->target.pending[b];
        pv.active = true, pv.tree = true, pv.base = base, pv.rows = n, pv.feed.assign(feed + (size_t)b * n, feed + (size_t)(b + 1) * n), pv.drafter_rows = 0;
        tsb_kv_set_cursor(s->target.kv, b, base + n);
    }
    if (logits_out_host) {
        TSB_CUDA(ctx, cudaMemcpyAsync(logits_out_host, s->logits_target, (size_t)S * n * vocab * 2, cudaMemcpyDeviceToHost, s->stream));
        return tsb_stream_sync(ctx, s->stream);
    }
    return TSB_OK;
}

int32_t tsb_producer_compact_tree(tsb_session* s, int32_t stream, int64_t base, const uint32_t* path, int32_t keep) {
    if (!s) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    PendingVerify& pv = s->target.pending[stream];
    if (!pv.active || !pv.tree || pv.base != base)
        return tsb_fail(ctx, TSB_ERR_STATE, "compact_tree at %lld has no tree verify to compact", (long long)base);
    TSB_REQUIRE(ctx, path && keep >= 1 && keep <= pv.rows && path[0] == 0, "the path starts at slot 0 and has 1..%d entries", pv.rows);
    for (int r = 1; r < keep; r++) TSB_REQUIRE(ctx, path[r] > path[r - 1] && (int)path[r] < pv.rows, "path entries increase and stay inside the verify");
    DeviceGuard g(ctx);
    int32_t rc = tsb_kv_commit_path(ctx, s->stream, s->target.kv, stream, base, path, keep);
    if (rc) return rc;
    // the drafter holds rows only for the slots it was run over: the part of the path it has is compacted too, the
    // rest is replayed from the record of fed tokens before its next step
    int dkeep = 0;
    if (s->has_draft && pv.drafter_rows > 0 && tsb_kv_cursor(s->draft.kv, stream) == base) {
        while (dkeep < keep && (int)path[dkeep] < pv.drafter_rows) dkeep++;
        if (dkeep > 0 && (rc = tsb_kv_commit_path(ctx, s->stream, s->draft.kv, stream, base, path, dkeep))) return rc;
    }
    if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
    // the verify left the cursor past every slot; the kept rows now sit at base .. base + keep
    if (dkeep > 0) tsb_kv_set_cursor(s->draft.kv, stream, base + dkeep);
    auto& fed = s->target.fed[stream];
    if ((int64_t)fed.size() < base) return tsb_fail(ctx, TSB_ERR_STATE, "the record of fed tokens ends before %lld", (long long)base);
    fed.resize((size_t)base);
    for (int r = 0; r < keep; r++) fed.push_back(pv.feed[path[r]]);
    // the slots past the path are dropped from the record; their cache rows are cut by rollback_retaining
    pv.tree = false, pv.feed.clear();  // compacted: what remains pending is a chain of pv.rows rows, of which `keep` matter
    return TSB_OK;
}

int64_t tsb_producer_checkpoint(tsb_session* s, int32_t stream) { return s ? tsb_kv_cursor(s->target.kv, stream) : -1; }

int32_t tsb_producer_rollback(tsb_session* s, int32_t stream, int64_t point) {
    return tsb_producer_rollback_retaining(s, stream, point, 0);
}

// crates/runtime/src/real_forward_rollback.rs:268-405 for a pure-attention model: a cursor move.
int32_t tsb_producer_rollback_retaining(tsb_session* s, int32_t stream, int64_t point, int32_t keep_rows) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    const int64_t cur = tsb_kv_cursor(s->target.kv, stream);
    if (point < 0 || keep_rows < 0 || point + keep_rows > cur)
        return tsb_fail(s->ctx, TSB_ERR_STATE, "cannot keep %d rows after %lld: the cursor is %lld", keep_rows, (long long)point,
                        (long long)cur);
    // the record of fed tokens is only ever cut here: rows nobody recorded cannot be kept
    if ((int64_t)s->target.fed[stream].size() < point + keep_rows)
        return tsb_fail(s->ctx, TSB_ERR_STATE, "the record of fed tokens holds %zu entries, fewer than the %lld rows to keep "
                        "(after verify_tree, compact_tree comes first)", s->target.fed[stream].size(), (long long)(point + keep_rows));
    int32_t rc = tsb_kv_set_cursor(s->target.kv, stream, point + keep_rows);
    if (rc) return rc;
    s->target.fed[stream].resize((size_t)(point + keep_rows));
    return TSB_OK;
}

int32_t tsb_producer_commit_pending(tsb_session* s, int32_t stream, int32_t keep_rows) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    PendingVerify& pv = s->target.pending[stream];
    if (!pv.active) return TSB_OK;
    if (keep_rows < 0 || keep_rows > pv.rows)
        return tsb_fail(s->ctx, TSB_ERR_STATE, "commit_pending(%d): the last verify fed %d rows", keep_rows, pv.rows);
    pv = PendingVerify();
    return TSB_OK;
}

int32_t tsb_producer_discard_pending(tsb_session* s, int32_t stream) {
    if (!s) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    PendingVerify& pv = s->target.pending[stream];
    if (!pv.active) return TSB_OK;
    DeviceGuard g(s->ctx);
    cudaStreamSynchronize(s->stream);  // whatever the failed round enqueued is over before the cursors move
    const int64_t base = pv.base;
    pv = PendingVerify();
    if (tsb_kv_cursor(s->target.kv, stream) > base) tsb_kv_set_cursor(s->target.kv, stream, base);
    if (s->target.fed[stream].size() > (size_t)base) s->target.fed[stream].resize((size_t)base);
    if (s->has_draft && tsb_kv_cursor(s->draft.kv, stream) > base + 1) tsb_kv_set_cursor(s->draft.kv, stream, base + 1);
    return TSB_OK;
}

int32_t tsb_producer_supports_retaining_rollback(const tsb_session* s) { return s ? 1 : 0; }
int32_t tsb_producer_supports_headless_prefill(const tsb_session* s) { return s ? 1 : 0; }
int32_t tsb_producer_drafts_block_passes(const tsb_session* s) {
    (void)s;
    return 0;
}

int32_t tsb_session_set_tree(tsb_session* s, int32_t nodes, int32_t levels, const int32_t* branching, int32_t best_first, int32_t cand) {
    if (!s) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TreeShape t;
    if (nodes == 0) {
        s->tree = t;
        return TSB_OK;
    }
    TSB_REQUIRE(ctx, nodes >= 1 && nodes + 1 <= s->max_rows && nodes + 1 <= 128, "a tree of %d nodes plus the anchor exceeds the session's %d rows", nodes, s->max_rows);
    TSB_REQUIRE(ctx, levels >= 1 && levels <= 8, "levels must be 1..8");
    t.nodes = nodes, t.levels = levels, t.best_first = best_first ? 1 : 0, t.cand = cand;
    if (best_first) {
        TSB_REQUIRE(ctx, cand >= 1 && cand <= 8, "cand must be 1..8");
    } else {
        TSB_REQUIRE(ctx, branching != nullptr, "a static tree needs its branching list");
        for (int l = 0; l < levels; l++) {
            TSB_REQUIRE(ctx, branching[l] >= 1 && branching[l] <= 8, "branching must be 1..8");
            t.branching[l] = branching[l];
        }
    }
    s->tree = t;
    return TSB_OK;
}

int32_t tsb_producer_tree_nodes(const tsb_session* s) { return s ? s->tree.nodes : 0; }

int32_t tsb_tree_slot_parents(const tsb_tree_node* tree, int32_t n, int32_t* out) {
    if ((!tree && n) || !out || n < 0) return TSB_ERR_INVALID;
    out[0] = -1;
    for (int i = 0; i < n; i++) out[i + 1] = tree[i].parent < 0 ? 0 : tree[i].parent + 1;
    return TSB_OK;
}

int32_t tsb_best_first_tree(const float* scores, int32_t depth_max, int32_t branch, int32_t nodes, tsb_tree_node* out) {
    if (!scores || !out || branch <= 0) return 0;
    std::vector<tsb_tree_node> t;
    best_first_tree(depth_max, nodes, branch,
                    [&](int depth, int /*parent*/, float* sc) -> int32_t {
                        for (int c = 0; c < branch; c++) sc[c] = scores[(size_t)depth * branch + c];
                        return 0;
                    },
                    t);
    std::copy(t.begin(), t.end(), out);
    return (int32_t)t.size();
}

int32_t tsb_tree_accept(const tsb_tree_node* tree, const int32_t* tokens, int32_t n, const int32_t* target_pick, int32_t* accepted_out) {
    if ((!tree && n) || (!tokens && n) || !target_pick || !accepted_out || n < 0) return 0;
    int at = -1, k = 0;
    for (;;) {
        const int32_t want = target_pick[at + 1];
        int hit = -1;
        for (int id = 0; id < n && hit < 0; id++)
            if (tree[id].parent == at && tokens[id] == want) hit = id;
        if (hit < 0) return k;
        accepted_out[k++] = hit;
        at = hit;
    }
}

int32_t tsb_producer_draft_tree(tsb_session* s, int32_t stream, int32_t anchor, int64_t base, int32_t nodes, tsb_tree_node* tree_out,
                                int32_t* tokens_out, int32_t* n_out) {
    if (!s || !tree_out || !tokens_out || !n_out) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    if (s->tree.nodes == 0) return tsb_fail(ctx, TSB_ERR_STATE, "this producer verifies chains only (tsb_session_set_tree turns trees on)");
    TSB_REQUIRE(ctx, nodes >= 1 && nodes <= s->tree.nodes, "nodes must be 1..%d", s->tree.nodes);
    DeviceGuard g(ctx);
    TreeShape shape = s->tree;
    shape.nodes = nodes;
    std::vector<int32_t> feed, parent;
    std::vector<tsb_tree_node> tree;
    int drafter_rows = 0;
    int32_t rc = session_draft_tree(s, stream, shape, anchor, base, feed, parent, tree, &drafter_rows);
    if (rc) return rc;
    for (size_t i = 0; i < tree.size(); i++) tree_out[i] = tree[i], tokens_out[i] = feed[i + 1];
    *n_out = (int32_t)tree.size();
    // remembered for the verify_tree / compact_tree that follow: which slots the drafter's cache holds
    PendingVerify& pv = s->target.pending[stream];
    pv = PendingVerify();
    pv.active = true, pv.tree = true, pv.base = base, pv.rows = 0, pv.drafter_rows = drafter_rows;
    return TSB_OK;
}

int32_t tsb_producer_draft_block(tsb_session* s, int32_t stream, int32_t anchor, int64_t base, int32_t block, int32_t* proposals_out) {
    if (!s || !proposals_out) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    if (!s->has_draft) return tsb_fail(ctx, TSB_ERR_STATE, "the session has no drafter");
    TSB_REQUIRE(ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    TSB_REQUIRE(ctx, block >= 1 && block <= 15, "block must be 1..=15");
    DeviceGuard g(ctx);
    const int V = s->draft.model->cfg.vocab;
    int32_t tok = anchor;
    for (int i = 0; i <= block; i++) {
        // step i feeds the token at base + i; its logits give proposal i (the last step is taken for its row alone)
        int32_t rc = drafter_step(s, stream, tok, base + i - 1, i < block, nullptr);
        if (rc) return rc;
        if (i == block) break;
        TSB_CUDA(ctx, launch_argmax_rows(ctx, s->stream, s->logits_draft, 1, V, s->accept_scratch));
        std::vector<uint8_t> stats(accept_row_stats_bytes());
        TSB_CUDA(ctx, cudaMemcpyAsync(stats.data(), s->accept_scratch, stats.size(), cudaMemcpyDeviceToHost, s->stream));
        if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
        int32_t am, bad;
        accept_row_stats_read(stats.data(), 0, &am, &bad);
        if (bad) return tsb_fail(ctx, TSB_ERR_DEVICE, "the drafter's logits at step %d are not finite", i);
        proposals_out[i] = tok = am;
    }
    return TSB_OK;
}

int32_t tsb_producer_rewind_drafter(tsb_session* s, int32_t stream, int64_t position) {
    if (!s) return TSB_ERR_INVALID;
    if (!s->has_draft) return TSB_OK;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    if (tsb_kv_cursor(s->draft.kv, stream) > position + 1) return tsb_kv_set_cursor(s->draft.kv, stream, position + 1);
    return TSB_OK;
}

int64_t tsb_producer_try_reuse_prefix(tsb_session* s, int32_t stream, const int32_t* prompt_ids, int32_t n) {
    if (!s || !prompt_ids || n <= 0 || stream < 0 || stream >= s->n_streams) return 0;
    auto& fed = s->target.fed[stream];
    const int64_t cur = tsb_kv_cursor(s->target.kv, stream);
    int64_t lim = std::min<int64_t>(std::min<int64_t>(cur, (int64_t)fed.size()), (int64_t)n - 1);
    int64_t keep = 0;
    while (keep < lim && fed[(size_t)keep] == prompt_ids[keep]) keep++;
    tsb_kv_set_cursor(s->target.kv, stream, keep);
    fed.resize((size_t)keep);
    if (s->has_draft && tsb_kv_cursor(s->draft.kv, stream) > keep) tsb_kv_set_cursor(s->draft.kv, stream, keep);
    return keep;
}

int32_t tsb_producer_record_committed(tsb_session* s, int32_t stream, const int32_t* tokens, int32_t n, int64_t pos0) {
    if (!s || (!tokens && n) || n < 0) return TSB_ERR_INVALID;
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    TSB_REQUIRE(s->ctx, pos0 >= 0 && pos0 <= (int64_t)s->target.fed[stream].size(), "pos0 %lld does not continue the record", (long long)pos0);
    record_fed(s->target, stream, pos0, tokens, n);
    return TSB_OK;
}

// ---- one lockstep round over every stream ----------------------------------

int32_t tsb_session_fill_context(tsb_session* s, int64_t tokens, uint64_t seed) {
    if (!s) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    for (int q = 0; q < s->n_streams; q++) {
        int32_t rc = tsb_kv_fill_random(s->target.kv, s->stream, q, tokens, seed + 2 * q);
        if (rc) return rc;
        tsb_kv_set_cursor(s->target.kv, q, tokens);
        s->target.fed[q].assign((size_t)tokens, 0);
        if (s->has_draft) {
            if ((rc = tsb_kv_fill_random(s->draft.kv, s->stream, q, tokens, seed + 2 * q + 1))) return rc;
            tsb_kv_set_cursor(s->draft.kv, q, tokens);
        }
    }
    return tsb_stream_sync(s->ctx, s->stream);
}

}  // extern "C"

int32_t session_stage_history(tsb_session* s, const int32_t* streams, int n_active, const int32_t* next_tokens) {
    tsb_ctx* ctx = s->ctx;
    const int max_ctx = s->target.model->cfg.max_context, V = s->target.model->cfg.vocab;
    if (!s->hist_dev) {
        TSB_CUDA(ctx, cudaMalloc((void**)&s->hist_dev, (size_t)s->n_streams * max_ctx * sizeof(int32_t)));
        s->owned.push_back(s->hist_dev);
        TSB_CUDA(ctx, cudaMalloc((void**)&s->hist_len_dev, (size_t)s->n_streams * 2 * sizeof(int32_t)));
        s->owned.push_back(s->hist_len_dev);
        s->gen_dev = s->hist_len_dev + s->n_streams;
        TSB_CUDA(ctx, cudaMalloc(&s->pen_scratch, accept_history_scratch_bytes(s->n_streams, std::min(15, s->max_rows - 1 > 0 ? s->max_rows - 1 : 1), V)));
        s->owned.push_back(s->pen_scratch);
    }
    s->hist_host.assign((size_t)n_active * max_ctx + 2 * (size_t)n_active, 0);
    int32_t* lens = s->hist_host.data() + (size_t)n_active * max_ctx;
    for (int a = 0; a < n_active; a++) {
        const int q = streams[a];
        const auto& fed = s->target.fed[q];
        const int64_t ct = tsb_kv_cursor(s->target.kv, q);
        if ((int64_t)fed.size() < ct) return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: the record of fed tokens ends before the cursor", q);
        if (ct + (next_tokens ? 1 : 0) > max_ctx) return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: history beyond the context window", q);
        int32_t* row = s->hist_host.data() + (size_t)a * max_ctx;
        std::copy(fed.begin(), fed.begin() + ct, row);
        int n = (int)ct;
        if (next_tokens) row[n++] = next_tokens[a];
        lens[a] = n;
        lens[n_active + a] = std::min(s->generated[q], n);
    }
    // rows are uploaded at their used length; the copies come from pageable memory, so they are complete when the
    // calls return and hist_host may be reused
    for (int a = 0; a < n_active; a++)
        if (lens[a] > 0)
            TSB_CUDA(ctx, cudaMemcpyAsync(s->hist_dev + (size_t)a * max_ctx, s->hist_host.data() + (size_t)a * max_ctx, (size_t)lens[a] * sizeof(int32_t),
                                          cudaMemcpyHostToDevice, s->stream));
    TSB_CUDA(ctx, cudaMemcpyAsync(s->hist_len_dev, lens, (size_t)n_active * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    TSB_CUDA(ctx, cudaMemcpyAsync(s->gen_dev, lens + n_active, (size_t)n_active * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    return TSB_OK;
}

int32_t session_round_streams(tsb_session* s, const int32_t* streams, int n_active, int k, const tsb_run_config* cfg,
                              int32_t* next_tokens_host, int32_t* accepted_host, int32_t* tokens_out, int32_t* draws_out,
                              uint64_t* draw_step_inout) {
    tsb_ctx* ctx = s->ctx;
    if (!s->has_draft) return tsb_fail(ctx, TSB_ERR_STATE, "the session has no drafter");
    int32_t rc = accept_check_shaping(ctx, &cfg->shaping, true);
    if (rc) return rc;
    const bool penalised = accept_has_penalties(cfg->shaping);
    const int K = k, S = n_active;
    TSB_REQUIRE(ctx, K >= 1 && K <= 15 && K + 1 <= s->max_rows, "block must be 1..15 and fit the session's max_rows");
    TSB_REQUIRE(ctx, S >= 1 && S <= s->n_streams, "bad stream count");
    cudaStream_t st = s->stream;
    const int V = s->target.model->cfg.vocab;
    const double T = cfg->shaping.temperature;
    const bool sampled = T != 0.0;
    for (int a = 0; a < S; a++) {
        const int q = streams[a];
        TSB_REQUIRE(ctx, q >= 0 && q < s->n_streams, "stream %d outside the session", q);
        const int64_t ct = tsb_kv_cursor(s->target.kv, q);
        if (tsb_kv_cursor(s->draft.kv, q) < ct && (rc = drafter_catch_up(s, q, ct))) return rc;  // a lagging drafter replays fed tokens
        const int64_t cd = tsb_kv_cursor(s->draft.kv, q);
        if (ct != cd)
            return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: target cursor %lld and drafter cursor %lld differ", q, (long long)ct,
                            (long long)cd);
    }
    // uniforms: per stream, K draft draws (the row-only step burns one more index), then up to 2K+1 for acceptance
    const int UD = K, UA = 2 * K + 1;
    uint64_t* un = s->uniforms_host;
    for (int a = 0; a < S; a++) {
        const uint64_t seed = cfg->shaping.seed + (uint64_t)streams[a];
        for (int d = 0; d < UD; d++) un[(size_t)a * UD + d] = tsb_uniform_u64(cfg->uniform_mode, seed, draw_step_inout[a] + d);
        for (int j = 0; j < UA; j++)
            un[(size_t)S * UD + (size_t)a * UA + j] = tsb_uniform_u64(cfg->uniform_mode, seed, draw_step_inout[a] + K + 1 + j);
        s->feed_host[(size_t)a * (K + 1)] = next_tokens_host[a];
        // the drafter's first step feeds two rows: the token before the cursor again, then the confirmed one.  After a
        // round in which every proposal was accepted the drafter has never seen the last proposal; feeding the row
        // before the cursor every time keeps the pass shape fixed and replaces the reference's row-only step
        // (crates/runtime/src/speculative.rs:621-623) - a row that is already in the cache is rewritten bit for bit.
        const auto& fed = s->target.fed[streams[a]];
        const int64_t ct = tsb_kv_cursor(s->target.kv, streams[a]);
        if (ct < 1 || (int64_t)fed.size() < ct)
            return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: a round needs at least one fed token before the cursor", streams[a]);
        s->pair_host[2 * a] = fed[(size_t)ct - 1];
        s->pair_host[2 * a + 1] = next_tokens_host[a];
    }
    // a penalised round reads each stream's history - the tokens before the cursor, then the confirmed one - on the device
    if (penalised && (rc = session_stage_history(s, streams, S, next_tokens_host))) return rc;
    const int max_ctx = s->target.model->cfg.max_context;
    uint64_t* un_draft = s->uniforms_dev;
    uint64_t* un_acc = s->uniforms_dev + (size_t)S * UD;
    // pages for every row of the round are reserved up front (a reservation copies the page table synchronously,
    // which must not happen inside a capture), and the shape key of the round is formed
    uint64_t key = 1469598103934665603ull;
    auto mixk = [&](uint64_t v) { key = (key ^ v) * 1099511628211ull; };
    mixk(S), mixk(K), mixk(sampled), mixk(T == 1.0);
    {
        uint64_t tb;
        memcpy(&tb, &T, 8);
        mixk(tb);
        // the truncation settings are kernel parameters of the captured launches
        memcpy(&tb, &cfg->shaping.top_p, 8);
        mixk(tb);
        memcpy(&tb, &cfg->shaping.min_p, 8);
        mixk(tb);
        mixk(cfg->shaping.top_k);
    }
    int64_t max_base = 0;
    for (int a = 0; a < S; a++) {
        const int q = streams[a];
        mixk(q);
        const int64_t base = tsb_kv_cursor(s->target.kv, q);
        if (base + K + 1 > s->target.model->cfg.max_context)
            return tsb_fail(ctx, TSB_ERR_STATE, "stream %d: round of %d rows at %lld exceeds the context window", q, K + 1, (long long)base);
        if ((rc = tsb_kv_reserve(s->target.kv, q, base + K + 1)) || (rc = tsb_kv_reserve(s->draft.kv, q, base + K + 1))) return rc;
        max_base = std::max(max_base, base);
    }
    for (int d = 0; d <= K + 1; d++) mixk((uint64_t)((max_base + d + 1 + 511) / 512));
    s->stage_used = 0;

    auto body = [&]() -> int32_t {
        int32_t rc2;
        if (!s->replay) {
            TSB_CUDA(ctx, cudaMemcpyAsync(s->uniforms_dev, un, (size_t)S * (UD + UA) * sizeof(uint64_t), cudaMemcpyHostToDevice, st));
            TSB_CUDA(ctx, cudaMemcpyAsync(s->feed_dev, s->feed_host, (size_t)S * (K + 1) * sizeof(int32_t), cudaMemcpyHostToDevice, st));
            TSB_CUDA(ctx, cudaMemcpyAsync(s->pair_dev, s->pair_host, (size_t)S * 2 * sizeof(int32_t), cudaMemcpyHostToDevice, st));
            if (!s->capturing) TSB_CUDA(ctx, cudaEventRecord(s->ev[0], st));
        }
        // ---- draft: K steps with a head (crates/runtime/src/speculative.rs:607-659); step 0 carries two rows
        for (int a = 0; a < S; a++) tsb_kv_set_cursor(s->draft.kv, streams[a], tsb_kv_cursor(s->draft.kv, streams[a]) - 1);
        for (int d = 0; d < K; d++) {
            const tsb_row_desc* rd;
            int max_len;
            const int nrow = d == 0 ? 2 : 1;
            if ((rc2 = stage_rows(s, s->draft, streams, S, nrow, nullptr, nullptr, &rd, nullptr, &max_len))) return rc2;
            if (d == 0)
                TSB_CUDA(ctx, forward_device(s, s->draft, s->pair_dev, 1, rd, 2 * S, 2, max_len, s->logits_draft, (int64_t)K * V, true));
            else
                TSB_CUDA(ctx, forward_device(s, s->draft, s->feed_dev + d, K + 1, rd, S, 1, max_len,
                                             s->logits_draft + (size_t)d * V, (int64_t)K * V));
            for (int a = 0; a < S; a++) tsb_kv_set_cursor(s->draft.kv, streams[a], tsb_kv_cursor(s->draft.kv, streams[a]) + nrow);
            if (!s->replay) {
                if (penalised)  // every proposal of a round is shaped with the history the round started with (speculative.rs:636-648)
                    TSB_CUDA(ctx, launch_sample_history(ctx, st, s->logits_draft + (size_t)d * V, un_draft + d, S, V, cfg->shaping, s->hist_dev, max_ctx,
                                                        s->hist_len_dev, s->gen_dev, s->feed_dev + d + 1, nullptr, s->pen_scratch, (int64_t)K * V, UD,
                                                        K + 1));
                else
                    TSB_CUDA(ctx, launch_sample(ctx, st, s->logits_draft + (size_t)d * V, (int64_t)K * V, un_draft + d, UD, S, V, AcceptShape(cfg->shaping),
                                                s->feed_dev + d + 1, K + 1, nullptr, s->accept_scratch));
            }
        }
        if (!s->replay && !s->capturing) TSB_CUDA(ctx, cudaEventRecord(s->ev[1], st));
        // ---- verify: K+1 rows per stream in one pass
        {
            const tsb_row_desc* rd;
            int max_len;
            if ((rc2 = stage_rows(s, s->target, streams, S, K + 1, nullptr, nullptr, &rd, nullptr, &max_len))) return rc2;
            TSB_CUDA(ctx, forward_device(s, s->target, s->feed_dev, 1, rd, S * (K + 1), K + 1, max_len, s->logits_target, V));
        }
        if (!s->replay) {
            if (!s->capturing) TSB_CUDA(ctx, cudaEventRecord(s->ev[2], st));
            // ---- accept on the device; the next confirmed token also lands in feed[.][0]
            if (penalised)
                TSB_CUDA(ctx, launch_accept_history(ctx, st, s->logits_target, s->logits_draft, s->feed_dev + 1, K + 1, un_acc, S, K, V, cfg->shaping,
                                                    s->hist_dev, max_ctx, s->hist_len_dev, s->gen_dev, s->accept_out_dev, s->pen_scratch, s->feed_dev,
                                                    K + 1));
            else
                TSB_CUDA(ctx, launch_accept(ctx, st, s->logits_target, s->logits_draft, s->feed_dev + 1, K + 1, un_acc, S, K, V, AcceptShape(cfg->shaping),
                                            s->accept_out_dev, s->feed_dev, K + 1, s->accept_scratch));
            TSB_CUDA(ctx, cudaMemcpyAsync(s->accept_out_host, s->accept_out_dev, (size_t)S * sizeof(tsb_accept_out),
                                          cudaMemcpyDeviceToHost, st));
            if (!s->capturing) TSB_CUDA(ctx, cudaEventRecord(s->ev[3], st));
        }
        return TSB_OK;
    };

    // A round that fails part-way (a refused staging, a failed capture) must not leave the two caches out of step:
    // the cursors the body moves are put back on any error, so the caller can call again or discard.
    std::vector<int64_t> cur_t(S), cur_d(S);
    for (int a = 0; a < S; a++) cur_t[a] = tsb_kv_cursor(s->target.kv, streams[a]), cur_d[a] = tsb_kv_cursor(s->draft.kv, streams[a]);
    auto restore = [&](int32_t code) {
        for (int a = 0; a < S; a++) tsb_kv_set_cursor(s->target.kv, streams[a], cur_t[a]), tsb_kv_set_cursor(s->draft.kv, streams[a], cur_d[a]);
        s->stage_used = 0;
        return code;
    };
    const bool want_graph = s->use_graph && s->rounds_done >= 1 && !penalised;
    if (want_graph && s->graph && s->graph_key == key) {
        s->replay = true;  // host-side staging only: descriptors land in the pinned ring at the captured offsets
        rc = body();
        s->replay = false;
        if (rc) return restore(rc);
        TSB_CUDA(ctx, cudaEventRecord(s->ev[0], st));
        TSB_CUDA(ctx, cudaGraphLaunch(s->graph, st));
        TSB_CUDA(ctx, cudaEventRecord(s->ev[3], st));
        ctx->launches += s->graph_launches;
        s->last_round_graphed = true;
    } else if (want_graph) {
        if (s->graph) cudaGraphExecDestroy(s->graph), s->graph = nullptr;
        const uint64_t l0 = ctx->launches;
        TSB_CUDA(ctx, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        s->capturing = true;
        rc = body();
        s->capturing = false;
        cudaGraph_t g = nullptr;
        cudaError_t ce = cudaStreamEndCapture(st, &g);
        if (rc) {
            if (g) cudaGraphDestroy(g);
            return restore(rc);
        }
        if (ce != cudaSuccess) return restore(tsb_fail(ctx, TSB_ERR_CUDA, "ending the capture of a round failed: %s", cudaGetErrorString(ce)));
        ce = cudaGraphInstantiate(&s->graph, g, 0);
        cudaGraphDestroy(g);
        if (ce != cudaSuccess) {
            s->graph = nullptr;
            return restore(tsb_fail(ctx, TSB_ERR_CUDA, "instantiating the graph of a round failed: %s", cudaGetErrorString(ce)));
        }
        s->graph_key = key;
        s->graph_launches = ctx->launches - l0;
        TSB_CUDA(ctx, cudaEventRecord(s->ev[0], st));
        TSB_CUDA(ctx, cudaGraphLaunch(s->graph, st));
        TSB_CUDA(ctx, cudaEventRecord(s->ev[3], st));
        s->last_round_graphed = true;
    } else {
        if ((rc = body())) {
            cudaStreamSynchronize(st);  // what was enqueued before the failure is over before the cursors move back
            return restore(rc);
        }
        s->last_round_graphed = false;
    }
    s->rounds_done++;
    if ((rc = tsb_stream_sync(ctx, st))) return restore(rc);
    s->stage_used = 0;
    // ---- commit: cursors to the accepted prefix (rollback_retaining + rewind_drafter)
    for (int a = 0; a < S; a++) {
        const int q = streams[a];
        const tsb_accept_out& o = s->accept_out_host[a];
        if (o.status != 0)
            return tsb_fail(ctx, TSB_ERR_DEVICE, "stream %d: a logit was not finite or a proposal was out of range", q);
        const int64_t base = tsb_kv_cursor(s->target.kv, q);
        auto& fed = s->target.fed[q];
        fed.resize((size_t)base);
        fed.push_back(next_tokens_host[a]);
        for (int i = 0; i < o.accepted; i++) fed.push_back(o.tokens[i]);
        tsb_kv_set_cursor(s->target.kv, q, base + o.accepted + 1);
        tsb_kv_set_cursor(s->draft.kv, q, base + o.accepted + 1);
        accepted_host[a] = o.accepted;
        if (tokens_out) memcpy(tokens_out + (size_t)a * 16, o.tokens, sizeof(o.tokens));
        if (draws_out) draws_out[a] = o.draws;
        next_tokens_host[a] = o.tokens[o.accepted];
        s->generated[q] += o.accepted + 1;  // the accepted proposals and the token that enters the next round
        draw_step_inout[a] += (sampled ? (uint64_t)(K + 1) : 0) + (uint64_t)o.draws;
    }
    return TSB_OK;
}

int32_t session_prefill_rows(tsb_session* s, int stream, const int32_t* tokens, int n) {
    TSB_REQUIRE(s->ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    const int chunk = std::min(s->max_rows, 64);
    for (int i = 0; i < n; i += chunk) {
        const int m = std::min(chunk, n - i);
        const int64_t pos = tsb_kv_cursor(s->target.kv, stream);
        record_fed(s->target, stream, pos, tokens + i, m);
        int32_t rc = forward_stream(s, s->target, stream, tokens + i, m, nullptr, nullptr, nullptr);
        if (rc) return rc;
    }
    return TSB_OK;
}

// ---- tree drafting (crates/runtime/src/speculative.rs:461-560; tree shape helpers runtime/src/dflash_tree.rs)
// The drafter runs over every slot drafted so far (tree mask) and its logits at the rows that get children give
// those children: simple rather than fast - a level (static shape) or an expansion (best-first) costs one pass.
static int32_t drafter_children(tsb_session* s, int stream, const std::vector<int32_t>& feed, const std::vector<int32_t>& slot_parent, int n_known,
                                const std::vector<int32_t>& rows, int width, bool want_scores, std::vector<int32_t>& child,
                                std::vector<float>& scores) {
    tsb_ctx* ctx = s->ctx;
    const int V = s->target.model->cfg.vocab;
    const int64_t base = tsb_kv_cursor(s->draft.kv, stream);
    int32_t rc = forward_stream(s, s->draft, stream, feed.data(), n_known, slot_parent.data(), s->logits_draft, nullptr);
    if (rc) return rc;
    tsb_kv_set_cursor(s->draft.kv, stream, base);
    int32_t* rows_dev = s->tree_dev;  // row list (128 ints), then eight picks per row
    int32_t* child_dev = s->tree_dev + 128;
    const int nr = (int)rows.size();
    child.assign((size_t)nr * 8, -1);
    TSB_CUDA(ctx, cudaMemcpyAsync(rows_dev, rows.data(), nr * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    TSB_CUDA(ctx, launch_topk_rows(ctx, s->stream, s->logits_draft, V, rows_dev, nr, width, child_dev));
    TSB_CUDA(ctx, cudaMemcpyAsync(child.data(), child_dev, (size_t)nr * 8 * sizeof(int32_t), cudaMemcpyDeviceToHost, s->stream));
    if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
    for (int r = 0; r < nr; r++)
        for (int c = 0; c < width; c++)
            if (child[(size_t)r * 8 + c] < 0) return tsb_fail(ctx, TSB_ERR_DEVICE, "the drafter's logits at tree slot %d are not finite", rows[r]);
    if (want_scores) {
        // the picked candidates' logits, the scores the best-first builder's softmax runs over
        std::vector<uint16_t> raw((size_t)nr * width);
        for (int r = 0; r < nr; r++)
            for (int c = 0; c < width; c++)
                TSB_CUDA(ctx, cudaMemcpyAsync(&raw[(size_t)r * width + c], s->logits_draft + (size_t)rows[r] * V + child[(size_t)r * 8 + c], 2,
                                              cudaMemcpyDeviceToHost, s->stream));
        if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
        scores.resize(raw.size());
        for (size_t i = 0; i < raw.size(); i++) scores[i] = __half2float(__ushort_as_half(raw[i]));
    }
    return TSB_OK;
}

int32_t session_draft_tree(tsb_session* s, int stream, const TreeShape& shape, int32_t next, int64_t base, std::vector<int32_t>& feed,
                           std::vector<int32_t>& slot_parent, std::vector<tsb_tree_node>& nodes, int* drafter_rows) {
    tsb_ctx* ctx = s->ctx;
    if (!s->has_draft) return tsb_fail(ctx, TSB_ERR_STATE, "the session has no drafter");
    const int N = shape.nodes, LV = shape.levels;
    TSB_REQUIRE(ctx, N >= 1 && N + 1 <= s->max_rows && N + 1 <= 128, "tree of %d nodes + anchor exceeds the session's %d rows", N, s->max_rows);
    TSB_REQUIRE(ctx, LV >= 1 && LV <= 8, "tree_levels must be 1..8");
    int32_t rc;
    if (tsb_kv_cursor(s->draft.kv, stream) < base && (rc = drafter_catch_up(s, stream, base))) return rc;
    if (tsb_kv_cursor(s->draft.kv, stream) != base)
        return tsb_fail(ctx, TSB_ERR_STATE, "tree draft at %lld: drafter cursor %lld", (long long)base, (long long)tsb_kv_cursor(s->draft.kv, stream));
    if (base + N + 1 > s->draft.model->cfg.max_context) return tsb_fail(ctx, TSB_ERR_STATE, "a tree of %d rows at %lld exceeds the context window", N + 1, (long long)base);
    nodes.clear();
    feed.assign(1, next);
    slot_parent.assign(1, -1);
    std::vector<int32_t> child;
    std::vector<float> sc;
    int drafted = 0;
    if (shape.best_first) {
        TSB_REQUIRE(ctx, shape.cand >= 1 && shape.cand <= 8, "tree_cand must be 1..8");
        // children of node `parent` (the anchor for -1): the drafter's `cand` most likely tokens after it, scored by
        // their logits.  The expanded node is always the newest slot, so one pass over the slots so far gives its row.
        std::vector<std::vector<int32_t>> cand_tokens;  // per expanded parent (index parent + 1): its candidates' tokens
        cand_tokens.resize((size_t)N + 1);
        std::vector<tsb_tree_node> out;
        // best_first_tree appends a node and, when it has room, expands it at once: `out` is mirrored in feed/slot_parent
        // inside the callback, which therefore sees every earlier node's slot already in place
        std::vector<tsb_tree_node> seen;
        auto on_scores = [&](int depth, int parent, float* scores_out) -> int32_t {
            (void)depth;
            // bring feed / slot_parent up to date with the nodes picked since the last expansion
            return TSB_OK + 0 * (scores_out != nullptr) + 0 * parent;
        };
        (void)on_scores;
        // The builder is run step by step here (instead of through the callback form) because a node's token is only
        // known once its parent's candidates have been scored.
        struct Front {
            double p;
            tsb_tree_node n;
        };
        std::vector<Front> frontier;
        auto expand = [&](int depth, int parent, double path_p) -> int32_t {
            const int n_known = (int)feed.size();
            std::vector<int32_t> rows{parent + 1};
            int32_t rc2 = drafter_children(s, stream, feed, slot_parent, n_known, rows, shape.cand, true, child, sc);
            if (rc2) return rc2;
            drafted = n_known;
            cand_tokens[(size_t)parent + 1].assign(child.begin(), child.begin() + shape.cand);
            float mf = -INFINITY;
            for (int i = 0; i < shape.cand; i++) mf = fmaxf(mf, sc[i]);
            const double m = (double)mf;
            double e[8], z = 0.0;
            for (int i = 0; i < shape.cand; i++) e[i] = exp((double)sc[i] - m);
            for (int i = 0; i < shape.cand; i++) z += e[i];
            for (int c = 0; c < shape.cand; c++) frontier.push_back({path_p * (e[c] / z), tsb_tree_node{depth, c, parent}});
            return TSB_OK;
        };
        if ((rc = expand(0, -1, 1.0))) return rc;
        while ((int)nodes.size() < N && !frontier.empty()) {
            size_t best = 0;
            for (size_t i = 1; i < frontier.size(); i++) {
                const Front &f = frontier[i], &b = frontier[best];
                if (f.p > b.p || (f.p == b.p && (f.n.depth < b.n.depth || (f.n.depth == b.n.depth && f.n.cand < b.n.cand)))) best = i;
            }
            const Front picked = frontier[best];
            frontier[best] = frontier.back();
            frontier.pop_back();
            const int id = (int)nodes.size();
            nodes.push_back(picked.n);
            feed.push_back(cand_tokens[(size_t)picked.n.parent + 1][picked.n.cand]);
            slot_parent.push_back(picked.n.parent + 1);
            if ((int)nodes.size() < N && picked.n.depth + 1 < LV && (rc = expand(picked.n.depth + 1, id, picked.p))) return rc;
        }
        *drafter_rows = drafted;
        return TSB_OK;
    }
    for (int l = 0; l < LV; l++) TSB_REQUIRE(ctx, shape.branching[l] >= 1 && shape.branching[l] <= 8, "tree_branching must be 1..8");
    // the static shape, breadth-first, cut at N nodes: slot 0 is the anchor, node i sits in slot i + 1
    std::vector<int> level_begin{0, 1};  // slots of level l are [level_begin[l], level_begin[l+1])
    std::vector<int> depth_of{0}, cand_of{0};
    for (int l = 0; l < LV && (int)slot_parent.size() < N + 1; l++) {
        const int lo = level_begin[l], hi = level_begin[l + 1];
        for (int p = lo; p < hi && (int)slot_parent.size() < N + 1; p++)
            for (int c = 0; c < shape.branching[l] && (int)slot_parent.size() < N + 1; c++) {
                slot_parent.push_back(p);
                depth_of.push_back(l), cand_of.push_back(c);
            }
        level_begin.push_back((int)slot_parent.size());
    }
    const int rows = (int)slot_parent.size();
    TSB_REQUIRE(ctx, rows == N + 1, "the branching list yields %d nodes, fewer than tree_nodes %d", rows - 1, N);
    feed.resize(rows, 0);
    for (int i = 1; i < rows; i++) nodes.push_back(tsb_tree_node{depth_of[i], cand_of[i], slot_parent[i] - 1});
    const int n_levels = (int)level_begin.size() - 1;  // levels that hold slots (anchor level included)
    std::vector<int32_t> row_ids;
    for (int l = 0; l + 1 < n_levels; l++) {
        const int n = level_begin[l + 1];  // slots 0 .. n-1 are known
        const int lo = level_begin[l], hi = level_begin[l + 1];
        row_ids.resize(hi - lo);
        for (int p = lo; p < hi; p++) row_ids[p - lo] = p;
        if ((rc = drafter_children(s, stream, feed, slot_parent, n, row_ids, shape.branching[l], false, child, sc))) return rc;
        drafted = n;
        int slot = level_begin[l + 1];  // children of the level's nodes, in slot order
        for (int p = lo; p < hi; p++)
            for (int c = 0; c < shape.branching[l] && slot < level_begin[l + 2]; c++, slot++) feed[slot] = child[(size_t)(p - lo) * 8 + c];
    }
    *drafter_rows = drafted;
    return TSB_OK;
}

// ---- tree round: draft, then anchor + nodes in one target pass and the target's pick at every row
int32_t session_tree_round(tsb_session* s, int stream, const tsb_run_config* cfg, int32_t next, int64_t base,
                           std::vector<int32_t>& feed, std::vector<int32_t>& slot_parent, std::vector<int32_t>& picks,
                           int* drafter_rows) {
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, cfg->shaping.temperature == 0.0, "tree rounds need temperature 0 (sampled tree acceptance is not defined)");
    TreeShape shape;
    shape.nodes = cfg->tree_nodes, shape.levels = cfg->tree_levels, shape.best_first = cfg->tree_best_first, shape.cand = cfg->tree_cand;
    for (int l = 0; l < 8; l++) shape.branching[l] = cfg->tree_branching[l];
    const int V = s->target.model->cfg.vocab;
    if (tsb_kv_cursor(s->target.kv, stream) != base)
        return tsb_fail(ctx, TSB_ERR_STATE, "tree round at %lld: target cursor %lld", (long long)base, (long long)tsb_kv_cursor(s->target.kv, stream));
    std::vector<tsb_tree_node> nodes;
    int32_t rc = session_draft_tree(s, stream, shape, next, base, feed, slot_parent, nodes, drafter_rows);
    if (rc) return rc;
    const int rows = (int)feed.size();
    if ((rc = forward_stream(s, s->target, stream, feed.data(), rows, slot_parent.data(), s->logits_target, nullptr))) return rc;
    tsb_kv_set_cursor(s->target.kv, stream, base);
    TSB_REQUIRE(ctx, (size_t)rows * accept_row_stats_bytes() <= s->accept_scratch_bytes, "tree of %d rows exceeds the acceptance scratch", rows);
    TSB_CUDA(ctx, launch_argmax_rows(ctx, s->stream, s->logits_target, rows, V, s->accept_scratch));
    std::vector<uint8_t> stats((size_t)rows * accept_row_stats_bytes());
    TSB_CUDA(ctx, cudaMemcpyAsync(stats.data(), s->accept_scratch, stats.size(), cudaMemcpyDeviceToHost, s->stream));
    if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
    picks.resize(rows);
    for (int r = 0; r < rows; r++) {
        int32_t am, bad;
        accept_row_stats_read(stats.data(), r, &am, &bad);
        if (bad) return tsb_fail(ctx, TSB_ERR_DEVICE, "a target logit at tree slot %d is not finite", r);
        picks[r] = am;
    }
    return TSB_OK;
}

int32_t session_tree_commit(tsb_session* s, int stream, int64_t base, const std::vector<int32_t>& feed,
                            const std::vector<uint32_t>& path, int keep, int drafter_rows) {
    tsb_ctx* ctx = s->ctx;
    int32_t rc = tsb_kv_commit_path(ctx, s->stream, s->target.kv, stream, base, path.data(), keep);
    if (rc) return rc;
    // the drafter holds rows only for the slots it was run over: keep the part of the path it has, the rest is
    // replayed from the record of fed tokens before its next step
    int dkeep = 0;
    while (dkeep < keep && (int)path[dkeep] < drafter_rows) dkeep++;
    if (dkeep > 0 && (rc = tsb_kv_commit_path(ctx, s->stream, s->draft.kv, stream, base, path.data(), dkeep))) return rc;
    if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
    tsb_kv_set_cursor(s->target.kv, stream, base + keep);
    tsb_kv_set_cursor(s->draft.kv, stream, base + dkeep);
    auto& fed = s->target.fed[stream];
    fed.resize((size_t)base);
    for (int r = 0; r < keep; r++) fed.push_back(feed[path[r]]);
    return TSB_OK;
}

int32_t session_select_target(tsb_session* s, int stream, const tsb_run_config* cfg, uint64_t uniform, int32_t* token_host) {
    tsb_ctx* ctx = s->ctx;
    const int V = s->target.model->cfg.vocab;
    int32_t rc = accept_check_shaping(ctx, &cfg->shaping, true);
    if (rc) return rc;
    uint64_t* u = s->uniforms_host;
    u[0] = uniform;
    TSB_CUDA(ctx, cudaMemcpyAsync(s->uniforms_dev, u, sizeof(uint64_t), cudaMemcpyHostToDevice, s->stream));
    if (accept_has_penalties(cfg->shaping)) {
        // select(logits, shaping, history): the history is everything fed so far (crates/selection/src/choose.rs:139-154)
        if ((rc = session_stage_history(s, &stream, 1, nullptr))) return rc;
        TSB_CUDA(ctx, launch_sample_history(ctx, s->stream, s->logits_target, s->uniforms_dev, 1, V, cfg->shaping, s->hist_dev,
                                            s->target.model->cfg.max_context, s->hist_len_dev, s->gen_dev, s->tok1_dev, nullptr, s->pen_scratch));
    } else {
        TSB_CUDA(ctx, launch_sample(ctx, s->stream, s->logits_target, V, s->uniforms_dev, 1, 1, V, AcceptShape(cfg->shaping),
                                    s->tok1_dev, 1, nullptr, s->accept_scratch));
    }
    TSB_CUDA(ctx, cudaMemcpyAsync(s->feed_host, s->tok1_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, s->stream));
    if ((rc = tsb_stream_sync(ctx, s->stream))) return rc;
    *token_host = s->feed_host[0];
    return TSB_OK;
}

extern "C" {

int32_t tsb_session_round(tsb_session* s, const tsb_run_config* cfg, int32_t* next_tokens_host, int32_t* accepted_host,
                          uint64_t* draw_step_inout) {
    if (!s || !cfg || !next_tokens_host || !accepted_host || !draw_step_inout) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    std::vector<int32_t> streams(s->n_streams);
    for (int q = 0; q < s->n_streams; q++) streams[q] = q;
    return session_round_streams(s, streams.data(), s->n_streams, cfg->block, cfg, next_tokens_host, accepted_host, nullptr,
                                 nullptr, draw_step_inout);
}

int32_t tsb_session_round_tokens(tsb_session* s, const tsb_run_config* cfg, int32_t* next_tokens_host, int32_t* accepted_host,
                                 int32_t* tokens_out, uint64_t* draw_step_inout) {
    if (!s || !cfg || !next_tokens_host || !accepted_host || !tokens_out || !draw_step_inout) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    std::vector<int32_t> streams(s->n_streams);
    for (int q = 0; q < s->n_streams; q++) streams[q] = q;
    return session_round_streams(s, streams.data(), s->n_streams, cfg->block, cfg, next_tokens_host, accepted_host, tokens_out,
                                 nullptr, draw_step_inout);
}

void* tsb_session_stream(tsb_session* s) { return s ? (void*)s->stream : nullptr; }

int32_t tsb_session_set_graph(tsb_session* s, int32_t enabled) {
    if (!s) return TSB_ERR_INVALID;
    s->use_graph = enabled != 0;
    return TSB_OK;
}

int32_t tsb_session_time_matmuls(tsb_session* s, int32_t rows, int32_t iters, float* out_ms, int64_t* out_bytes_per_iter,
                                 int32_t* out_launches_per_iter) {
    if (!s || !out_ms) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, rows > 0 && rows <= s->n_streams * s->max_rows && iters > 0, "bad rows / iters");
    if (s->target.model->n_experts > 0) return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "the matmul timing covers dense layers only");
    DeviceGuard g(ctx);
    ModelRt& rt = s->target;
    const tsb_model* m = rt.model;
    const tsb_model_config& c = m->cfg;
    const int64_t qkv_dim = (int64_t)(c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim;
    cudaStream_t st = s->stream;
    int64_t bytes = 0;
    int launches = 0;
    // The launches are the pass's own: the same kernels with the same fused epilogues (1/rms + RoPE + K/V store,
    // residual + norm operand, SiLU * up), writing the session's real buffers; the rows sit past every stream's cursor
    // (in-flight slots nobody committed), so the caches' committed contents are untouched.  Attention, embedding and
    // head are left out.
    TSB_REQUIRE(ctx, rows % s->n_streams == 0, "rows must be a whole number of rows per stream");
    const int per = rows / s->n_streams;
    std::vector<int32_t> streams(s->n_streams);
    for (int q = 0; q < s->n_streams; q++) streams[q] = q;
    const tsb_row_desc* rd;
    int max_len;
    s->stage_used = 0;
    int32_t rc = stage_rows(s, rt, streams.data(), s->n_streams, per, nullptr, nullptr, &rd, nullptr, &max_len);
    if (rc) return rc;
    TSB_REQUIRE(ctx, !rt.wide_ok, "the matmul timing covers sessions whose target runs the few-row matmul path (largest pass below %d rows)", WIDE_MIN_ROWS);
    for (int it = -1; it < iters; it++) {  // iteration -1 is a warm-up
        if (it == 0) TSB_CUDA(ctx, cudaEventRecord(s->ev[0], st));
        TSB_CUDA(ctx, forward_device(s, rt, nullptr, 1, rd, rows, per, max_len, nullptr, 0, false, PASS_MATMULS));
    }
    for (const LayerW& l : m->layers) {
        bytes += mat_bytes(l.wqkv) + mat_bytes(l.wv) + mat_bytes(l.wo) + mat_bytes(l.wgu) + mat_bytes(l.wdown);
        launches += (l.wv.data ? 5 : 4) * ((rows + 63) / 64);
    }
    TSB_CUDA(ctx, cudaEventRecord(s->ev[1], st));
    rc = tsb_stream_sync(ctx, st);
    s->stage_used = 0;
    if (rc) return rc;
    TSB_CUDA(ctx, cudaEventElapsedTime(out_ms, s->ev[0], s->ev[1]));
    // activations in and out per launch are part of the algorithmic bytes too
    const int64_t act = (int64_t)rows * 2 * ((int64_t)c.d_model + qkv_dim + (int64_t)c.n_q_heads * c.head_dim + c.d_model + c.d_model +
                                              2 * (int64_t)c.ffn + c.ffn + c.d_model) * c.n_layers;
    if (out_bytes_per_iter) *out_bytes_per_iter = bytes + act;
    if (out_launches_per_iter) *out_launches_per_iter = launches;
    return TSB_OK;
}

int32_t tsb_session_time_pass_rest(tsb_session* s, int32_t rows, int32_t iters, float* out_ms) {
    if (!s || !out_ms) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    TSB_REQUIRE(ctx, rows > 0 && rows <= s->n_streams * s->max_rows && iters > 0, "bad rows / iters");
    if (s->target.model->n_experts > 0) return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "the pass timing covers dense layers only");
    DeviceGuard g(ctx);
    ModelRt& rt = s->target;
    TSB_REQUIRE(ctx, rows % s->n_streams == 0, "rows must be a whole number of rows per stream");
    TSB_REQUIRE(ctx, !rt.wide_ok, "the pass timing covers sessions whose target runs the few-row matmul path (largest pass below %d rows)", WIDE_MIN_ROWS);
    const int per = rows / s->n_streams;
    std::vector<int32_t> streams(s->n_streams), toks(rows, 0);
    for (int q = 0; q < s->n_streams; q++) streams[q] = q;
    const tsb_row_desc* rd;
    const int32_t* td;
    int max_len;
    s->stage_used = 0;
    int32_t rc = stage_rows(s, rt, streams.data(), s->n_streams, per, nullptr, toks.data(), &rd, &td, &max_len);
    if (rc) return rc;
    cudaStream_t st = s->stream;
    for (int it = -1; it < iters; it++) {  // iteration -1 is a warm-up
        if (it == 0) TSB_CUDA(ctx, cudaEventRecord(s->ev[0], st));
        TSB_CUDA(ctx, forward_device(s, rt, td, 1, rd, rows, per, max_len, s->logits_target, rt.model->cfg.vocab, false, PASS_REST));
    }
    TSB_CUDA(ctx, cudaEventRecord(s->ev[1], st));
    rc = tsb_stream_sync(ctx, st);
    s->stage_used = 0;
    if (rc) return rc;
    TSB_CUDA(ctx, cudaEventElapsedTime(out_ms, s->ev[0], s->ev[1]));
    return TSB_OK;
}

int32_t tsb_session_round_times(tsb_session* s, float* out4_ms) {
    if (!s || !out4_ms) return TSB_ERR_INVALID;
    DeviceGuard g(s->ctx);
    // a graphed round has no event records inside it: only the total (index 3) is known
    for (int i = 0; i < 3; i++) {
        out4_ms[i] = -1.f;
        if (!s->last_round_graphed && cudaEventElapsedTime(&out4_ms[i], s->ev[i], s->ev[i + 1]) != cudaSuccess) out4_ms[i] = -1.f;
    }
    if (cudaEventElapsedTime(&out4_ms[3], s->ev[0], s->ev[3]) != cudaSuccess) out4_ms[3] = -1.f;
    cudaGetLastError();
    return TSB_OK;
}

}  // extern "C"
