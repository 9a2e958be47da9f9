// Row operators around the matmuls: bit-exact dequantisation, embedding lookup,
// RMSNorm (optionally fused with the residual add before it), NeoX RoPE with a
// position per row, SiLU*up, residual add.  All are HBM/L2-trivial next to the
// weight streaming; what matters is that they keep the reference's rounding
// points (f16 storage between operators, fp32 arithmetic) and that the ones
// feeding a matmul emit its activation operand directly (swizzled f16 + the
// per-32 sums), so no separate preparation launch is needed.
#include "rowops.cuh"

namespace {

// ----------------------------------------------------------- exact dequantise
// crates/compute/src/quant_gguf/q4_k.rs:43-54
__device__ __forceinline__ void q4k_scale_min_dev(int j, const uint8_t* p, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = p[j] & 63u;
        m = p[j + 4] & 63u;
    } else {
        sc = (p[j + 4] & 0xFu) | ((uint32_t)(p[j - 4] >> 6) << 4);
        m = (uint32_t)(p[j + 4] >> 4) | ((uint32_t)(p[j] >> 6) << 4);
    }
}

__constant__ float kMxfp4Values[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f,
                                       0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};

// One element of a quantized row, with the reference's operation order and no
// fused multiply-add, so the value matches dequantize_* bit for bit.
template <int QT>
__device__ __forceinline__ float dequant_elem(const uint8_t* row, int e) {
    if constexpr (QT == TSB_Q4_K) {
        // q4_k.rs:67-108: d_lo = d*sc; min_lo = dmin*m; out = d_lo*q - min_lo
        const uint8_t* blk = row + (size_t)(e >> 8) * 144;
        const int ie = e & 255, g = ie >> 6, within = ie & 63, l = within & 31, hi = within >> 5;
        const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
        uint32_t sc, m;
        q4k_scale_min_dev(2 * g + hi, blk + 4, sc, m);
        const uint32_t byte = blk[16 + g * 32 + l];
        const float q = (float)(hi ? (byte >> 4) : (byte & 0xFu));
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), q), __fmul_rn(dmin, (float)m));
    } else if constexpr (QT == TSB_Q6_K) {
        // q6_k.rs:52-95: out = d * sc * q, left to right
        const uint8_t* blk = row + (size_t)(e >> 8) * 210;
        const int ie = e & 255, h = ie >> 7, within = ie & 127, k = within >> 5, l = within & 31;
        const uint8_t* ql = blk + h * 64;
        const uint32_t qh = blk[128 + h * 32 + l];
        const uint32_t lowb = ql[l + ((k & 1) ? 32 : 0)];
        const uint32_t low = (k & 2) ? (lowb >> 4) : (lowb & 0xFu);
        const int q = (int)(low | (((qh >> (2 * k)) & 3u) << 4)) - 32;
        const int sc = (int)(int8_t)blk[192 + h * 8 + (l >> 4) + 2 * k];
        const float d = __half2float(__ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8))));
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    } else if constexpr (QT == TSB_Q5_K) {
        // q5_k.rs:43-100: Q4_K's scales; fifth bit of (group g, half hi, byte l) is bit 2g+hi of qh[l]
        const uint8_t* blk = row + (size_t)(e >> 8) * 176;
        const int ie = e & 255, g = ie >> 6, within = ie & 63, l = within & 31, hi = within >> 5;
        const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
        uint32_t sc, m;
        q4k_scale_min_dev(2 * g + hi, blk + 4, sc, m);
        const uint32_t byte = blk[48 + g * 32 + l];
        const uint32_t q = (hi ? (byte >> 4) : (byte & 0xFu)) + ((((uint32_t)blk[16 + l] >> (2 * g + hi)) & 1u) << 4);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    } else if constexpr (QT == TSB_Q8_0) {
        // q8_0.rs:20-47: out = q * d, q signed
        const uint8_t* blk = row + (size_t)(e >> 5) * 34;
        const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
        return __fmul_rn((float)(int8_t)blk[2 + (e & 31)], d);
    } else {
        // quant_gguf_mxfp4.rs:114-141
        const uint8_t* blk = row + (size_t)(e >> 5) * 17;
        const int j = e & 31;
        const uint32_t ex = blk[0];
        const float d = __uint_as_float(ex < 2 ? (0x00200000u << ex) : ((ex - 1u) << 23));
        const uint32_t byte = blk[1 + (j & 15)];
        return __fmul_rn(kMxfp4Values[(j < 16) ? (byte & 0xFu) : (byte >> 4)], d);
    }
}

template <int QT, bool TO_F16>
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ w, int64_t row_bytes, int64_t table_rows, int cols,
                                    const int32_t* __restrict__ ids, int id_stride, int n, void* __restrict__ out,
                                    float out_scale, uint32_t* __restrict__ err) {
    pdl_wait();
    const int r = blockIdx.y;
    int64_t src = ids ? (int64_t)ids[(size_t)r * id_stride] : (int64_t)r;
    if (src < 0 || src >= table_rows) {
        if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
        src = 0;
    }
    const uint8_t* row = w + src * row_bytes;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < cols; e += gridDim.x * blockDim.x) {
        const float v = dequant_elem<QT>(row, e);
        if constexpr (TO_F16)
            reinterpret_cast<__half*>(out)[(size_t)r * cols + e] = __float2half_rn(__fmul_rn(v, out_scale));
        else
            reinterpret_cast<float*>(out)[(size_t)r * cols + e] = v;
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------- RMSNorm
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_ITERS = 8;  // d <= 256 * 8 * 8 = 16384

// MIX: the residual row is not read but formed here as the routed experts' weighted sum,
// half(sum over slots in slot order of float(w[r, s]) * values[r * k + s][.]) (the routed layer's combine step,
// crates/gpu/src/shaders/moe_gguf.metal:625-678 over a zero residual).
template <bool MIX>
__global__ void __launch_bounds__(NORM_THREADS)
    rmsnorm_rows_kernel(__half* __restrict__ x, const __half* __restrict__ residual, const uint16_t* __restrict__ w_bf16,
                        __half* __restrict__ out, ActOut act, int d, float eps, const float* __restrict__ mix_values,
                        const __half* __restrict__ mix_weights, int mix_k) {
    __shared__ float warp_sums[NORM_THREADS / 32];
    pdl_wait();
    const int r = blockIdx.x;
    __half* xr = x + (size_t)r * d;
    float v[NORM_MAX_ITERS][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NORM_MAX_ITERS; it++) {
        const int e0 = (it * NORM_THREADS + threadIdx.x) * 8;
        if (e0 < d) {
            uint4 raw = *reinterpret_cast<const uint4*>(xr + e0);
            const __half* hp = reinterpret_cast<const __half*>(&raw);
            if (MIX || residual) {
                uint4 rr;
                if constexpr (MIX) {
                    float a8[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) a8[i] = 0.f;
                    for (int sl = 0; sl < mix_k; sl++) {
                        const float wgt = __half2float(mix_weights[(size_t)r * mix_k + sl]);
                        const float4* vp = reinterpret_cast<const float4*>(mix_values + ((size_t)r * mix_k + sl) * d + e0);
                        const float4 v0 = vp[0], v1 = vp[1];
                        const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                        for (int i = 0; i < 8; i++) a8[i] = __fadd_rn(a8[i], __fmul_rn(wgt, vv[i]));
                    }
                    __half* rw = reinterpret_cast<__half*>(&rr);
#pragma unroll
                    for (int i = 0; i < 8; i++) rw[i] = __float2half_rn(a8[i]);
                } else {
                    rr = *reinterpret_cast<const uint4*>(residual + (size_t)r * d + e0);
                }
                const __half* rp = reinterpret_cast<const __half*>(&rr);
                uint4 upd;
                __half* up = reinterpret_cast<__half*>(&upd);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    up[i] = __float2half_rn(__half2float(hp[i]) + __half2float(rp[i]));
                    v[it][i] = __half2float(up[i]);
                }
                *reinterpret_cast<uint4*>(xr + e0) = upd;  // the residual stream keeps the f16-rounded sum
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) v[it][i] = __half2float(hp[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) ss = fmaf(v[it][i], v[it][i], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; i++) total += warp_sums[i];
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    pdl_launch_dependents();
#pragma unroll
    for (int it = 0; it < NORM_MAX_ITERS; it++) {
        const int e0 = (it * NORM_THREADS + threadIdx.x) * 8;
        const bool active = e0 < d;  // uniform per warp: d is a multiple of 256
        float o[8];
        if (active) {
            const uint4 wr = *reinterpret_cast<const uint4*>(w_bf16 + e0);
            const uint16_t* wp = reinterpret_cast<const uint16_t*>(&wr);
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = v[it][i] * bf16_bits_to_float(wp[i]) * inv;  // (x*w)*inv as rms_norm.rs:5-14
            if (out) {
                uint4 pk;
                __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
                for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(o[i]);
                *reinterpret_cast<uint4*>(out + (size_t)r * d + e0) = pk;
            }
        }
        if (act.xp && (it * NORM_THREADS * 8) < d) {
            if (!active) {
#pragma unroll
                for (int i = 0; i < 8; i++) o[i] = 0.f;
            }
            act_store8(o, act.xp, act.xs, r, active ? e0 : 0, d >> 8, active);
        }
    }
}

// ---------------------------------------------------------------------- RoPE
// crates/compute/src/rope.rs:208-255: angle = pos * exp(-(2i/head_dim) * ln theta) in f32, NeoX pairs.
// exp / sin / cos are evaluated in double and rounded once, which reproduces a
// correctly rounded f32 libm.
__global__ void rope_rows_kernel(__half* __restrict__ x, int heads, int head_dim, int rotated_pairs, int64_t row_stride,
                                 const int32_t* __restrict__ positions, float log_theta) {
    extern __shared__ float cs[];  // cos[rotated_pairs], sin[rotated_pairs]
    pdl_wait();
    const int r = blockIdx.x;
    const float pos = (float)positions[r];
    for (int i = threadIdx.x; i < rotated_pairs; i += blockDim.x) {
        const float exponent = -((float)(2 * i)) / (float)head_dim;
        const float freq = (float)exp((double)__fmul_rn(exponent, log_theta));
        const float angle = __fmul_rn(pos, freq);
        cs[i] = (float)cos((double)angle);
        cs[rotated_pairs + i] = (float)sin((double)angle);
    }
    __syncthreads();
    pdl_launch_dependents();
    const int half = head_dim / 2;
    __half* row = x + (size_t)r * row_stride;
    for (int idx = threadIdx.x; idx < heads * rotated_pairs; idx += blockDim.x) {
        const int h = idx / rotated_pairs, i = idx % rotated_pairs;
        __half* p = row + h * head_dim;
        const float x0 = __half2float(p[i]), x1 = __half2float(p[half + i]);
        const float c = cs[i], s = cs[rotated_pairs + i];
        p[i] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        p[half + i] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
    }
}

// ------------------------------------------------------------ SiLU(gate) * up
__global__ void silu_mul_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                __half* __restrict__ out, ActOut act, int rows, int n, int64_t in_stride,
                                int64_t out_stride) {
    pdl_wait();
    const int per_row = n >> 3;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = idx < (int64_t)rows * per_row;
    const int r = active ? (int)(idx / per_row) : 0;
    const int e0 = active ? (int)(idx % per_row) * 8 : 0;
    float o[8];
    if (active) {
        const uint4 g4 = *reinterpret_cast<const uint4*>(gate + (size_t)r * in_stride + e0);
        const uint4 u4 = *reinterpret_cast<const uint4*>(up + (size_t)r * in_stride + e0);
        const __half* gp = reinterpret_cast<const __half*>(&g4);
        const __half* upp = reinterpret_cast<const __half*>(&u4);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float g = __half2float(gp[i]);
            // utility.metal:41-52: (g / (1 + exp(-g))) * u, f32; exp rounded once from double
            const float e = (float)exp((double)(-g));
            o[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), __half2float(upp[i]));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = 0.f;
    }
    pdl_launch_dependents();
    if (out && active) {
        uint4 pk;
        __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(o[i]);
        *reinterpret_cast<uint4*>(out + (size_t)r * out_stride + e0) = pk;
    }
    if (act.xp) act_store8(o, act.xp, act.xs, r, e0, n >> 8, active);
}

__global__ void residual_add_kernel(__half* __restrict__ x, const __half* __restrict__ y, int64_t n) {
    pdl_wait();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i + 8 <= n) {
        uint4 a = *reinterpret_cast<const uint4*>(x + i);
        const uint4 b = *reinterpret_cast<const uint4*>(y + i);
        __half* ap = reinterpret_cast<__half*>(&a);
        const __half* bp = reinterpret_cast<const __half*>(&b);
#pragma unroll
        for (int k = 0; k < 8; k++) ap[k] = __float2half_rn(__half2float(ap[k]) + __half2float(bp[k]));
        *reinterpret_cast<uint4*>(x + i) = a;
    } else {
        for (int64_t k = i; k < n; k++) x[k] = __float2half_rn(__half2float(x[k]) + __half2float(y[k]));
    }
    pdl_launch_dependents();
}

// Embedding for the fused forward: h[r,:] = f16(dequantised row), the first layer's matmul operand f16(h * g), one
// partial sum of h^2 per row, and the row's RoPE table cos|sin (double-precision exp / sin / cos rounded once, which
// reproduces a correctly rounded f32 libm: crates/compute/src/rope.rs:208-255).  One CTA per row.
template <int QT>
__global__ void __launch_bounds__(256)
    embed_norm_kernel(const uint8_t* __restrict__ w, int64_t row_bytes, int64_t table_rows, int d,
                      const int32_t* __restrict__ ids, int id_stride, __half* __restrict__ h, const uint16_t* __restrict__ g,
                      ActOut act, float* __restrict__ ss_out, float* __restrict__ cs, const tsb_row_desc* __restrict__ rows,
                      int head_dim, float log_theta, uint32_t* __restrict__ err) {
    __shared__ float warp_sums[8];
    pdl_wait();
    const int r = blockIdx.x;
    int64_t src = (int64_t)ids[(size_t)r * id_stride];
    if (src < 0 || src >= table_rows) {
        if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
        src = 0;
    }
    const uint8_t* row = w + src * row_bytes;
    const int half = head_dim >> 1;
    const float pos = (float)rows[r].position;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float exponent = -((float)(2 * i)) / (float)head_dim;
        const float freq = (float)exp((double)__fmul_rn(exponent, log_theta));
        const float angle = __fmul_rn(pos, freq);
        cs[(size_t)r * head_dim + i] = (float)cos((double)angle);
        cs[(size_t)r * head_dim + half + i] = (float)sin((double)angle);
    }
    float ss = 0.f;
    for (int base = 0; base < d; base += 256 * 8) {
        const int e0 = base + threadIdx.x * 8;
        const bool active = e0 < d;  // d is a multiple of 256, so a warp is active or idle as a whole
        float xg[8];
#pragma unroll
        for (int i = 0; i < 8; i++) xg[i] = 0.f;
        if (active) {
            uint4 hv;
            __half* hh = reinterpret_cast<__half*>(&hv);
            const uint4 gv = *reinterpret_cast<const uint4*>(g + e0);
            const uint16_t* gg = reinterpret_cast<const uint16_t*>(&gv);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                hh[i] = __float2half_rn(dequant_elem<QT>(row, e0 + i));
                const float hn = __half2float(hh[i]);
                ss = fmaf(hn, hn, ss);
                xg[i] = hn * bf16_bits_to_float(gg[i]);
            }
            *reinterpret_cast<uint4*>(h + (size_t)r * d + e0) = hv;
        }
        act_store8(xg, act.xp, act.xs, r, active ? e0 : 0, d >> 8, active);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; i++) t += warp_sums[i];
        ss_out[r] = t;
    }
}

template <bool F16>
cudaError_t launch_dequant(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t table_rows, int cols,
                           const int32_t* ids, int id_stride, int n, void* out, float scale) {
    const int64_t rb = tsb_row_bytes(qtype, cols);
    dim3 grid((unsigned)min(8, (cols + 255) / 256), (unsigned)n);
    switch (qtype) {
        case TSB_Q4_K:
            return tsb_launch(ctx, dequant_rows_kernel<TSB_Q4_K, F16>, grid, dim3(256), 0, st, true, w, rb, table_rows,
                              cols, ids, id_stride, n, out, scale, ctx->dev_error);
        case TSB_Q6_K:
            return tsb_launch(ctx, dequant_rows_kernel<TSB_Q6_K, F16>, grid, dim3(256), 0, st, true, w, rb, table_rows,
                              cols, ids, id_stride, n, out, scale, ctx->dev_error);
        case TSB_Q5_K:
            return tsb_launch(ctx, dequant_rows_kernel<TSB_Q5_K, F16>, grid, dim3(256), 0, st, true, w, rb, table_rows,
                              cols, ids, id_stride, n, out, scale, ctx->dev_error);
        case TSB_Q8_0:
            return tsb_launch(ctx, dequant_rows_kernel<TSB_Q8_0, F16>, grid, dim3(256), 0, st, true, w, rb, table_rows,
                              cols, ids, id_stride, n, out, scale, ctx->dev_error);
        default:
            return tsb_launch(ctx, dequant_rows_kernel<TSB_MXFP4, F16>, grid, dim3(256), 0, st, true, w, rb, table_rows,
                              cols, ids, id_stride, n, out, scale, ctx->dev_error);
    }
}

}  // namespace

cudaError_t launch_embed_rows(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t vocab_rows, int cols,
                              const int32_t* ids, int id_stride, int n, __half* out, float out_scale) {
    return launch_dequant<true>(ctx, st, qtype, w, vocab_rows, cols, ids, id_stride, n, out, out_scale);
}

cudaError_t launch_embed_norm(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t vocab_rows, int d,
                              const int32_t* ids, int id_stride, int n, __half* h, const void* g_bf16, ActOut act, float* ss_out,
                              float* cs, const tsb_row_desc* rows, int head_dim, float theta) {
    const int64_t rb = tsb_row_bytes(qtype, d);
    const float lt = logf(theta);
    switch (qtype) {
        case TSB_Q4_K:
            return tsb_launch(ctx, embed_norm_kernel<TSB_Q4_K>, dim3((unsigned)n), dim3(256), 0, st, true, w, rb, vocab_rows, d, ids,
                              id_stride, h, (const uint16_t*)g_bf16, act, ss_out, cs, rows, head_dim, lt, ctx->dev_error);
        case TSB_Q6_K:
            return tsb_launch(ctx, embed_norm_kernel<TSB_Q6_K>, dim3((unsigned)n), dim3(256), 0, st, true, w, rb, vocab_rows, d, ids,
                              id_stride, h, (const uint16_t*)g_bf16, act, ss_out, cs, rows, head_dim, lt, ctx->dev_error);
        case TSB_Q5_K:
            return tsb_launch(ctx, embed_norm_kernel<TSB_Q5_K>, dim3((unsigned)n), dim3(256), 0, st, true, w, rb, vocab_rows, d, ids,
                              id_stride, h, (const uint16_t*)g_bf16, act, ss_out, cs, rows, head_dim, lt, ctx->dev_error);
        case TSB_Q8_0:
            return tsb_launch(ctx, embed_norm_kernel<TSB_Q8_0>, dim3((unsigned)n), dim3(256), 0, st, true, w, rb, vocab_rows, d, ids,
                              id_stride, h, (const uint16_t*)g_bf16, act, ss_out, cs, rows, head_dim, lt, ctx->dev_error);
        default:
            return tsb_launch(ctx, embed_norm_kernel<TSB_MXFP4>, dim3((unsigned)n), dim3(256), 0, st, true, w, rb, vocab_rows, d, ids,
                              id_stride, h, (const uint16_t*)g_bf16, act, ss_out, cs, rows, head_dim, lt, ctx->dev_error);
    }
}

cudaError_t launch_rmsnorm_rows(tsb_ctx* ctx, cudaStream_t st, __half* x, const __half* residual, const void* w_bf16,
                                __half* out, ActOut act, int rows, int d, float eps) {
    return tsb_launch(ctx, rmsnorm_rows_kernel<false>, dim3((unsigned)rows), dim3(NORM_THREADS), 0, st, true, x, residual,
                      (const uint16_t*)w_bf16, out, act, d, eps, (const float*)nullptr, (const __half*)nullptr, 0);
}

cudaError_t launch_combine_norm_rows(tsb_ctx* ctx, cudaStream_t st, __half* x, const float* values, const __half* weights, int k,
                                     const void* w_bf16, __half* out, ActOut act, int rows, int d, float eps) {
    return tsb_launch(ctx, rmsnorm_rows_kernel<true>, dim3((unsigned)rows), dim3(NORM_THREADS), 0, st, true, x, (const __half*)nullptr,
                      (const uint16_t*)w_bf16, out, act, d, eps, values, weights, k);
}

cudaError_t launch_silu_mul(tsb_ctx* ctx, cudaStream_t st, const __half* gate, const __half* up, __half* out, ActOut act,
                            int rows, int n, int64_t in_stride, int64_t out_stride) {
    const int64_t total = (int64_t)rows * (n / 8);
    return tsb_launch(ctx, silu_mul_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true, gate, up, out,
                      act, rows, n, in_stride, out_stride);
}

extern "C" {

int32_t tsb_dequant_rows(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off, int64_t cols,
                         const int32_t* row_ids, int32_t n_rows, float* out_f32) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, region && out_f32 && n_rows > 0 && cols > 0, "bad arguments");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    TSB_REQUIRE(ctx, cols % ((qtype == TSB_MXFP4 || qtype == TSB_Q8_0) ? 32 : 256) == 0, "cols is not a whole number of blocks");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_dequant<false>(ctx, (cudaStream_t)s, qtype, (const uint8_t*)region + w_off, INT64_MAX,
                                        (int)cols, row_ids, 1, n_rows, out_f32, 1.0f));
    return TSB_OK;
}

int32_t tsb_embed_rows(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off,
                       int64_t vocab_rows, int64_t cols, const int32_t* token_ids, int32_t n, void* out_f16,
                       float out_scale) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, region && out_f16 && token_ids && n > 0 && cols > 0 && vocab_rows > 0, "bad arguments");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    TSB_REQUIRE(ctx, cols % ((qtype == TSB_MXFP4 || qtype == TSB_Q8_0) ? 32 : 256) == 0, "cols is not a whole number of blocks");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_embed_rows(ctx, (cudaStream_t)s, qtype, (const uint8_t*)region + w_off, vocab_rows, (int)cols,
                                    token_ids, 1, n, (__half*)out_f16, out_scale));
    return TSB_OK;
}

int32_t tsb_rmsnorm_rows(tsb_ctx* ctx, tsb_stream s, void* x_f16, const void* residual_f16, const void* w_bf16,
                         void* out_f16, int32_t rows, int32_t d, float eps) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, x_f16 && w_bf16 && out_f16 && rows > 0, "bad arguments");
    if (d <= 0 || d % 256 != 0 || d > NORM_THREADS * 8 * NORM_MAX_ITERS)
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "d (%d) must be a multiple of 256 up to %d", d,
                        NORM_THREADS * 8 * NORM_MAX_ITERS);
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_rmsnorm_rows(ctx, (cudaStream_t)s, (__half*)x_f16, (const __half*)residual_f16, w_bf16,
                                      (__half*)out_f16, ActOut{nullptr, nullptr}, rows, d, eps));
    return TSB_OK;
}

int32_t tsb_rope_neox_rows_positions(tsb_ctx* ctx, tsb_stream s, void* x_f16, int32_t rows, int32_t heads,
                                     int32_t head_dim, int32_t rotated_pairs, int64_t row_stride,
                                     const int32_t* positions, float theta) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, x_f16 && positions && rows > 0 && heads > 0 && head_dim > 0, "bad arguments");
    TSB_REQUIRE(ctx, rotated_pairs >= 0 && rotated_pairs * 2 <= head_dim, "rotated_pairs * 2 must not exceed head_dim");
    TSB_REQUIRE(ctx, row_stride >= (int64_t)heads * head_dim, "row_stride smaller than a row");
    DeviceGuard g(ctx);
    if (rotated_pairs == 0) return TSB_OK;
    TSB_CUDA(ctx, tsb_launch(ctx, rope_rows_kernel, dim3((unsigned)rows), dim3(128), 2 * rotated_pairs * sizeof(float),
                             (cudaStream_t)s, true, (__half*)x_f16, heads, head_dim, rotated_pairs, row_stride,
                             positions, logf(theta)));
    return TSB_OK;
}

int32_t tsb_silu_mul(tsb_ctx* ctx, tsb_stream s, const void* gate_f16, const void* up_f16, void* out_f16, int32_t rows,
                     int32_t n, int64_t in_stride, int64_t out_stride) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, gate_f16 && up_f16 && out_f16 && rows > 0 && n > 0, "bad arguments");
    if (n % 32 != 0 || in_stride % 8 != 0 || out_stride % 8 != 0)
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "n must be a multiple of 32 and strides multiples of 8");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_silu_mul(ctx, (cudaStream_t)s, (const __half*)gate_f16, (const __half*)up_f16, (__half*)out_f16,
                                  ActOut{nullptr, nullptr}, rows, n, in_stride, out_stride));
    return TSB_OK;
}

int32_t tsb_residual_add(tsb_ctx* ctx, tsb_stream s, void* x_f16, const void* y_f16, int64_t n) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, x_f16 && y_f16 && n > 0, "bad arguments");
    DeviceGuard g(ctx);
    const int64_t threads = (n + 7) / 8;
    TSB_CUDA(ctx, tsb_launch(ctx, residual_add_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                             (cudaStream_t)s, true, (__half*)x_f16, (const __half*)y_f16, n));
    return TSB_OK;
}

}  // extern "C"
