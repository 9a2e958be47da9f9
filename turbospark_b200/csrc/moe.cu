// Mixture-of-experts feed-forward for a handful of token rows: routing, the expert pair
// (gate/up -> activation, down) and the weighted reduction onto the residual.
//
// Semantics follow the reference's host router and its two MoE kernels:
//   routing   router_topk_gemma4 (crates/runtime/src/real_forward_dispatch.rs:1135-1158): top-k by logit,
//             ties to the lower expert index, softmax over the SELECTED logits only (f32, max = best),
//             times a per-expert scale; the weights travel as f16 (families/llama/moe.rs:118-127)
//   phase 1   acts[slot][f] = half(act(gate . x) * (up . x)), f32 dot products   (shaders/moe_gguf.metal:561-606)
//   phase 2   y[d] = half(residual[d] + sum over slots IN SLOT ORDER of float(w16[slot]) * (down[d] . acts[slot]))
//             (moe_gguf.metal:625-678; slot order is reduction order)
//
// The expert matrices are verbatim block rows (any format the matmul kernel reads; the benchmark shape uses
// MXFP4), laid out per expert as gate rows then up rows [2F, D], and down rows [D, F].  Token rows routed to the
// same expert are gathered into that expert's tiles of a padded token space (dispatch lists built on the device)
// and each phase is one grouped launch of the matmul kernel over all experts: no host round trip.
#include <algorithm>
#include <vector>

#include "gemm_quant.cuh"

constexpr int MOE_MAX_EXPERTS = 512;

namespace {

constexpr int ROUTER_MAX_EXPERTS = 512;

// One warp routes one token: k rounds of arg-max over the logits (ties to the lower index), then the softmax over
// the picks.  `row` may live in shared or global memory.
__device__ __forceinline__ void route_row(const float* row, int n_experts, int k, const float* __restrict__ scale,
                                          int32_t* __restrict__ ids, __half* __restrict__ weights, int lane, uint32_t* __restrict__ err) {
    float held[ROUTER_MAX_EXPERTS / 32];  // this lane's logits, read once
    uint32_t alive = 0;                   // bit i: expert lane + 32 i is still to be picked
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_EXPERTS / 32; i++) {
        const bool in = lane + 32 * i < n_experts;
        held[i] = in ? row[lane + 32 * i] : 0.f;
        alive |= in ? (1u << i) : 0u;
    }
    // lane r keeps pick r
    int my_pick = 0x7fffffff;
    float my_val = 0.f;
#pragma unroll
    for (int r = 0; r < 8; r++) {
        if (r < k) {
            float best = 0.f;
            int bi = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < ROUTER_MAX_EXPERTS / 32; i++) {
                const float v = held[i];
                // total order of f32::total_cmp on the values a router emits (finite): larger first, then lower index;
                // within a lane the candidates come in ascending index order, so a strict compare keeps the lower one
                if (((alive >> i) & 1u) && (bi == 0x7fffffff || v > best)) best = v, bi = lane + 32 * i;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) best = ob, bi = oi;
            }
            if (bi != 0x7fffffff && (bi & 31) == lane) alive &= ~(1u << (bi >> 5));
            if (lane == r) my_pick = bi, my_val = best;
        }
    }
    // softmax over the picks: max = the first pick, exp per lane, the sum in pick order
    const float mx = __shfl_sync(0xffffffffu, my_val, 0);
    const bool mine = lane < k;
    const float ex = mine ? (float)exp((double)(my_val - mx)) : 0.f;  // correctly rounded f32 exp
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const float er = __shfl_sync(0xffffffffu, ex, r);
        if (r < k) sum = __fadd_rn(sum, er);
    }
    const bool bad_lane = mine && (my_pick == 0x7fffffff || !isfinite(my_val));
    const bool bad = __any_sync(0xffffffffu, bad_lane);
    if (bad && lane == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_NONFINITE);
    if (mine) {
        const int e = bad ? 0 : my_pick;
        const float sc = scale ? scale[e] : 1.0f;
        ids[lane] = e;
        weights[lane] = __float2half_rn(__fmul_rn(__fdiv_rn(ex, sum), sc));
    }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int n_experts, int k, const float* __restrict__ scale,
                                 int32_t* __restrict__ ids, __half* __restrict__ weights, int tokens, uint32_t* __restrict__ err) {
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    route_row(logits + (size_t)t * n_experts, n_experts, k, scale, ids + (size_t)t * k, weights + (size_t)t * k, lane, err);
}

// One (token, expert) router logit by one warp: lane l takes columns 2l, 2l+1 of every 64-column group, as the
// reference's kernel does (shaders/moe.metal:131-144), effective scale all ones; the lanes are then added as a
// butterfly (partners 16, 8, 4, 2, 1 apart), which is also how the CPU restatement adds them.
__device__ __forceinline__ float router_logit(const uint8_t* __restrict__ qr, const uint16_t* __restrict__ sr, const uint16_t* __restrict__ br,
                                              const __half* __restrict__ xr, int groups, int lane) {
    float acc = 0.f;
    for (int g0 = 0; g0 < groups; g0 += 32) {
        // every load of the next 32 groups first (one latency), then the sums in group order
        uint32_t qq[32], ss[32], bb[32];
        __half2 xx[32];
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const int g = g0 + i;
            const bool in = g < groups;
            const int idx = (in ? g : g0) * 64 + lane * 2;
            qq[i] = *reinterpret_cast<const uint16_t*>(qr + idx);
            xx[i] = *reinterpret_cast<const __half2*>(xr + idx);
            ss[i] = sr[in ? g : g0];
            bb[i] = br[in ? g : g0];
        }
#pragma unroll
        for (int i = 0; i < 32; i++) {
            if (g0 + i < groups) {
                const float s = __uint_as_float(ss[i] << 16), b = __uint_as_float(bb[i] << 16);
                const float2 x = __half22float2(xx[i]);
                const float q0 = (float)(qq[i] & 0xFFu), q1 = (float)(qq[i] >> 8);
                acc = __fmaf_rn(s, __fadd_rn(__fmul_rn(q0, x.x), __fmul_rn(q1, x.y)), acc);
                acc = __fmaf_rn(b, __fadd_rn(x.x, x.y), acc);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    return acc;
}

__global__ void router_logits_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scale, const uint16_t* __restrict__ bias,
                                     const __half* __restrict__ x, int64_t x_stride, int tokens, int n_experts, int d,
                                     float* __restrict__ out) {
    pdl_wait();
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (int64_t)tokens * n_experts) return;
    const int t = (int)(w / n_experts), e = (int)(w % n_experts);
    const int groups = d / 64;
    const float total = router_logit(q + (size_t)e * d, scale + (size_t)e * groups, bias + (size_t)e * groups, x + (size_t)t * x_stride, groups, lane);
    if (lane == 0) out[w] = total;
}

// y[t][d] = half(float(residual[t][d]) + sum_s float(w[t][s]) * values[t*k+s][d]), slots in order.
__global__ void moe_combine_kernel(const __half* __restrict__ residual, const float* __restrict__ values,
                                   const __half* __restrict__ weights, int k, int d_model, int tokens, __half* __restrict__ y) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)tokens * d_model) return;
    const int t = (int)(idx / d_model), d = (int)(idx % d_model);
    float acc = __half2float(residual[idx]);
    for (int s = 0; s < k; s++)
        acc = __fadd_rn(acc, __fmul_rn(__half2float(weights[(size_t)t * k + s]), values[((size_t)t * k + s) * d_model + d]));
    y[idx] = __float2half_rn(acc);
}


// Dispatch lists on the device.  Every expert's rows are laid out in a padded token space: expert e owns the
// token tiles [tile_start[e], tile_start[e] + ceil(count[e] / 8)), so each expert's operand starts on a tile
// boundary.  src_pad[p] = source token of padded slot p (or -1), dst_pad[p] = its (token, slot) pair (or -1).
// One CTA; the slot order inside an expert comes from an atomic counter, which is harmless: a row's result does
// not depend on its batch mates.
__global__ void __launch_bounds__(1024)
    moe_dispatch_kernel(const int32_t* __restrict__ ids, int P, int k, int n_experts, int32_t* __restrict__ count,
                        int32_t* __restrict__ tile_start, int32_t* __restrict__ src_pad, int32_t* __restrict__ dst_pad, int pad_slots,
                        uint32_t* __restrict__ err, int n_total, int expert_lo) {
    // n_experts experts are held here: [expert_lo, expert_lo + n_experts) of the n_total the router picks from;
    // pairs routed to the others belong to another rank and are left out
    __shared__ int cnt[MOE_MAX_EXPERTS], fill[MOE_MAX_EXPERTS], tstart[MOE_MAX_EXPERTS];
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0, fill[e] = 0;
    for (int p = threadIdx.x; p < pad_slots; p += blockDim.x) src_pad[p] = -1, dst_pad[p] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        int e = ids[i];
        if (e < 0 || e >= n_total) {
            atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
            e = expert_lo;
        }
        e -= expert_lo;
        if (e < 0 || e >= n_experts) continue;
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < n_experts; e++) {
            tstart[e] = t;
            t += (cnt[e] + 7) >> 3;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        int e = ids[i];
        if (e < 0 || e >= n_total) e = expert_lo;
        e -= expert_lo;
        if (e < 0 || e >= n_experts) continue;
        const int p = tstart[e] * 8 + atomicAdd(&fill[e], 1);
        src_pad[p] = i / k, dst_pad[p] = i;
    }
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cnt[e], tile_start[e] = tstart[e];
    pdl_launch_dependents();
}

struct MoeLayout {
    int pad_tiles;  // tiles of the padded token space, with eight spare tiles the widest launch may read past the last expert
    size_t off_count, off_tstart, off_src, off_dst, off_xin_p, off_xin_s, off_act_p, off_act_s, off_values, total;
};

MoeLayout moe_layout(int tokens, int k, int n_experts, int d_model, int ffn) {
    MoeLayout L;
    const int P = tokens * k;
    L.pad_tiles = (P + 7) / 8 + std::min(P, n_experts) + 8;
    const int slots = L.pad_tiles * 8;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t o = 0;
    L.off_count = o, o += up((size_t)n_experts * 4);
    L.off_tstart = o, o += up((size_t)n_experts * 4);
    L.off_src = o, o += up((size_t)slots * 4);
    L.off_dst = o, o += up((size_t)slots * 4);
    L.off_xin_p = o, o += up(act_xp_bytes(slots, d_model));
    L.off_xin_s = o, o += up(act_xs_bytes(slots, d_model));
    L.off_act_p = o, o += up(act_xp_bytes(slots, ffn));
    L.off_act_s = o, o += up(act_xs_bytes(slots, ffn));
    L.off_values = o, o += up((size_t)P * d_model * sizeof(float));
    L.total = o;
    return L;
}

}  // namespace

cudaError_t launch_router_logits(tsb_ctx* ctx, cudaStream_t st, const uint8_t* q, const uint16_t* scale, const uint16_t* bias,
                                 const __half* x, int64_t x_stride, int tokens, int n_experts, int d, float* out) {
    const int64_t warps = (int64_t)tokens * n_experts;
    return tsb_launch(ctx, router_logits_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, st, true, q, scale, bias, x, x_stride,
                      tokens, n_experts, d, out);
}

cudaError_t launch_moe_route(tsb_ctx* ctx, cudaStream_t st, const float* logits, int tokens, int n_experts, int k, int32_t* ids,
                             __half* weights) {
    if (n_experts > ROUTER_MAX_EXPERTS) return cudaErrorInvalidValue;
    const int wpb = 4;
    return tsb_launch(ctx, moe_route_kernel, dim3((unsigned)((tokens + wpb - 1) / wpb)), dim3(wpb * 32), 0, st, true, logits, n_experts, k,
                      (const float*)nullptr, ids, weights, tokens, ctx->dev_error);
}

const float* moe_ffn_values(const void* workspace, int tokens, int k, int n_experts, int d_model, int ffn) {
    return reinterpret_cast<const float*>(static_cast<const uint8_t*>(workspace) + moe_layout(tokens, k, n_experts, d_model, ffn).off_values);
}

size_t moe_ffn_workspace_bytes(int tokens, int k, int n_experts, int d_model, int ffn) {
    return moe_layout(tokens, k, n_experts, d_model, ffn).total;
}

// The routed feed-forward without a host round trip: dispatch on the device, one gather, one grouped launch per
// phase (per 64 rows of the fullest expert's possible load), the slot-ordered combine.  Graph-capturable.
cudaError_t launch_moe_ffn(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* gate_up, const uint8_t* down, int n_experts,
                           int d_model, int ffn, const __half* x, int64_t x_stride, const __half* residual, const int32_t* ids,
                           const __half* weights, int tokens, int k, __half* y, void* workspace, int expert_lo, int n_local) {
    const MoeLayout L = moe_layout(tokens, k, n_experts, d_model, ffn);
    const int n_total = n_experts;
    if (n_local > 0) n_experts = n_local;  // the matrices hold this rank's experts only
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int32_t* count = reinterpret_cast<int32_t*>(ws + L.off_count);
    int32_t* tstart = reinterpret_cast<int32_t*>(ws + L.off_tstart);
    int32_t* src_pad = reinterpret_cast<int32_t*>(ws + L.off_src);
    int32_t* dst_pad = reinterpret_cast<int32_t*>(ws + L.off_dst);
    const ActOut xin_w{reinterpret_cast<uint4*>(ws + L.off_xin_p), reinterpret_cast<uint4*>(ws + L.off_xin_s)};
    const ActOut act_w{reinterpret_cast<uint4*>(ws + L.off_act_p), reinterpret_cast<uint4*>(ws + L.off_act_s)};
    const ActOperand xin{xin_w.xp, xin_w.xs}, act{act_w.xp, act_w.xs};
    float* values = reinterpret_cast<float*>(ws + L.off_values);
    const int P = tokens * k, slots = L.pad_tiles * 8;
    cudaError_t e = cudaSuccess;
    // a sharded call writes only its own experts' (row, slot) outputs: the others must read as zero for the exact sum
    if (n_local > 0 && (e = cudaMemsetAsync(values, 0, (size_t)P * d_model * sizeof(float), st)) != cudaSuccess) return e;
    e = tsb_launch(ctx, moe_dispatch_kernel, dim3(1), dim3(1024), 0, st, n_local == 0, ids, P, k, n_experts, count, tstart, src_pad,
                   dst_pad, slots, ctx->dev_error, n_total, n_local > 0 ? expert_lo : 0);
    if (e != cudaSuccess) return e;
    if ((e = launch_act_prepare_gather(ctx, st, x, x_stride, src_pad, slots, d_model, xin_w.xp, xin_w.xs)) != cudaSuccess) return e;
    const int64_t gu_bytes = (int64_t)2 * ffn * tsb_row_bytes(qtype, d_model), down_bytes = (int64_t)d_model * tsb_row_bytes(qtype, ffn);
    EpiArgs a1;
    a1.out = act_w;
    if ((e = launch_gemm_grouped(ctx, st, qtype, gate_up, gu_bytes, n_experts, 2 * ffn, d_model, xin, count, tstart, tokens, EPI_MOE_ACT, a1)) !=
        cudaSuccess)
        return e;
    EpiArgs a2;
    a2.y = values, a2.y_stride = d_model, a2.y_f32 = 1, a2.y_rows = dst_pad;
    if ((e = launch_gemm_grouped(ctx, st, qtype, down, down_bytes, n_experts, d_model, ffn, act, count, tstart, tokens, EPI_PLAIN, a2)) !=
        cudaSuccess)
        return e;
    if (!y) return cudaSuccess;  // the caller combines (moe_ffn_values) together with its next operator
    const int64_t total = (int64_t)tokens * d_model;
    return tsb_launch(ctx, moe_combine_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true, residual,
                      (const float*)values, weights, (int)k, (int)d_model, (int)tokens, y);
}

namespace {
__global__ void f32_to_f16_kernel(const float* __restrict__ x, __half* __restrict__ y, int64_t n) {
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}
}  // namespace

cudaError_t launch_f32_to_f16(tsb_ctx* ctx, cudaStream_t st, const float* x, __half* y, int64_t n) {
    return tsb_launch(ctx, f32_to_f16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, false, x, y, n);
}

extern "C" {

int32_t tsb_moe_route(tsb_ctx* ctx, tsb_stream s, const float* router_logits_f32, int32_t tokens, int32_t n_experts, int32_t k,
                      const float* per_expert_scale, int32_t* ids_out, void* weights_f16_out) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, router_logits_f32 && ids_out && weights_f16_out, "null buffer");
    TSB_REQUIRE(ctx, tokens > 0 && n_experts > 0 && n_experts <= ROUTER_MAX_EXPERTS && k >= 1 && k <= 8 && k <= n_experts,
                "need 1 <= k <= min(8, experts) and at most 512 experts");
    DeviceGuard g(ctx);
    const int wpb = 4;
    TSB_CUDA(ctx, tsb_launch(ctx, moe_route_kernel, dim3((unsigned)((tokens + wpb - 1) / wpb)), dim3(wpb * 32), 0, (cudaStream_t)s,
                             true, router_logits_f32, (int)n_experts, (int)k, per_expert_scale, ids_out,
                             (__half*)weights_f16_out, (int)tokens, ctx->dev_error));
    return TSB_OK;
}

int32_t tsb_router_logits(tsb_ctx* ctx, tsb_stream s, const void* q_u8, const void* scale_bf16, const void* bias_bf16,
                          const void* x_f16, int32_t tokens, int32_t n_experts, int32_t d_model, float* logits_out) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, q_u8 && scale_bf16 && bias_bf16 && x_f16 && logits_out, "null buffer");
    TSB_REQUIRE(ctx, tokens > 0 && n_experts > 0 && d_model > 0 && d_model % 64 == 0, "d_model must be a multiple of the 64-column group");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_router_logits(ctx, (cudaStream_t)s, (const uint8_t*)q_u8, (const uint16_t*)scale_bf16, (const uint16_t*)bias_bf16,
                                       (const __half*)x_f16, d_model, tokens, n_experts, d_model, logits_out));
    return TSB_OK;
}

int32_t tsb_moe_ffn(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* gate_up_region, uint64_t gate_up_off,
                    const void* down_region, uint64_t down_off, int32_t n_experts, int32_t d_model, int32_t ffn,
                    const void* x_f16, const void* residual_f16, const int32_t* ids_dev, const void* weights_f16_dev, int32_t tokens,
                    int32_t k, void* y_f16) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, gate_up_region && down_region && x_f16 && residual_f16 && ids_dev && weights_f16_dev && y_f16, "null buffer");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    TSB_REQUIRE(ctx, tokens > 0 && tokens <= 4096 && k >= 1 && k <= 8 && n_experts >= k && n_experts <= MOE_MAX_EXPERTS,
                "bad token / expert counts");
    TSB_REQUIRE(ctx, d_model > 0 && d_model % 256 == 0 && ffn > 0 && ffn % 256 == 0, "d_model and the expert width must be multiples of 256");
    TSB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(gate_up_region) + gate_up_off) & 15u) == 0 && ((reinterpret_cast<uintptr_t>(down_region) + down_off) & 15u) == 0,
                "expert matrices must start on a 16-byte boundary");
    DeviceGuard g(ctx);
    cudaStream_t st = (cudaStream_t)s;
    void* ws = nullptr;
    TSB_CUDA(ctx, cudaMallocAsync(&ws, moe_ffn_workspace_bytes(tokens, k, n_experts, d_model, ffn), st));
    cudaError_t e = launch_moe_ffn(ctx, st, qtype, static_cast<const uint8_t*>(gate_up_region) + gate_up_off,
                                   static_cast<const uint8_t*>(down_region) + down_off, n_experts, d_model, ffn, (const __half*)x_f16, d_model,
                                   (const __half*)residual_f16, ids_dev, (const __half*)weights_f16_dev, tokens, k, (__half*)y_f16, ws);
    cudaFreeAsync(ws, st);
    TSB_CUDA(ctx, e);
    return TSB_OK;
}

}  // extern "C"
