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
// same expert are gathered and run through the fused matmul kernel once per expert; the dispatch lists are built
// on the host from the device's routing result (one small readback per call).
#include <algorithm>
#include <vector>

#include "gemm_quant.cuh"

namespace {

// One warp per token: k rounds of arg-max over the logits (ties to the lower index), then the softmax over the picks.
__global__ void moe_route_kernel(const float* __restrict__ logits, int n_experts, int k, const float* __restrict__ scale,
                                 int32_t* __restrict__ ids, __half* __restrict__ weights, int tokens, uint32_t* __restrict__ err) {
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const float* row = logits + (size_t)t * n_experts;
    int picked[8];
    float pv[8];
    for (int r = 0; r < k; r++) {
        float best = 0.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            bool taken = false;
            for (int c = 0; c < r; c++) taken |= picked[c] == e;
            if (taken) continue;
            const float v = row[e];
            // total order of f32::total_cmp on the values a router emits (finite): larger first, then lower index
            if (bi == 0x7fffffff || v > best || (v == best && e < bi)) best = v, bi = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) best = ob, bi = oi;
        }
        picked[r] = bi, pv[r] = best;
    }
    if (lane == 0) {
        bool bad = false;
        for (int r = 0; r < k; r++) bad |= picked[r] == 0x7fffffff || !isfinite(pv[r]);
        if (bad) atomicCAS(err, 0u, (uint32_t)TSB_DEV_NONFINITE);
        const float mx = pv[0];
        float ex[8], sum = 0.f;
        for (int r = 0; r < k; r++) {
            ex[r] = (float)exp((double)(pv[r] - mx));  // correctly rounded f32 exp
            sum += ex[r];
        }
        for (int r = 0; r < k; r++) {
            const int e = bad ? 0 : picked[r];
            const float sc = scale ? scale[e] : 1.0f;
            ids[(size_t)t * k + r] = e;
            weights[(size_t)t * k + r] = __float2half_rn(__fmul_rn(__fdiv_rn(ex[r], sum), sc));
        }
    }
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

}  // namespace

extern "C" {

int32_t tsb_moe_route(tsb_ctx* ctx, tsb_stream s, const float* router_logits_f32, int32_t tokens, int32_t n_experts, int32_t k,
                      const float* per_expert_scale, int32_t* ids_out, void* weights_f16_out) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, router_logits_f32 && ids_out && weights_f16_out, "null buffer");
    TSB_REQUIRE(ctx, tokens > 0 && n_experts > 0 && k >= 1 && k <= 8 && k <= n_experts, "need 1 <= k <= min(8, experts)");
    DeviceGuard g(ctx);
    const int wpb = 4;
    TSB_CUDA(ctx, tsb_launch(ctx, moe_route_kernel, dim3((unsigned)((tokens + wpb - 1) / wpb)), dim3(wpb * 32), 0, (cudaStream_t)s,
                             true, router_logits_f32, (int)n_experts, (int)k, per_expert_scale, ids_out,
                             (__half*)weights_f16_out, (int)tokens, ctx->dev_error));
    return TSB_OK;
}

int32_t tsb_moe_ffn(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* gate_up_region, uint64_t gate_up_off,
                    const void* down_region, uint64_t down_off, int32_t n_experts, int32_t d_model, int32_t ffn,
                    const void* x_f16, const void* residual_f16, const int32_t* ids_dev, const void* weights_f16_dev, int32_t tokens,
                    int32_t k, void* y_f16) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, gate_up_region && down_region && x_f16 && residual_f16 && ids_dev && weights_f16_dev && y_f16, "null buffer");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    TSB_REQUIRE(ctx, tokens > 0 && tokens <= 4096 && k >= 1 && k <= 8 && n_experts >= k, "bad token / expert counts");
    TSB_REQUIRE(ctx, d_model > 0 && d_model % 256 == 0 && ffn > 0 && ffn % 256 == 0, "d_model and the expert width must be multiples of 256");
    DeviceGuard g(ctx);
    cudaStream_t st = (cudaStream_t)s;
    const int P = tokens * k;
    // routing result to the host: the dispatch lists are built here
    std::vector<int32_t> ids(P);
    TSB_CUDA(ctx, cudaMemcpyAsync(ids.data(), ids_dev, (size_t)P * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    TSB_CUDA(ctx, cudaStreamSynchronize(st));
    std::vector<int> count(n_experts, 0), start(n_experts + 1, 0);
    for (int i = 0; i < P; i++) {
        if (ids[i] < 0 || ids[i] >= n_experts) return tsb_fail(ctx, TSB_ERR_INVALID, "expert id %d outside 0..%d", ids[i], n_experts);
        count[ids[i]]++;
    }
    for (int e = 0; e < n_experts; e++) start[e + 1] = start[e] + count[e];
    std::vector<int32_t> src(P), dst(P);  // per dispatch row: source token, (token, slot) row of the value matrix
    {
        std::vector<int> fill(start.begin(), start.end() - 1);
        for (int i = 0; i < P; i++) {
            const int at = fill[ids[i]]++;
            src[at] = i / k, dst[at] = i;
        }
    }
    int max_n = 1;
    for (int e = 0; e < n_experts; e++) max_n = std::max(max_n, count[e]);
    // scratch, stream-ordered: dispatch lists, the gathered operand, the activation operand, the per-slot values
    const size_t lists_b = ((size_t)2 * P * sizeof(int32_t) + 255) & ~(size_t)255;
    const size_t xin_b = ((act_xp_bytes(max_n, d_model) + 255) & ~(size_t)255) + ((act_xs_bytes(max_n, d_model) + 255) & ~(size_t)255);
    const size_t act_b = ((act_xp_bytes(max_n, ffn) + 255) & ~(size_t)255) + ((act_xs_bytes(max_n, ffn) + 255) & ~(size_t)255);
    const size_t val_b = (size_t)P * d_model * sizeof(float);
    uint8_t* scratch = nullptr;
    TSB_CUDA(ctx, cudaMallocAsync((void**)&scratch, lists_b + xin_b + act_b + val_b, st));
    int32_t* src_dev = reinterpret_cast<int32_t*>(scratch);
    int32_t* dst_dev = src_dev + P;
    uint4* xin_p = reinterpret_cast<uint4*>(scratch + lists_b);
    uint4* xin_s = reinterpret_cast<uint4*>(scratch + lists_b + ((act_xp_bytes(max_n, d_model) + 255) & ~(size_t)255));
    uint4* act_p = reinterpret_cast<uint4*>(scratch + lists_b + xin_b);
    uint4* act_s = reinterpret_cast<uint4*>(scratch + lists_b + xin_b + ((act_xp_bytes(max_n, ffn) + 255) & ~(size_t)255));
    float* values = reinterpret_cast<float*>(scratch + lists_b + xin_b + act_b);
    cudaError_t e = cudaMemcpyAsync(src_dev, src.data(), (size_t)P * sizeof(int32_t), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst_dev, dst.data(), (size_t)P * sizeof(int32_t), cudaMemcpyHostToDevice, st);
    const int64_t gu_bytes = (int64_t)2 * ffn * tsb_row_bytes(qtype, d_model), down_bytes = (int64_t)d_model * tsb_row_bytes(qtype, ffn);
    const uint8_t* gu0 = static_cast<const uint8_t*>(gate_up_region) + gate_up_off;
    const uint8_t* dn0 = static_cast<const uint8_t*>(down_region) + down_off;
    for (int ex = 0; ex < n_experts && e == cudaSuccess; ex++) {
        const int n = count[ex];
        if (!n) continue;
        e = launch_act_prepare_gather(ctx, st, (const __half*)x_f16, d_model, src_dev + start[ex], n, d_model, xin_p, xin_s);
        if (e != cudaSuccess) break;
        EpiArgs a1;
        a1.out = ActOut{act_p, act_s};
        e = launch_gemm_fused(ctx, st, qtype, gu0 + (int64_t)ex * gu_bytes, 2 * ffn, d_model, ActOperand{xin_p, xin_s}, n, EPI_MOE_ACT, a1);
        if (e != cudaSuccess) break;
        EpiArgs a2;
        a2.y = values, a2.y_stride = d_model, a2.y_f32 = 1, a2.y_rows = dst_dev + start[ex];
        e = launch_gemm_fused(ctx, st, qtype, dn0 + (int64_t)ex * down_bytes, d_model, ffn, ActOperand{act_p, act_s}, n, EPI_PLAIN, a2);
    }
    if (e == cudaSuccess) {
        const int64_t total = (int64_t)tokens * d_model;
        e = tsb_launch(ctx, moe_combine_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true,
                       (const __half*)residual_f16, (const float*)values, (const __half*)weights_f16_dev, (int)k, (int)d_model,
                       (int)tokens, (__half*)y_f16);
    }
    cudaFreeAsync(scratch, st);
    TSB_CUDA(ctx, e);
    return TSB_OK;
}

}  // extern "C"
