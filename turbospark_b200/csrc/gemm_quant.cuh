// Internal interface of the quantized-matmul kernels (shared with the model runner).
#pragma once
#include "common.cuh"

// The activation operand the GEMM kernels consume: for every token, the f16
// row in "pair-swizzled" order (each aligned group of four halves x0,x1,x2,x3 is
// stored x0,x2,x1,x3, which is the order the mma B fragment wants next to the
// nibble-pair dequantisation) plus, per 32-element sub-block, the f32 sum of the
// row's f16 values split into an f16 high part and an f16 remainder (the Q4_K
// min term multiplies these sums).
struct ActOperand {
    const __half* xp;     // [tokens, cols] swizzled
    const __half* xs_hi;  // [tokens, cols/32]
    const __half* xs_lo;  // [tokens, cols/32]
};

// Bytes of the two side arrays for `tokens` x `cols`.
inline size_t act_side_bytes(int64_t tokens, int64_t cols) { return (size_t)tokens * (cols / 32) * sizeof(__half); }

// x [tokens, cols] f16 natural order -> ActOperand buffers.
cudaError_t launch_act_prepare(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, int tokens, int cols,
                               __half* xp, __half* xs_hi, __half* xs_lo);

// y[t, r] = W[r,:] . x[t,:]; y f16 or f32, [tokens, rows] with row stride y_stride (elements).
cudaError_t launch_gemm_quant(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, void* y, int64_t y_stride, int tokens, bool y_f32);

#ifdef __CUDACC__
// Device helper for producers of GEMM inputs: a thread that holds eight
// consecutive f32 outputs v[0..8) of element index e0 (a multiple of 8) of
// token row t stores them, rounded to f16, in swizzled order, and the four
// threads of an aligned quad (lane & 3) that together cover one 32-element
// sub-block add up the rounded values and store the hi/lo sums.  All 32 lanes
// of the warp must call it together.
__device__ __forceinline__ void act_store8(const float (&v)[8], __half* xp_row, __half* hi_row, __half* lo_row, int e0,
                                           bool active) {
    __half h[8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        h[i] = __float2half_rn(v[i]);
        s += __half2float(h[i]);
    }
    if (!active) s = 0.f;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (active) {
        uint4 o;
        __half2 a = __halves2half2(h[0], h[2]), b = __halves2half2(h[1], h[3]);
        __half2 c = __halves2half2(h[4], h[6]), d = __halves2half2(h[5], h[7]);
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
        o.z = *reinterpret_cast<uint32_t*>(&c);
        o.w = *reinterpret_cast<uint32_t*>(&d);
        *reinterpret_cast<uint4*>(xp_row + e0) = o;
        if ((threadIdx.x & 3) == 0) {
            __half hi = __float2half_rn(s);
            hi_row[e0 >> 5] = hi;
            lo_row[e0 >> 5] = __float2half_rn(s - __half2float(hi));
        }
    }
}
#endif
