// Internal interface of the quantized-matmul kernels (shared with the model runner).
#pragma once
#include "common.cuh"

// The activation operand the GEMM kernels consume ("fragment-major" f16).
//
// Tokens are grouped in tiles of eight (an mma B operand has eight columns) and
// columns in blocks of 256.  For tile nt and block blk the data is eight chunks
// of 32 uint4: chunk c = (r*2 + jj)*2 + hi, slot = token_in_tile*4 + tig, where
// a column col (0..255) of the block maps to
//     g = col / 64, hi = (col % 64) / 32, l = col % 32,
//     r = g / 2, tig = (g % 2) * 2 + l / 16, jj = (l % 16) / 8
// and the eight columns col..col+7 (col % 8 == 0) fill one uint4 in the order
// x0,x2,x1,x3,x4,x6,x5,x7.  This is exactly the order in which one warp's lanes
// (lane = token_in_tile*4 + tig) pull mma B fragments next to the Q4_K
// nibble-pair dequantisation, so every activation load of the hot loop is one
// fully coalesced 512-byte request.  Unused token slots of the last tile must
// be readable (they are computed and never stored).
//
// xs holds, per tile, block and lane, a uint2: the f32 sum of each 32-column
// sub-block's f16 values split into an f16 high part and an f16 remainder;
// .x = hi(sub 2tig) | hi(sub 2tig+1) << 16, .y the same for the remainders
// (the Q4_K min term multiplies these sums).
struct ActOperand {
    const uint4* xp;  // [tiles][cols/256][8][32]
    const uint2* xs;  // [tiles][cols/256][32]
};

inline int act_tiles(int tokens) { return (tokens + 7) / 8; }
inline size_t act_xp_bytes(int tokens, int64_t cols) { return (size_t)act_tiles(tokens) * 8 * cols * sizeof(__half); }
inline size_t act_xs_bytes(int tokens, int64_t cols) { return (size_t)act_tiles(tokens) * (cols / 256) * 32 * sizeof(uint2); }

// x [tokens, cols] f16 natural order -> ActOperand buffers.
cudaError_t launch_act_prepare(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, int tokens, int cols,
                               uint4* xp, uint2* xs);

// y[t, r] = W[r,:] . x[t,:]; y f16 or f32, [tokens, rows] with row stride y_stride (elements).
cudaError_t launch_gemm_quant(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, void* y, int64_t y_stride, int tokens, bool y_f32);

#ifdef __CUDACC__
// uint4 index (within the operand) of the run of eight columns starting at col8 (multiple of 8) of token t.
__device__ __forceinline__ size_t act_xp_index(int t, int col8, int nblk) {
    const int blk = col8 >> 8, col = col8 & 255;
    const int g = col >> 6, hi = (col >> 5) & 1, l = col & 31;
    const int r = g >> 1, tig = ((g & 1) << 1) | (l >> 4), jj = (l >> 3) & 1;
    const int chunk = ((r * 2 + jj) << 1) | hi;
    return ((((size_t)(t >> 3) * nblk + blk) * 8 + chunk) << 5) + ((t & 7) << 2) + tig;
}
// half index of one column (for the formats that read narrower runs).
__device__ __forceinline__ size_t act_xp_half_index(int t, int col, int nblk) {
    // within a uint4 the stored order is x0,x2,x1,x3,x4,x6,x5,x7
    const int w = col & 7, q = w & 3;
    const int pos = (w & 4) | (q == 1 ? 2 : (q == 2 ? 1 : q));
    return act_xp_index(t, col & ~7, nblk) * 8 + pos;
}

// Device helper for producers of GEMM inputs: a thread that holds eight
// consecutive f32 outputs v[0..8) of column e0 (a multiple of 8) of token t
// stores them, rounded to f16, into the operand, and the four threads of an
// aligned quad (lane & 3) that together cover one 32-column sub-block add up
// the rounded values and store the hi/lo sums.  All 32 lanes of the warp must
// call it together.
__device__ __forceinline__ void act_store8(const float (&v)[8], uint4* xp, uint2* xs, int t, int e0, int nblk,
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
        xp[act_xp_index(t, e0, nblk)] = o;
        if ((threadIdx.x & 3) == 0) {
            const int blk = e0 >> 8, sb = (e0 >> 5) & 7;
            __half* q = reinterpret_cast<__half*>(xs + ((((size_t)(t >> 3) * nblk + blk) << 5) + ((t & 7) << 2) + (sb >> 1)));
            const __half hi = __float2half_rn(s);
            q[sb & 1] = hi;
            q[2 + (sb & 1)] = __float2half_rn(s - __half2float(hi));
        }
    }
}
#endif
