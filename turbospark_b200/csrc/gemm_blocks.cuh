// Device code shared by the quantized-matmul kernels: the per-format block routines (weights of one 256-column
// unit of two rows against the fragment-major activation operand), the work decomposition into groups of row
// tiles, and the epilogues.  Included by the matmul kernel's translation unit.
#pragma once
#include "gemm_quant.cuh"

namespace {

constexpr int TILE_ROWS = 16;
constexpr int STAGE_UNITS = 8;  // 256-column units per row per stage (one per consumer warp)
constexpr int CONSUMER_WARPS = 8;
constexpr int GEMM_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int NUM_STAGES = 3;
// Row stride inside a stage: the payload (<= 8*210 + 30 slack) rounded so that
// stride = 64 (mod 128) bytes, which makes the 16-byte fragment loads of the
// eight row groups hit distinct banks (Q4_K).  The other formats' routines read
// 4-byte words, the four lanes of a row group side by side: there stride = 16
// (mod 128) puts the eight row groups of a warp on eight different 16-byte bank
// groups (with stride = 64 every second row group met the same banks: a
// four-way conflict on every load).
__host__ __device__ constexpr int row_stride_for(int unit_bytes) {
    int span = STAGE_UNITS * unit_bytes + 32;
    int s = (span + 127) / 128 * 128 + (unit_bytes == 144 ? 64 : 16);
    return s;
}

template <int QT>
struct Fmt;
template <>
struct Fmt<TSB_Q4_K> {
    static constexpr int UNIT_BYTES = 144;
};
template <>
struct Fmt<TSB_Q6_K> {
    static constexpr int UNIT_BYTES = 210;
};
template <>
struct Fmt<TSB_MXFP4> {
    static constexpr int UNIT_BYTES = 136;  // eight 17-byte blocks
};
template <>
struct Fmt<TSB_Q5_K> {
    static constexpr int UNIT_BYTES = 176;
};
template <>
struct Fmt<TSB_Q8_0> {
    static constexpr int UNIT_BYTES = 272;  // eight 34-byte blocks
};

__device__ __forceinline__ uint32_t lds_u32_unaligned(const uint8_t* p) {
    uint32_t a = smem_u32(p);
    uint32_t base = a & ~3u;
    uint32_t lo, hi;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lo) : "r"(base));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(hi) : "r"(base + 4));
    return __funnelshift_r(lo, hi, (a & 3u) * 8u);
}

// ---- Q4_K: one 144-byte superblock for rows (gid, gid+8) -------------------
// Layout (crates/compute/src/quant_gguf/q4_k.rs:17-41): f16 d, f16 dmin, 12
// packed bytes of 6-bit scales/mins, 128 nibble bytes; in group g (64 elements)
// byte l holds element 64g+l (low nibble, sub-block 2g) and 64g+32+l (high
// nibble, sub-block 2g+1); w = d*sc*q - dmin*m.
//
// q*sc <= 15*63 is exact in f16, so the A operand is q*sc, built as
// fma(1024+q, sc, -1024*sc) from the (nibble | 0x6400) bit pattern, and the
// block's sum needs one multiply by d afterwards.  The min term is a second,
// tiny contraction over the eight sub-blocks: sum_sub m[sub] * xsum[sub].
// Per-lane activation pointers, fixed for the whole kernel: token index is
// clamped (columns past `tokens` compute a duplicate that is never stored), so
// the hot loop carries no predicates.
template <int NT>
struct LaneAct {
    const uint4* xp[NT];  // token tile nt of the fragment-major operand, advanced by the lane index
    const uint4* xs[NT];  // 16-column sums of tile nt, advanced by the lane index
    int nblk;
};

__device__ __forceinline__ void mma_16816_first(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(0.f));
}
__device__ __forceinline__ void mma_1688_first(float (&d)[4], const uint32_t (&a)[2], uint32_t b) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(b), "f"(0.f));
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// rowA/rowB: the 144-byte superblock of rows gid and gid+8 in shared memory.
// blk: index of the 256-column block (for the activation offsets).
template <int NT>
__device__ __forceinline__ void q4k_block(const uint4* __restrict__ rowA, const uint4* __restrict__ rowB,
                                          const LaneAct<NT>& la, int blk, int tig, float (&acc)[NT][4]) {
    // all activation loads of the block first: one scoreboard wait, hidden behind the scale decode
    uint4 xl[2][2][NT], xh[2][2][NT];
    uint4 xsum[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const uint4* p = la.xp[nt] + blk * 256;  // eight 32-lane chunks per block
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int jj = 0; jj < 2; jj++) {
                xl[r][jj][nt] = __ldg(p + ((r * 2 + jj) * 2) * 32);
                xh[r][jj][nt] = __ldg(p + ((r * 2 + jj) * 2 + 1) * 32);  // sub-block 2g+1
            }
        xsum[nt] = __ldg(la.xs[nt] + blk * 32);
    }
    const uint4 hA = rowA[0];
    const uint4 hB = rowB[0];
    const int h = tig >> 1;
    // this lane's nibble bytes: group g = 2r + h, bytes (tig&1)*16 .. +15  -> uint4 index 1 + 2g + (tig&1)
    const int qoff = 1 + 2 * h + (tig & 1);
    const uint4 qA0 = rowA[qoff], qB0 = rowB[qoff];
    const uint4 qA1 = rowA[qoff + 4], qB1 = rowB[qoff + 4];

    const __half2 ddA = *reinterpret_cast<const __half2*>(&hA.x);
    const __half2 ddB = *reinterpret_cast<const __half2*>(&hB.x);
    const float dA = __low2float(ddA), dminA = __high2float(ddA);
    const float dB = __low2float(ddB), dminB = __high2float(ddB);

    // 6-bit fields as bytes: sc0..3 | sc4..7 | m0..3 | m4..7
    const uint32_t scA_lo = hA.y & 0x3F3F3F3Fu, scA_hi = (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u);
    const uint32_t scB_lo = hB.y & 0x3F3F3F3Fu, scB_hi = (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u);
    const uint32_t mA_lo = hA.z & 0x3F3F3F3Fu, mA_hi = ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u);
    const uint32_t mB_lo = hB.z & 0x3F3F3F3Fu, mB_hi = ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u);

    const uint32_t k1024 = 0x64006400u;
    // --- min term: one m16n8k16 over the block's sixteen 16-column sums; k slots (2tig, 2tig+1) belong to
    // sub-block tig, slots (2tig+8, 2tig+9) to sub-block tig+4, so A repeats each min twice
    {
        const uint32_t sel = (uint32_t)tig * 0x0101u | 0x4040u;
        uint32_t amin[4];
        amin[0] = hsub2_u32(__byte_perm(mA_lo, 0x64646464u, sel), k1024);
        amin[1] = hsub2_u32(__byte_perm(mB_lo, 0x64646464u, sel), k1024);
        amin[2] = hsub2_u32(__byte_perm(mA_hi, 0x64646464u, sel), k1024);
        amin[3] = hsub2_u32(__byte_perm(mB_hi, 0x64646464u, sel), k1024);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint32_t bhi[2] = {xsum[nt].x, xsum[nt].y}, blo[2] = {xsum[nt].z, xsum[nt].w};
            float c[4];
            mma_16816_first(c, amin, bhi);
            mma_16816(c, amin, blo);
            acc[nt][0] -= dminA * c[0];
            acc[nt][1] -= dminA * c[1];
            acc[nt][2] -= dminB * c[2];
            acc[nt][3] -= dminB * c[3];
        }
    }

    const uint32_t selE = 0x4040u | ((2u * h) * 0x0101u);
    const uint32_t selO = selE + 0x0101u;
    const uint32_t kNeg1024 = 0xE400E400u;  // half2(-1024)
    const uint32_t kNeg64 = 0xD400D400u;    // half2(-64)

    float cL[NT][4], cH[NT][4];  // two independent mma chains (low / high nibbles)
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 qA = r ? qA1 : qA0, qB = r ? qB1 : qB0;
        // scales of sub-blocks 2g (low nibbles) and 2g+1 (high nibbles) as half2(sc, sc)
        const uint32_t scLA = hsub2_u32(__byte_perm(r ? scA_hi : scA_lo, 0x64646464u, selE), k1024);
        const uint32_t scHA = hsub2_u32(__byte_perm(r ? scA_hi : scA_lo, 0x64646464u, selO), k1024);
        const uint32_t scLB = hsub2_u32(__byte_perm(r ? scB_hi : scB_lo, 0x64646464u, selE), k1024);
        const uint32_t scHB = hsub2_u32(__byte_perm(r ? scB_hi : scB_lo, 0x64646464u, selO), k1024);
        const uint32_t offLA = hmul2_u32(scLA, kNeg1024), offHA = hmul2_u32(scHA, kNeg64);
        const uint32_t offLB = hmul2_u32(scLB, kNeg1024), offHB = hmul2_u32(scHB, kNeg64);

        const uint32_t wA[4] = {qA.x, qA.y, qA.z, qA.w};
        const uint32_t wB[4] = {qB.x, qB.y, qB.z, qB.w};
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
#pragma unroll
            for (int j2 = 0; j2 < 2; j2++) {
                const int j = jj * 2 + j2;
                uint32_t alo[4], ahi[4];
                const uint32_t a = wA[j], b = wB[j];
                const uint32_t a8 = a >> 8, b8 = b >> 8;
                alo[0] = hfma2_u32(lop3_and_or(a, 0x000F000Fu, 0x64006400u), scLA, offLA);
                alo[1] = hfma2_u32(lop3_and_or(b, 0x000F000Fu, 0x64006400u), scLB, offLB);
                alo[2] = hfma2_u32(lop3_and_or(a8, 0x000F000Fu, 0x64006400u), scLA, offLA);
                alo[3] = hfma2_u32(lop3_and_or(b8, 0x000F000Fu, 0x64006400u), scLB, offLB);
                ahi[0] = hfma2_u32(lop3_and_or(a, 0x00F000F0u, 0x54005400u), scHA, offHA);
                ahi[1] = hfma2_u32(lop3_and_or(b, 0x00F000F0u, 0x54005400u), scHB, offHB);
                ahi[2] = hfma2_u32(lop3_and_or(a8, 0x00F000F0u, 0x54005400u), scHA, offHA);
                ahi[3] = hfma2_u32(lop3_and_or(b8, 0x00F000F0u, 0x54005400u), scHB, offHB);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    uint32_t bl[2], bh[2];
                    bl[0] = j2 ? xl[r][jj][nt].z : xl[r][jj][nt].x;
                    bl[1] = j2 ? xl[r][jj][nt].w : xl[r][jj][nt].y;
                    bh[0] = j2 ? xh[r][jj][nt].z : xh[r][jj][nt].x;
                    bh[1] = j2 ? xh[r][jj][nt].w : xh[r][jj][nt].y;
                    if (r == 0 && j == 0) {
                        mma_16816_first(cL[nt], alo, bl);
                        mma_16816_first(cH[nt], ahi, bh);
                    } else {
                        mma_16816(cL[nt], alo, bl);
                        mma_16816(cH[nt], ahi, bh);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        acc[nt][0] += dA * (cL[nt][0] + cH[nt][0]);
        acc[nt][1] += dA * (cL[nt][1] + cH[nt][1]);
        acc[nt][2] += dB * (cL[nt][2] + cH[nt][2]);
        acc[nt][3] += dB * (cL[nt][3] + cH[nt][3]);
    }
}

// ---- MXFP4: eight 17-byte blocks (256 columns) for rows (gid, gid+8) -------
// Block (crates/compute/src/quant_gguf_mxfp4.rs:60-78): e8m0 byte, 16 nibble
// bytes; byte j = element j (low) and j+16 (high); w = LUT[code] * 2^(e-128)
// with LUT = 2 * e2m1.
__device__ __forceinline__ float mxfp4_scale_dev(uint32_t e) {
    // crates/compute/src/quant_gguf_mxfp4.rs:95-102: 2^(e-128), subnormal for e < 2.
    return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1u) << 23));
}

// Four code bytes -> four f16 pairs with the hardware conversion (cvt.rn.f16x2.e2m1x2: the byte's low nibble becomes the
// low half, its high nibble the high half; the eight magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 are exact in f16).  Byte i
// of a block holds elements i (low) and i + 16 (high), so pair i is (element i, element i + 16).
__device__ __forceinline__ void e2m1_bytes_to_f16x2(uint32_t v, uint32_t& p0, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}"
        : "=r"(p0), "=r"(p1), "=r"(p2), "=r"(p3)
        : "r"(v));
}

// One 256-column unit = eight 17-byte blocks.  One mma must stay inside one block, because the block scale
// multiplies its fp32 sum.  Lane tig takes code bytes 4tig..4tig+3 of every block: byte 4tig+i converts to the pair
// (element 4tig+i, element 16+4tig+i), which is one A register, so the contraction slots of an mma are numbered
// (2tig, 2tig+1) = the two elements of byte 4tig+2m and (2tig+8, 2tig+9) = those of byte 4tig+2m+1 for mma m = 0, 1
// of the block.  The B registers follow the same numbering: the operand keeps a token's columns as (x0,x2),(x1,x3)
// words, elements 4tig.. in one 8-byte slot and 16+4tig.. in the next 16-byte slot, so a byte permute of the two
// words (low halves for mma 0, high halves for mma 1) pairs column e with column e + 16.  With b unrolled every
// offset is an immediate: uint4 index ((b/4)*4 + (b&1))*32 + ((b/2)&1)*2 past the lane's base.  Rows start on a
// 4-byte boundary (checked where the weights come in) and a unit is 136 bytes, so the lane's code word of block b,
// bytes 17b + 1 + 4tig .. +3, is a funnel shift by an immediate over two aligned words.  The reference's table holds
// 2 * e2m1 (crates/compute/src/quant_gguf_mxfp4.rs:76-78): the factor 2 goes into the block scale.
template <int NT>
__device__ __forceinline__ void mxfp4_unit(const uint8_t* rA, const uint8_t* rB, const ActOperand& act, int nblk,
                                           int unit, int gid, int tig, float (&acc)[NT][4]) {
    const uint2* xb[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
        xb[nt] = reinterpret_cast<const uint2*>(act.xp + ((size_t)nt * nblk + unit) * 256 + (tig >> 1) * 64 + gid * 4) + (tig & 1);
    const uint32_t* wA = reinterpret_cast<const uint32_t*>(rA) + tig;
    const uint32_t* wB = reinterpret_cast<const uint32_t*>(rB) + tig;
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const int o = 17 * b + 1;  // byte offset of the block's code bytes in the row
        const float scA = mxfp4_scale_dev(rA[o - 1]), scB = mxfp4_scale_dev(rB[o - 1]);
        uint32_t cwA = wA[o >> 2], cwB = wB[o >> 2];
        if ((o & 3) != 0) {
            cwA = __funnelshift_r(cwA, wA[(o >> 2) + 1], (o & 3) * 8);
            cwB = __funnelshift_r(cwB, wB[(o >> 2) + 1], (o & 3) * 8);
        }
        uint32_t pa[4], pb[4];
        e2m1_bytes_to_f16x2(cwA, pa[0], pa[1], pa[2], pa[3]);
        e2m1_bytes_to_f16x2(cwB, pb[0], pb[1], pb[2], pb[3]);
        const uint32_t a0[4] = {pa[0], pb[0], pa[1], pb[1]}, a1[4] = {pa[2], pb[2], pa[3], pb[3]};
        const float sA2 = scA + scA, sB2 = scB + scB;
        const int u4 = (((b >> 2) * 4 + (b & 1)) * 32 + ((b >> 1) & 1) * 2) * 2;  // in uint2 units
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint2 l = __ldg(xb[nt] + u4), hh = __ldg(xb[nt] + u4 + 2);
            const uint32_t b0[2] = {__byte_perm(l.x, hh.x, 0x5410), __byte_perm(l.y, hh.y, 0x5410)};
            const uint32_t b1[2] = {__byte_perm(l.x, hh.x, 0x7632), __byte_perm(l.y, hh.y, 0x7632)};
            float c[4];
            mma_16816_first(c, a0, b0);
            mma_16816(c, a1, b1);
            acc[nt][0] += sA2 * c[0];
            acc[nt][1] += sA2 * c[1];
            acc[nt][2] += sB2 * c[2];
            acc[nt][3] += sB2 * c[3];
        }
    }
}

// ---- Q6_K: one 210-byte superblock for rows (gid, gid+8) -------------------
// Layout (crates/compute/src/quant_gguf/q6_k.rs:17-50): ql[128], qh[64],
// int8 sc[16], f16 d; per half h and l < 32 the four 6-bit values of elements
// 128h + l + 32k (k = 0..3) take their low nibble from ql[64h + l + 32(k&1)]
// (low nibble for k < 2, high for k >= 2) and bits 2k..2k+1 of qh[32h + l];
// w = d * sc[8h + l/16 + 2k] * (q - 32).  One mma covers exactly one 16-element
// scale group, so the int8 scale multiplies the fp32 partial sum.
__device__ __forceinline__ float s8_to_float(uint32_t byte) {
    // exact: (0x4B000000 | (b ^ 0x80)) is 8388608 + (b ^ 0x80)
    return __uint_as_float(0x4B000000u | ((byte ^ 0x80u) & 0xFFu)) - 8388736.0f;
}

template <int NT>
__device__ __forceinline__ void q6k_block(const uint8_t* rA, const uint8_t* rB, const ActOperand& act, int nblk,
                                          int blk, int gid, int tig, float (&acc)[NT][4]) {
    float blkacc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) blkacc[nt][i] = 0.f;
    const uint32_t k1056 = 0x64206420u;  // half2(1056) = 1024 + 32
#pragma unroll 1
    for (int hh = 0; hh < 2; hh++) {
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const int l = 16 * m + 4 * tig;
            const uint32_t qhA = lds_u32_unaligned(rA + 128 + 32 * hh + l);
            const uint32_t qhB = lds_u32_unaligned(rB + 128 + 32 * hh + l);
            const uint32_t qlA0 = lds_u32_unaligned(rA + 64 * hh + l), qlA1 = lds_u32_unaligned(rA + 64 * hh + 32 + l);
            const uint32_t qlB0 = lds_u32_unaligned(rB + 64 * hh + l), qlB1 = lds_u32_unaligned(rB + 64 * hh + 32 + l);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t la = (k & 1) ? qlA1 : qlA0, lb = (k & 1) ? qlB1 : qlB0;
                const uint32_t va = (((k & 2) ? (la >> 4) : la) & 0x0F0F0F0Fu) | (((qhA >> (2 * k)) & 0x03030303u) << 4);
                const uint32_t vb = (((k & 2) ? (lb >> 4) : lb) & 0x0F0F0F0Fu) | (((qhB >> (2 * k)) & 0x03030303u) << 4);
                uint32_t a[4];
                a[0] = lop3_and_or(va, 0x00FF00FFu, 0x64006400u);
                a[1] = lop3_and_or(vb, 0x00FF00FFu, 0x64006400u);
                a[2] = lop3_and_or(va >> 8, 0x00FF00FFu, 0x64006400u);
                a[3] = lop3_and_or(vb >> 8, 0x00FF00FFu, 0x64006400u);
#pragma unroll
                for (int i = 0; i < 4; i++) asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(a[i]) : "r"(a[i]), "r"(k1056));
                const int si = 8 * hh + m + 2 * k;
                const float sA = s8_to_float(rA[192 + si]);
                const float sB = s8_to_float(rB[192 + si]);
                const int k0 = blk * 256 + 128 * hh + 32 * k + l;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int token = nt * 8 + gid;
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    uint32_t bb[2];
                    {
                        const __half* xh16 = reinterpret_cast<const __half*>(act.xp);
                        const uint2 x = __ldg(reinterpret_cast<const uint2*>(xh16 + act_xp_half_index(token, k0, nblk)));
                        bb[0] = x.x, bb[1] = x.y;
                    }
                    mma_16816(c, a, bb);
                    blkacc[nt][0] += sA * c[0];
                    blkacc[nt][1] += sA * c[1];
                    blkacc[nt][2] += sB * c[2];
                    blkacc[nt][3] += sB * c[3];
                }
            }
        }
    }
    const float dA = __half2float(__ushort_as_half((unsigned short)(rA[208] | (rA[209] << 8))));
    const float dB = __half2float(__ushort_as_half((unsigned short)(rB[208] | (rB[209] << 8))));
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        acc[nt][0] += dA * blkacc[nt][0];
        acc[nt][1] += dA * blkacc[nt][1];
        acc[nt][2] += dB * blkacc[nt][2];
        acc[nt][3] += dB * blkacc[nt][3];
    }
}

// ---- Q5_K: one 176-byte superblock for rows (gid, gid+8) -------------------
// Layout (crates/compute/src/quant_gguf/q5_k.rs:12-24,43-100): f16 d, f16 dmin, Q4_K's 12 packed scale/min
// bytes, qh[32], ql[128]; element (group g, half hi, byte l) = 64g + 32hi + l takes its low four bits from
// nibble hi of ql[32g + l] and its fifth from bit 2g+hi of qh[l]; w = d*sc*q - dmin*m with q in 0..31.
// One mma covers 16 elements of one sub-block with the exact integers q as the A operand; a second mma with
// an all-ones A operand yields the activation sum the sub-block's min multiplies.
__device__ __forceinline__ void q4k_scale_min_smem(int j, const uint8_t* p, float& sc, float& m) {
    // crates/compute/src/quant_gguf/q4_k.rs:43-54
    uint32_t s, mm;
    if (j < 4) {
        s = p[j] & 63u, mm = p[j + 4] & 63u;
    } else {
        s = (p[j + 4] & 0xFu) | ((uint32_t)(p[j - 4] >> 6) << 4);
        mm = (uint32_t)(p[j + 4] >> 4) | ((uint32_t)(p[j] >> 6) << 4);
    }
    sc = (float)s, m = (float)mm;
}

template <int NT>
__device__ __forceinline__ void q5k_block(const uint8_t* rA, const uint8_t* rB, const ActOperand& act, int nblk,
                                          int blk, int gid, int tig, float (&acc)[NT][4]) {
    float bq[NT][4], bm[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) bq[nt][i] = 0.f, bm[nt][i] = 0.f;
    const uint32_t k1024 = 0x64006400u, kOne = 0x3C003C00u;
    const uint32_t ones[4] = {kOne, kOne, kOne, kOne};
#pragma unroll 1
    for (int j = 0; j < 8; j++) {  // sub-block j = 2g + hi
        const int g = j >> 1, hi = j & 1;
        float scA, mA, scB, mB;
        q4k_scale_min_smem(j, rA + 4, scA, mA);
        q4k_scale_min_smem(j, rB + 4, scB, mB);
        float cq[NT][4], cs[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) cq[nt][i] = 0.f, cs[nt][i] = 0.f;
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const int l = 16 * m + 4 * tig;
            const uint32_t qlA = *reinterpret_cast<const uint32_t*>(rA + 48 + 32 * g + l);
            const uint32_t qlB = *reinterpret_cast<const uint32_t*>(rB + 48 + 32 * g + l);
            const uint32_t qhA = *reinterpret_cast<const uint32_t*>(rA + 16 + l);
            const uint32_t qhB = *reinterpret_cast<const uint32_t*>(rB + 16 + l);
            const uint32_t vA = ((qlA >> (4 * hi)) & 0x0F0F0F0Fu) | (((qhA >> j) & 0x01010101u) << 4);
            const uint32_t vB = ((qlB >> (4 * hi)) & 0x0F0F0F0Fu) | (((qhB >> j) & 0x01010101u) << 4);
            uint32_t a[4];
            a[0] = hsub2_u32(lop3_and_or(vA, 0x00FF00FFu, k1024), k1024);
            a[1] = hsub2_u32(lop3_and_or(vB, 0x00FF00FFu, k1024), k1024);
            a[2] = hsub2_u32(lop3_and_or(vA >> 8, 0x00FF00FFu, k1024), k1024);
            a[3] = hsub2_u32(lop3_and_or(vB >> 8, 0x00FF00FFu, k1024), k1024);
            const int k0 = blk * 256 + 32 * j + l;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const __half* xh16 = reinterpret_cast<const __half*>(act.xp);
                const uint2 x = __ldg(reinterpret_cast<const uint2*>(xh16 + act_xp_half_index(nt * 8 + gid, k0, nblk)));
                const uint32_t bb[2] = {x.x, x.y};
                mma_16816(cq[nt], a, bb);
                mma_16816(cs[nt], ones, bb);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            bq[nt][0] += scA * cq[nt][0], bq[nt][1] += scA * cq[nt][1];
            bq[nt][2] += scB * cq[nt][2], bq[nt][3] += scB * cq[nt][3];
            bm[nt][0] += mA * cs[nt][0], bm[nt][1] += mA * cs[nt][1];
            bm[nt][2] += mB * cs[nt][2], bm[nt][3] += mB * cs[nt][3];
        }
    }
    const __half2 ddA = *reinterpret_cast<const __half2*>(rA), ddB = *reinterpret_cast<const __half2*>(rB);
    const float dA = __low2float(ddA), dminA = __high2float(ddA), dB = __low2float(ddB), dminB = __high2float(ddB);
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        acc[nt][0] += dA * bq[nt][0] - dminA * bm[nt][0];
        acc[nt][1] += dA * bq[nt][1] - dminA * bm[nt][1];
        acc[nt][2] += dB * bq[nt][2] - dminB * bm[nt][2];
        acc[nt][3] += dB * bq[nt][3] - dminB * bm[nt][3];
    }
}

// ---- Q8_0: eight 34-byte blocks (256 columns) for rows (gid, gid+8) --------
// Block (crates/compute/src/quant_gguf/q8_0.rs:5-47): f16 d, 32 signed bytes; w = q * d.  A signed byte b
// becomes the f16 integer b through the bit pattern 0x6400 | (b ^ 0x80) = 1024 + 128 + b, minus 1152.
template <int NT>
__device__ __forceinline__ void q8_0_unit(const uint8_t* rA, const uint8_t* rB, const ActOperand& act, int nblk,
                                          int unit, int gid, int tig, float (&acc)[NT][4]) {
    const uint32_t k1152 = 0x64806480u;
#pragma unroll 2
    for (int b = 0; b < 8; b++) {
        const uint8_t* pA = rA + b * 34;
        const uint8_t* pB = rB + b * 34;
        const float dA = __half2float(*reinterpret_cast<const __half*>(pA));
        const float dB = __half2float(*reinterpret_cast<const __half*>(pB));
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) c[nt][i] = 0.f;
#pragma unroll
        for (int sgrp = 0; sgrp < 2; sgrp++) {
            const uint32_t wA = lds_u32_unaligned(pA + 2 + 16 * sgrp + 4 * tig) ^ 0x80808080u;
            const uint32_t wB = lds_u32_unaligned(pB + 2 + 16 * sgrp + 4 * tig) ^ 0x80808080u;
            uint32_t a[4];
            a[0] = hsub2_u32(__byte_perm(wA, 0x64646464u, 0x4240), k1152);  // elements (0, 2) of the lane's four
            a[1] = hsub2_u32(__byte_perm(wB, 0x64646464u, 0x4240), k1152);
            a[2] = hsub2_u32(__byte_perm(wA, 0x64646464u, 0x4341), k1152);  // elements (1, 3)
            a[3] = hsub2_u32(__byte_perm(wB, 0x64646464u, 0x4341), k1152);
            const int k0 = unit * 256 + b * 32 + 16 * sgrp + 4 * tig;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const __half* xh16 = reinterpret_cast<const __half*>(act.xp);
                const uint2 x = __ldg(reinterpret_cast<const uint2*>(xh16 + act_xp_half_index(nt * 8 + gid, k0, nblk)));
                const uint32_t bb[2] = {x.x, x.y};
                mma_16816(c[nt], a, bb);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            acc[nt][0] += dA * c[nt][0], acc[nt][1] += dA * c[nt][1];
            acc[nt][2] += dB * c[nt][2], acc[nt][3] += dB * c[nt][3];
        }
    }
}

// ---- work decomposition ----------------------------------------------------
// A group is one 16-row tile, or two tiles whose results meet in one epilogue:
//   EPI_SILU        group p: gate rows [16p, 16p+16) and up rows [rows/2 + 16p, ...)
//   EPI_ROPE_STORE  q and k heads: rows [16t, 16t+16) and [16t + hd/2, ...) of a head (the NeoX pair halves);
//                   v heads: single tiles
struct Group {
    int tile0, tile1, n;
};
template <int EPI>
__device__ __forceinline__ int num_groups(int n_tiles, const EpiArgs& e) {
    if (EPI == EPI_SILU || EPI == EPI_MOE_ACT) return n_tiles / 2;
    if (EPI == EPI_ROPE_STORE) {
        const int tph = e.head_dim / 16;  // tiles per head
        return (e.n_q_heads + e.n_kv_heads) * (tph / 2) + (e.n_v_heads < 0 ? e.n_kv_heads : e.n_v_heads) * tph;
    }
    return n_tiles;
}
template <int EPI>
__device__ __forceinline__ Group group_of(int g, int n_tiles, const EpiArgs& e) {
    Group r;
    if (EPI == EPI_SILU || EPI == EPI_MOE_ACT) {
        r.tile0 = g, r.tile1 = n_tiles / 2 + g, r.n = 2;
    } else if (EPI == EPI_ROPE_STORE) {
        const int tph = e.head_dim / 16, pph = tph / 2;
        const int paired = (e.n_q_heads + e.n_kv_heads) * pph;
        if (g < paired) {
            const int head = g / pph, t = g % pph;
            r.tile0 = head * tph + t, r.tile1 = r.tile0 + pph, r.n = 2;
        } else {
            r.tile0 = (e.n_q_heads + e.n_kv_heads) * tph + (g - paired), r.tile1 = 0, r.n = 1;
        }
    } else {
        r.tile0 = g, r.tile1 = 0, r.n = 1;
    }
    return r;
}

// What a group's epilogue will read from global memory, asked for early (an L1 prefetch issued before the
// reduction barrier, so the loads after it find their lines on chip): the residual-stream element and norm weight
// of the thread's output element, or its rotation table entries and row descriptor.
template <int EPI, int NT>
__device__ __forceinline__ void epilogue_prefetch(const EpiArgs& e, const Group& gr, int64_t rows, int tokens, int tok0) {
    const int idx = threadIdx.x;
    if (idx >= NT * 8 * 16) return;
    const int tok = idx >> 4, col = idx & 15;
    if (tok >= tokens) return;
    if constexpr (EPI == EPI_RESID_NORM) {
        const int gcol = gr.tile0 * TILE_ROWS + col;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(e.h + (size_t)(tok0 + tok) * rows + gcol));
        asm volatile("prefetch.global.L1 [%0];" ::"l"(e.g + gcol));
    } else if constexpr (EPI == EPI_ROPE_STORE) {
        const int hd = e.head_dim, tph = hd / 16;
        const int i = (gr.tile0 % tph) * 16 + col;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(e.cs + (size_t)(tok0 + tok) * hd + i));
        asm volatile("prefetch.global.L1 [%0];" ::"l"(e.cs + (size_t)(tok0 + tok) * hd + hd / 2 + i));
        asm volatile("prefetch.global.L1 [%0];" ::"l"(e.row_desc + tok0 + tok));
    }
}

// ---- epilogues: 256 consumer threads, results of the group's tiles in tile_out[which][token][row] ---------
template <int EPI, int NT>
__device__ __forceinline__ void run_epilogue(const EpiArgs& e, const Group& gr, const float* tile_out, const float* inv_rms,
                                             int64_t rows, int tokens, int tok0, uint32_t* err) {
    constexpr int NTOK = NT * 8;
    const int tid = threadIdx.x;
    if constexpr (EPI == EPI_PLAIN || EPI == EPI_SCALE) {
        // (these two epilogues are elementwise and normally run straight out of the reduction: store_plain below)
        const int64_t row0 = (int64_t)gr.tile0 * TILE_ROWS;
        for (int idx = tid; idx < NTOK * 16; idx += CONSUMER_WARPS * 32) {
            const int tok = idx >> 4, row = idx & 15;
            if (tok >= tokens || row0 + row >= rows) continue;
            int out_row = tok0 + tok;
            if (e.y_rows) {
                out_row = e.y_rows[tok0 + tok];
                if (out_row < 0) continue;
            }
            if (e.y_every > 1) {
                if (out_row % e.y_every != e.y_every - 1) continue;
                out_row /= e.y_every;
            }
            float v = tile_out[tok * 16 + row];
            if (EPI == EPI_SCALE) v *= inv_rms[tok];
            const size_t o = (size_t)out_row * e.y_stride + row0 + row;
            if (e.y_f32)
                reinterpret_cast<float*>(e.y)[o] = v;
            else
                reinterpret_cast<__half*>(e.y)[o] = __float2half_rn(v);
        }
    } else if constexpr (EPI == EPI_RESID_NORM) {
        // thread = one (token, column) of the tile; the sixteen columns of a token sit in one half-warp, which sums
        // their h^2 and their operand values with a butterfly
        for (int idx = tid; idx < NTOK * 16; idx += CONSUMER_WARPS * 32) {
            const int tok = idx >> 4, col = idx & 15;
            const bool active = tok < tokens;
            const int gcol = gr.tile0 * TILE_ROWS + col;
            float hn = 0.f, xv = 0.f;
            if (active) {
                __half* hp = e.h + (size_t)(tok0 + tok) * rows + gcol;
                // the matmul output is rounded to f16, then added to the residual stream in fp32 and rounded again
                // (crates/gpu/src/shaders/dequant_q4_k.metal:112-130, utility.metal:199-208)
                const float y = __half2float(__float2half_rn(tile_out[idx]));
                const __half hnew = __float2half_rn(__half2float(*hp) + y);
                *hp = hnew;
                hn = __half2float(hnew);
                const __half xg = __float2half_rn(hn * bf16_bits_to_float(e.g[gcol]));
                reinterpret_cast<__half*>(e.out.xp)[act_xp_half_index(tok0 + tok, gcol, (int)(rows >> 8))] = xg;
                xv = __half2float(xg);
            }
            float ss = hn * hn, sx = xv;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, o);
                sx += __shfl_xor_sync(0xffffffffu, sx, o);
            }
            if (active && col == 0) {
                act_store_sum16(e.out.xs, tok0 + tok, gr.tile0 * TILE_ROWS, (int)(rows >> 8), sx);
                e.ss_out[(size_t)(tok0 + tok) * (rows / 16) + gr.tile0] = ss;
            }
        }
    } else if constexpr (EPI == EPI_SILU || EPI == EPI_MOE_ACT) {
        // pair (gate tile, up tile): thread = one (token, column).  EPI_SILU: gate and up are the normed operand's
        // products, scaled by 1/rms and rounded to f16 first (utility.metal:41-52: (g / (1 + exp(-g))) * u in f32).
        // EPI_MOE_ACT: gate and up stay f32 (crates/gpu/src/shaders/moe_gguf.metal:561-606).
        const int ffn = (int)(rows / 2);
        for (int idx = tid; idx < NTOK * 16; idx += CONSUMER_WARPS * 32) {
            const int tok = idx >> 4, col = idx & 15;
            const bool active = tok < tokens;
            const int gcol = gr.tile0 * TILE_ROWS + col;
            float sx = 0.f;
            if (active) {
                float g = tile_out[idx], u = tile_out[NTOK * 16 + idx];
                if constexpr (EPI == EPI_SILU) {
                    const float inv = inv_rms[tok];
                    g = __half2float(__float2half_rn(inv * g));
                    u = __half2float(__float2half_rn(inv * u));
                }
                const float ex = (float)exp((double)(-g));
                const __half a = __float2half_rn(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, ex)), u));
                reinterpret_cast<__half*>(e.out.xp)[act_xp_half_index(tok0 + tok, gcol, ffn >> 8)] = a;
                sx = __half2float(a);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sx += __shfl_xor_sync(0xffffffffu, sx, o);
            if (active && col == 0) act_store_sum16(e.out.xs, tok0 + tok, gr.tile0 * TILE_ROWS, ffn >> 8, sx);
        }
    } else if constexpr (EPI == EPI_ROPE_STORE) {
        const int hd = e.head_dim, tph = hd / 16;
        const int head = gr.tile0 / tph, t_in = gr.tile0 % tph;
        for (int idx = tid; idx < NTOK * 16; idx += CONSUMER_WARPS * 32) {
            const int tok = idx >> 4, r = idx & 15;
            if (tok >= tokens) continue;
            const float inv = inv_rms[tok];
            const tsb_row_desc rd = e.row_desc[tok0 + tok];
            if (gr.n == 2) {
                // rows i and i + hd/2 of one head: NeoX pair (crates/compute/src/rope.rs:208-255)
                const int i = t_in * 16 + r;
                const float x0 = __half2float(__float2half_rn(inv * tile_out[tok * 16 + r]));
                const float x1 = __half2float(__float2half_rn(inv * tile_out[NTOK * 16 + tok * 16 + r]));
                const float c = e.cs[(size_t)(tok0 + tok) * hd + i], sn = e.cs[(size_t)(tok0 + tok) * hd + hd / 2 + i];
                const __half o0 = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)));
                const __half o1 = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c)));
                __half* dst;
                if (head < e.n_q_heads) {
                    dst = e.q_out + (size_t)(tok0 + tok) * e.n_q_heads * hd + (size_t)head * hd;
                } else {
                    dst = kv_row(e.kv, e.layer, 0, rd.seq, rd.base + rd.slot);
                    if (!dst) {
                        atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
                        continue;
                    }
                    dst += (size_t)(head - e.n_q_heads) * hd;
                }
                dst[i] = o0;
                dst[hd / 2 + i] = o1;
            } else {
                const int vh = head - e.n_q_heads - e.n_kv_heads;
                __half* dst = kv_row(e.kv, e.layer, 1, rd.seq, rd.base + rd.slot);
                if (!dst) {
                    atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
                    continue;
                }
                dst[(size_t)vh * hd + t_in * 16 + r] = __float2half_rn(inv * tile_out[tok * 16 + r]);
            }
        }
    }
}

}  // namespace
