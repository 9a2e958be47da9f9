// Quantized matmul for 16..64 token rows on the fifth-generation tensor cores: y[t, r] = W[r, :] . x[t, :].
//
// One CTA per SM walks 128-row tiles of a Q4_K matrix.  Roles:
//   warp 16      producer: cp.async.bulk copies of raw block rows (two 144-byte blocks per row per stage) and of
//                the activation chunks of each 256-column block into shared-memory rings, counted on mbarriers
//   warps 0-15   dequantisation: thread (row, g) turns the 64 nibbles of group g of its row's block into the
//                integers q * sc (exact in f16) and writes them straight into tensor memory (tcgen05.st) as the A
//                operand of the block's sixteen K=16 steps; a seventeenth step multiplies the sub-block mins m
//                with the activation's 32-column sums (hi + lo f16 split) into a second accumulator.  The block's
//                two accumulators are read back once the next block is dequantised and folded into registers as
//                acc += d * D1 - dmin * D2, so the per-block f16 scales d and dmin never lose a bit
//   warp 17      one thread issues tcgen05.mma (A from tensor memory, B from shared memory through a matrix
//                descriptor, fp32 accumulators in tensor memory) and commits completions onto the ring barriers
//   warps 0-15   epilogue: the tile's register accumulators are stored as f16 or f32
// Every weight byte is dequantised once per tile whatever the token count.
//
// Shared-memory B operand (K-major, no swizzle): chunk c (eight K positions, 16 bytes) of token n sits at
// c * n_pad * 16 + n * 16, so the eight tokens of a row group are contiguous (stride-byte-offset 128 bytes) and
// consecutive K chunks are n_pad * 16 bytes apart (leading-byte-offset).  Within a chunk the K order is
// x0,x2,x1,x3,x4,x6,x5,x7 - the order in which one LOP3 pulls nibble pairs out of a 32-bit word of quants - so
// no byte shuffle is needed on the weight side.  The global copy of the activations is laid out exactly like a
// stage of that ring, which makes the load of a block one bulk copy.
#include "gemm_quant.cuh"

namespace {

constexpr int WM = 128;              // weight rows per tile (UMMA M)
constexpr int WIDE_DEQ_WARPS = 16;
constexpr int WIDE_THREADS = (WIDE_DEQ_WARPS + 2) * 32;
constexpr int WIDE_UPS = 2;          // blocks per row per raw stage
constexpr int WIDE_RAW_STAGES = 3;
constexpr int WIDE_B_STAGES = 3;
constexpr int WIDE_NMAX = 64;        // token rows per pass
constexpr int WIDE_ROWB = WIDE_UPS * 144 + 16;  // row stride in a raw stage: an odd multiple of 16 mod 128, conflict-free LDS.128
constexpr int WIDE_RAW_BYTES = WM * WIDE_ROWB;
constexpr int WIDE_CHUNKS = 34;      // 32 chunks of 8 K positions + 2 chunks of 32-column sums per block
constexpr int WIDE_A_COLS = 136;     // tensor-memory columns of one A slot: 128 (256 f16 K positions) + 8 (sums step)
constexpr int WIDE_TMEM_COLS = 512;

__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hsub2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem_d] (+)= A[tmem_a] * B[smem descriptor]; M = 128, K = 16, f16 inputs, f32 accumulate
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_st2(uint32_t taddr, uint32_t a, uint32_t b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1,%2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tc_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}

struct WideBars {
    uint64_t raw_full[WIDE_RAW_STAGES], raw_empty[WIDE_RAW_STAGES];
    uint64_t b_full[WIDE_B_STAGES], b_empty[WIDE_B_STAGES];
    uint64_t a_full[2], a_empty[2];
    uint64_t d_full, d_empty;
    uint32_t tmem_base;
    uint32_t failed;
};

// x natural [tokens, cols] f16 -> per 256-column block, 34 chunks x n_pad tokens x 16 bytes (see the file header)
__global__ void wide_prepare_kernel(const __half* __restrict__ x, int64_t x_stride, int tokens, int n_pad, int units,
                                    uint4* __restrict__ xw) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)units * WIDE_CHUNKS * n_pad;
    if (idx >= total) return;
    const int n = (int)(idx % n_pad);
    const int c = (int)((idx / n_pad) % WIDE_CHUNKS);
    const int blk = (int)(idx / ((int64_t)n_pad * WIDE_CHUNKS));
    uint4 o = make_uint4(0, 0, 0, 0);
    if (n < tokens) {
        const __half* row = x + (size_t)n * x_stride + (size_t)blk * 256;
        if (c < 32) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + 8 * c);
            __half h[8];
            *reinterpret_cast<uint4*>(h) = raw;
            o = act_pack8(h);
        } else {
            __half out[8];
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const __half* p = row + ((c - 32) * 4 + s) * 32;
                float sum = 0.f;
                for (int i = 0; i < 32; i++) sum += __half2float(p[i]);
                const __half hi = __float2half_rn(sum);
                out[2 * s] = hi;
                out[2 * s + 1] = __float2half_rn(sum - __half2float(hi));
            }
            o = *reinterpret_cast<uint4*>(out);
        }
    }
    xw[idx] = o;
}

__global__ void __launch_bounds__(WIDE_THREADS, 1)
    gemm_wide_q4k_kernel(const uint8_t* __restrict__ W, int64_t rows, int units, const uint4* __restrict__ xw, int n_pad, int tokens,
                         void* __restrict__ y, int64_t y_stride, int y_f32, int ksplit, float* __restrict__ part,
                         uint32_t* __restrict__ err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    WideBars* bars = reinterpret_cast<WideBars*>(smem);
    uint8_t* raw_ring = smem + 1024;
    uint8_t* b_ring = raw_ring + WIDE_RAW_STAGES * WIDE_RAW_BYTES;
    const int b_stage_bytes = WIDE_CHUNKS * n_pad * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a work item is a 128-row tile, or (matrices with few tiles) one of `ksplit` runs of its blocks; the partial
    // sums of the runs go to `part` and a small kernel adds them in run order
    const int n_items = (int)(rows / WM) * ksplit;
    const int64_t row_bytes = (int64_t)units * 144;
    const int upk = ((units + ksplit - 1) / ksplit + WIDE_UPS - 1) / WIDE_UPS * WIDE_UPS;  // blocks per run, whole raw stages
    auto item_blocks = [&](int item, int* b0) {
        *b0 = (item % ksplit) * upk;
        return max(0, min(units, *b0 + upk) - *b0);
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < WIDE_RAW_STAGES; i++) mbar_init(&bars->raw_full[i], 1), mbar_init(&bars->raw_empty[i], WIDE_DEQ_WARPS);
        for (int i = 0; i < WIDE_B_STAGES; i++) mbar_init(&bars->b_full[i], 1), mbar_init(&bars->b_empty[i], 1);
        for (int i = 0; i < 2; i++) mbar_init(&bars->a_full[i], WIDE_DEQ_WARPS), mbar_init(&bars->a_empty[i], 1);
        mbar_init(&bars->d_full, 1), mbar_init(&bars->d_empty, WIDE_DEQ_WARPS);
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == WIDE_DEQ_WARPS + 1) {  // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)WIDE_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    const uint32_t tmem_d1 = tmem;                    // block accumulator of the quants, WIDE_NMAX columns
    const uint32_t tmem_d2 = tmem + WIDE_NMAX;        // block accumulator of the mins
    const uint32_t tmem_a0 = tmem + 2 * WIDE_NMAX;    // two A slots of WIDE_A_COLS columns
    pdl_wait();

    if (warp == WIDE_DEQ_WARPS) {
        // ---- producer
        uint32_t nraw = 0, nb = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            int b0;
            const int nblk = item_blocks(item, &b0);
            const int raw_iters = (nblk + WIDE_UPS - 1) / WIDE_UPS;
            const uint8_t* wt = W + (int64_t)(item / ksplit) * WM * row_bytes + (int64_t)b0 * 144;
            for (int it = 0; it < raw_iters && ok; it++, nraw++) {
                const uint32_t s = nraw % WIDE_RAW_STAGES;
                if (nraw >= WIDE_RAW_STAGES) ok = mbar_wait(&bars->raw_empty[s], ((nraw / WIDE_RAW_STAGES) - 1) & 1, err);
                if (!ok) break;
                const int nun = min(WIDE_UPS, nblk - it * WIDE_UPS);
                const uint32_t per_row = (uint32_t)nun * 144u;
                if (lane == 0) mbar_expect_tx(&bars->raw_full[s], per_row * WM);
                __syncwarp();
#pragma unroll
                for (int r = 0; r < WM / 32; r++) {
                    const int row = r * 32 + lane;
                    bulk_g2s(raw_ring + s * WIDE_RAW_BYTES + row * WIDE_ROWB, wt + row * row_bytes + (int64_t)it * WIDE_UPS * 144, per_row,
                             &bars->raw_full[s]);
                }
                // the activation chunks of the blocks of this stage
                for (int u = 0; u < nun && ok; u++, nb++) {
                    const uint32_t bs = nb % WIDE_B_STAGES;
                    if (nb >= WIDE_B_STAGES) ok = mbar_wait(&bars->b_empty[bs], ((nb / WIDE_B_STAGES) - 1) & 1, err);
                    if (!ok) break;
                    if (lane == 0) {
                        mbar_expect_tx(&bars->b_full[bs], (uint32_t)b_stage_bytes);
                        bulk_g2s(b_ring + bs * b_stage_bytes, xw + (size_t)(b0 + it * WIDE_UPS + u) * WIDE_CHUNKS * n_pad, (uint32_t)b_stage_bytes,
                                 &bars->b_full[bs]);
                    }
                    __syncwarp();
                }
            }
        }
        if (!ok) bars->failed = 1;
    } else if (warp == WIDE_DEQ_WARPS + 1) {
        // ---- MMA issue: one thread
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, f16 A and B, both K-major, N = n_pad, M = 128
            const uint32_t idesc = (1u << 4) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(WM >> 4) << 24);
            // shared-memory matrix descriptor of B without the start address: leading-byte-offset = chunk stride,
            // stride-byte-offset = 128 (eight tokens of 16 bytes), descriptor version 1, no swizzle
            const uint64_t desc_hi = ((uint64_t)((uint32_t)(n_pad * 16) >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
            uint32_t nb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int b0;
                const int nblk = item_blocks(item, &b0);
                for (int blk = 0; blk < nblk && ok; blk++, nb++) {
                    const uint32_t as = nb & 1, bs = nb % WIDE_B_STAGES;
                    ok = mbar_wait(&bars->a_full[as], (nb >> 1) & 1, err) && mbar_wait(&bars->b_full[bs], (nb / WIDE_B_STAGES) & 1, err);
                    if (ok && nb >= 1) ok = mbar_wait(&bars->d_empty, (nb - 1) & 1, err);  // the previous block's accumulators were read
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t b_addr = smem_u32(b_ring + bs * b_stage_bytes);
                    const uint32_t a_col = tmem_a0 + as * WIDE_A_COLS;
#pragma unroll 1
                    for (int j = 0; j < 17; j++) {
                        const uint64_t desc = desc_hi | (uint64_t)(((b_addr + (uint32_t)(2 * j) * (uint32_t)(n_pad * 16)) >> 4) & 0x3FFFu);
                        tc_mma_ts(j < 16 ? tmem_d1 : tmem_d2, a_col + 8 * j, desc, idesc, (j & 15) ? 1u : 0u);
                    }
                    tc_commit(&bars->a_empty[as]);
                    tc_commit(&bars->b_empty[bs]);
                    tc_commit(&bars->d_full);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else {
        // ---- dequantisation warps (also the epilogue): thread = (row of the tile, group g of the block)
        const int q4 = warp & 3, g = warp >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        uint32_t nraw = 0, nb = 0;
        bool ok = true;
        // the accumulator columns (token rows) are dealt evenly to the four warps of a lane quadrant: n_pad / 4 each
        const int cpw = n_pad >> 2;
        // fold block `which`'s accumulators into the registers: acc += d * D1 - dmin * D2
        auto drain = [&](uint32_t which, float d, float dmin, float (&acc)[16]) {
            if (ok) ok = mbar_wait(&bars->d_full, which & 1, err);
            if (ok) {
                tc_fence_after();
                // eight columns per round trip keeps the loaded values in sixteen registers
#pragma unroll
                for (int h = 0; h < 2; h++)
                    if (8 * h < cpw) {
                        uint32_t a4[2][4], b4[2][4];
#pragma unroll
                        for (int q = 0; q < 2; q++)
                            if (8 * h + 4 * q < cpw) {
                                tc_ld4(tmem_d1 + lane_base + g * cpw + 8 * h + 4 * q, a4[q]);
                                tc_ld4(tmem_d2 + lane_base + g * cpw + 8 * h + 4 * q, b4[q]);
                            }
                        tc_wait_ld();
#pragma unroll
                        for (int q = 0; q < 2; q++)
                            if (8 * h + 4 * q < cpw) {
#pragma unroll
                                for (int i = 0; i < 4; i++)
                                    acc[8 * h + 4 * q + i] = fmaf(d, __uint_as_float(a4[q][i]), fmaf(-dmin, __uint_as_float(b4[q][i]), acc[8 * h + 4 * q + i]));
                            }
                    }
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&bars->d_empty);
        };
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            int b0;
            const int nblk = item_blocks(item, &b0);
            const int raw_iters = (nblk + WIDE_UPS - 1) / WIDE_UPS;
            const int tile = item / ksplit, ks = item % ksplit;
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.f;
            float d_prev = 0.f, dmin_prev = 0.f;
            int blk = 0;
            for (int it = 0; it < raw_iters; it++, nraw++) {
                const uint32_t s = nraw % WIDE_RAW_STAGES;
                if (ok) ok = mbar_wait(&bars->raw_full[s], (nraw / WIDE_RAW_STAGES) & 1, err);
                const int nun = min(WIDE_UPS, nblk - it * WIDE_UPS);
                for (int u = 0; u < nun; u++, nb++, blk++) {
                    const uint32_t as = nb & 1;
                    if (ok && nb >= 2) ok = mbar_wait(&bars->a_empty[as], ((nb >> 1) - 1) & 1, err);
                    float d = 0.f, dmin = 0.f;
                    if (ok) {
                        tc_fence_after();
                        const uint8_t* bp = raw_ring + s * WIDE_RAW_BYTES + row * WIDE_ROWB + u * 144;
                        const uint4 hdr = *reinterpret_cast<const uint4*>(bp);
                        const uint4 qa = *reinterpret_cast<const uint4*>(bp + 16 + 32 * g);
                        const uint4 qb = *reinterpret_cast<const uint4*>(bp + 32 + 32 * g);
                        const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
                        d = __low2float(dd), dmin = __high2float(dd);
                        // 6-bit scale / min of sub-blocks j = 2g and 2g+1 (crates/compute/src/quant_gguf/q4_k.rs:43-54): byte
                        // j & 3 of the scale word (j < 4) or of the high word combined with two bits of the low words (j >= 4)
                        uint32_t scv[2], mv[2];
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int sh = 16 * (g & 1) + 8 * h;
                            const uint32_t y = hdr.y >> sh, z = hdr.z >> sh, w = hdr.w >> sh;
                            if (g < 2) {
                                scv[h] = y & 63u, mv[h] = z & 63u;
                            } else {
                                scv[h] = (w & 0xFu) | ((y >> 2) & 0x30u);
                                mv[h] = ((w >> 4) & 0xFu) | ((z >> 2) & 0x30u);
                            }
                        }
                        // integers up to 63 as f16 pairs: (0x6400 | v) is 1024 + v
                        const uint32_t k1024 = 0x64006400u;
                        const uint32_t s0 = hsub2_bits(scv[0] * 0x00010001u | k1024, k1024), s1 = hsub2_bits(scv[1] * 0x00010001u | k1024, k1024);
                        const uint32_t m0 = hsub2_bits(mv[0] * 0x00010001u | k1024, k1024), m1 = hsub2_bits(mv[1] * 0x00010001u | k1024, k1024);
                        const uint32_t off0 = hmul2_bits(s0, 0xE400E400u);  // -1024 * sc, exact
                        const uint32_t off1 = hmul2_bits(s1, 0xD400D400u);  // -64 * sc, exact
                        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                        uint32_t r[32];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const uint32_t v = w[i], v8 = v >> 8;
                            r[2 * i] = hfma2_u32(lop3_and_or(v, 0x000F000Fu, 0x64006400u), s0, off0);  // q * sc, exact
                            r[2 * i + 1] = hfma2_u32(lop3_and_or(v8, 0x000F000Fu, 0x64006400u), s0, off0);
                            r[16 + 2 * i] = hfma2_u32(lop3_and_or(v, 0x00F000F0u, 0x54005400u), s1, off1);
                            r[16 + 2 * i + 1] = hfma2_u32(lop3_and_or(v8, 0x00F000F0u, 0x54005400u), s1, off1);
                        }
                        const uint32_t a_col = tmem_a0 + as * WIDE_A_COLS + lane_base;
                        tc_st32(a_col + 32 * g, r);
                        tc_st2(a_col + 128 + 2 * g, m0, m1);
                    }
                    // while the stores to tensor memory are in flight: the previous block's products are ready by now
                    // (its MMAs ran under this block's dequantisation)
                    if (blk > 0) drain(nb - 1, d_prev, dmin_prev, acc);
                    if (ok) {
                        tc_wait_st();
                        tc_fence_before();
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&bars->a_full[as]);
                    d_prev = d, dmin_prev = dmin;
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&bars->raw_empty[s]);
            }
            if (nblk > 0) drain(nb - 1, d_prev, dmin_prev, acc);  // the item's last block
            if (ok) {
                const int64_t orow = (int64_t)tile * WM + row;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int n = g * cpw + i;
                    if (i < cpw && n < tokens) {
                        if (ksplit > 1)
                            part[((size_t)ks * tokens + n) * rows + orow] = acc[i];
                        else if (y_f32)
                            reinterpret_cast<float*>(y)[(size_t)n * y_stride + orow] = acc[i];
                        else
                            reinterpret_cast<__half*>(y)[(size_t)n * y_stride + orow] = __float2half_rn(acc[i]);
                    }
                }
            }
        }
        if (!ok && lane == 0) bars->failed = 1;
    }
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == WIDE_DEQ_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)WIDE_TMEM_COLS) : "memory");
    }
}

// y[n, r] = sum over runs, in run order, of part[run][n][r]
__global__ void wide_reduce_kernel(const float* __restrict__ part, int ksplit, int tokens, int64_t rows, void* __restrict__ y,
                                   int64_t y_stride, int y_f32) {
    pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)tokens * rows) return;
    const int n = (int)(idx / rows);
    const int64_t r = idx % rows;
    float v = 0.f;
    for (int k = 0; k < ksplit; k++) v += part[((size_t)k * tokens + n) * rows + r];
    if (y_f32)
        reinterpret_cast<float*>(y)[(size_t)n * y_stride + r] = v;
    else
        reinterpret_cast<__half*>(y)[(size_t)n * y_stride + r] = __float2half_rn(v);
}

}  // namespace

bool gemm_wide_supported(int qtype, int64_t rows, int64_t cols, int tokens) {
    return qtype == TSB_Q4_K && rows % WM == 0 && cols % 256 == 0 && tokens >= 1;
}

// x natural f16 [tokens, cols]; y [tokens, rows].  Token rows go through in passes of 64.
// how many runs a tile's blocks are cut into so that a matrix with few 128-row tiles still fills the device
static int wide_ksplit(const tsb_ctx* ctx, int64_t rows, int units) {
    const int tiles = (int)(rows / WM);
    int k = 1;
    while (k < 8 && tiles * (k * 2) <= ctx->sm_count + ctx->sm_count / 4 && units / (k * 2) >= 4) k *= 2;
    return k;
}
size_t gemm_wide_workspace_bytes(int64_t cols) { return (size_t)(cols / 256) * WIDE_CHUNKS * WIDE_NMAX * 16; }
size_t gemm_wide_partial_bytes(const tsb_ctx* ctx, int64_t rows, int64_t cols) {
    const int k = wide_ksplit(ctx, rows, (int)(cols / 256));
    return k > 1 ? (size_t)k * WIDE_NMAX * rows * sizeof(float) : 0;
}

cudaError_t launch_gemm_wide_q4k(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int64_t cols, const __half* x,
                                 int64_t x_stride, int tokens, void* y, int64_t y_stride, bool y_f32, void* workspace, void* partials) {
    const int units = (int)(cols / 256);
    const int ksplit = wide_ksplit(ctx, rows, units);
    static SmemOptIn configured;
    const size_t smem_max = 1024 + (size_t)WIDE_RAW_STAGES * WIDE_RAW_BYTES + (size_t)WIDE_B_STAGES * WIDE_CHUNKS * WIDE_NMAX * 16;
    if (cudaError_t e = tsb_opt_in_smem(ctx, gemm_wide_q4k_kernel, smem_max, configured); e != cudaSuccess) return e;
    for (int t0 = 0; t0 < tokens; t0 += WIDE_NMAX) {
        const int nt = min(WIDE_NMAX, tokens - t0);
        const int n_pad = (nt + 15) / 16 * 16;
        uint4* xw = static_cast<uint4*>(workspace);  // successive passes reuse it in stream order
        const size_t xw_bytes = (size_t)units * WIDE_CHUNKS * n_pad * 16;
        cudaError_t e = cudaSuccess;
        if (!workspace) e = cudaMallocAsync((void**)&xw, xw_bytes, st);
        if (e != cudaSuccess) return e;
        const int64_t total = (int64_t)units * WIDE_CHUNKS * n_pad;
        e = tsb_launch(ctx, wide_prepare_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true, x + (size_t)t0 * x_stride,
                       x_stride, nt, n_pad, units, xw);
        if (e == cudaSuccess) {
            // one CTA per SM: the kernel wants the whole tensor memory and most of the shared memory
            const size_t smem = 1024 + (size_t)WIDE_RAW_STAGES * WIDE_RAW_BYTES + (size_t)WIDE_B_STAGES * WIDE_CHUNKS * n_pad * 16;
            const int n_items = (int)(rows / WM) * ksplit;
            dim3 grid((unsigned)min(n_items, ctx->sm_count));
            uint8_t* yp = static_cast<uint8_t*>(y) + (size_t)t0 * y_stride * (y_f32 ? 4 : 2);
            float* part = static_cast<float*>(partials);
            if (ksplit > 1 && !part) e = cudaMallocAsync((void**)&part, (size_t)ksplit * nt * rows * sizeof(float), st);
            if (e == cudaSuccess)
                e = tsb_launch(ctx, gemm_wide_q4k_kernel, grid, dim3(WIDE_THREADS), smem, st, true, w, rows, units, (const uint4*)xw, n_pad,
                               nt, (void*)yp, y_stride, (int)(y_f32 ? 1 : 0), ksplit, part, ctx->dev_error);
            if (e == cudaSuccess && ksplit > 1) {
                const int64_t total = (int64_t)nt * rows;
                e = tsb_launch(ctx, wide_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true, (const float*)part,
                               ksplit, nt, rows, (void*)yp, y_stride, (int)(y_f32 ? 1 : 0));
            }
            if (ksplit > 1 && !partials && part) cudaFreeAsync(part, st);
        }
        if (!workspace) cudaFreeAsync(xw, st);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}
