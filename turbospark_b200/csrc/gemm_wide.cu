// Quantized matmul for 24..128 token rows per pass on the fifth-generation tensor cores: y[t, r] = W[r, :] . x[t, :].
//
// One CTA per SM walks 128-row tiles of a Q4_K matrix.  Roles:
//   warp 16      producer: cp.async.bulk copies of raw block rows (two 144-byte blocks per row per stage) and of
//                the activation chunks of each 256-column block into shared-memory rings, counted on mbarriers
//   warps 0-15   dequantisation: thread (row, g) turns the 64 nibbles of group g of its row's block into the
//                integers q * sc (exact in f16) and writes them straight into tensor memory (tcgen05.st) as the A
//                operand of the block's sixteen K=16 steps; the sub-block mins m go to a small shared-memory tile
//                that a seventeenth step multiplies with the activation's 32-column sums (hi + lo f16 split) into
//                a second accumulator.  A block's two accumulators are read back (tcgen05.ld) and folded into
//                registers as acc += d * D1 - dmin * D2, so the per-block f16 scales d and dmin never lose a bit
//   warp 17      one thread issues tcgen05.mma (A from tensor memory, or from shared memory for the mins step; B from
//                shared memory through a matrix descriptor; fp32 accumulators in tensor memory) and commits
//                completions onto the ring barriers
//   warps 0-15   epilogue: the tile's register accumulators are stored as f16 or f32
// Every weight byte is dequantised once per tile whatever the token count.
//
// Tensor memory (512 columns): two A slots of 128 columns, then the accumulators.  Up to 64 token rows there are two
// accumulator sets (D1 | D2 of n_pad columns each) and a block is folded two blocks after it was written: its MMAs
// have long finished, so the dequantising warps never wait for the tensor pipe.  From 80 to 128 token rows one set
// fills the rest of tensor memory and a block is folded right after the next one is dequantised.
//
// Shared-memory B operand (K-major, no swizzle): chunk c (eight K positions, 16 bytes) of token n sits at
// c * n_pad * 16 + n * 16, so the eight tokens of a row group are contiguous (stride-byte-offset 128 bytes) and
// consecutive K chunks are n_pad * 16 bytes apart (leading-byte-offset).  Within a chunk the K order is
// x0,x2,x1,x3,x4,x6,x5,x7 - the order in which one LOP3 pulls nibble pairs out of a 32-bit word of quants - so
// no byte shuffle is needed on the weight side.  The global copy of the activations is laid out exactly like a
// stage of that ring, which makes the load of a block one bulk copy.  The mins tile is the same layout with weight
// rows in place of tokens: chunk c of row r at c * 2048 + r * 16.
#include <cuda.h>

#include <map>
#include <mutex>

#include "gemm_quant.cuh"
#include "tc05.cuh"

namespace {

constexpr int WM = 128;              // weight rows per tile (UMMA M)
constexpr int WIDE_DEQ_WARPS = 16;
constexpr int WIDE_THREADS = (WIDE_DEQ_WARPS + 3) * 32;  // + raw-block producer, MMA issuer, activation producer
constexpr int WIDE_RAW_STAGES = 4;   // raw blocks in flight (one 128-row x 144-byte box each)
constexpr int WIDE_RAW_BYTES = WM * 144;
constexpr int WIDE_B_STAGES = 3;     // activation ring: 3 stages up to 64 token rows, 2 above (a stage doubles)
constexpr int WIDE_NMAX = 128;       // token rows per pass
constexpr int WIDE_NDUAL = 64;       // up to here two accumulator sets fit tensor memory
constexpr int WIDE_CHUNKS = 34;      // 32 chunks of 8 K positions + 2 chunks of 32-column sums per block
constexpr int WIDE_A_COLS = 128;     // tensor-memory columns of one A slot: 256 f16 K positions
constexpr int WIDE_MIN_BYTES = WM * 16 * 2;  // the mins step's A operand: 128 rows x 16 K positions of f16
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
#ifdef TSB_WIDE_TRACE
// development builds: nanosecond stamps of CTA 0 - [blk][0..7] from dequantising warp 0, [blk][8..11] from the MMA thread
__device__ unsigned long long* g_wide_trace = nullptr;
#define WTRC(blk, i) do { if (wtrc && lane == 0 && (blk) < 64) wtrc[(blk) * 16 + (i)] = global_timer_ns(); } while (0)
#else
#define WTRC(blk, i)
#endif

struct WideBars {
    uint64_t raw_full[WIDE_RAW_STAGES], raw_empty[WIDE_RAW_STAGES];
    uint64_t b_full[WIDE_B_STAGES], b_empty[WIDE_B_STAGES];
    uint64_t a_full[2];    // block nb's A operand and mins are written, and the block lag blocks back is folded
    uint64_t mma_done[2];  // block nb's MMAs have finished: its A slot is free and its accumulators are complete
    uint32_t tmem_base;
    uint32_t failed;
    uint32_t ticket;
};

// x natural [tokens, cols] f16 -> for every pass of `per_pass` token rows and every 256-column block, 34 chunks x n_pad
// tokens x 16 bytes (see the file header); pass p starts at p * units * 34 * per_pass chunks and its own n_pad is its
// token count rounded up to 16.  A CTA takes eight tokens of one block: warp = token, lane = 16-byte chunk; the
// 32-column sums come from two shuffles over the four lanes of a sub-block; the CTA's 34 x 8 chunks go out through
// shared memory as 128-byte runs.
__global__ void __launch_bounds__(256) wide_prepare_kernel(const __half* __restrict__ x, int64_t x_stride, int tokens, int per_pass, int units,
                                                           uint4* __restrict__ xw) {
    __shared__ uint4 tile[WIDE_CHUNKS][8];
    pdl_wait();
    const int blk = blockIdx.x;
    const int pass = blockIdx.y / (per_pass >> 3), grp = blockIdx.y % (per_pass >> 3);
    const int nt = min(per_pass, tokens - pass * per_pass);  // token rows of this pass
    const int n_pad = (nt + 15) / 16 * 16;
    if (nt <= 0 || grp * 8 >= n_pad) return;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = grp * 8 + w;  // token row within the pass
    uint4 o = make_uint4(0, 0, 0, 0);
    float sum = 0.f;
    if (n < nt) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(pass * per_pass + n) * x_stride + (size_t)blk * 256 + 8 * lane);
        __half h[8];
        *reinterpret_cast<uint4*>(h) = raw;
#pragma unroll
        for (int i = 0; i < 8; i++) sum += __half2float(h[i]);
        o = act_pack8(h);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    tile[lane][w] = o;
    if ((lane & 3) == 0) {  // sub-block lane / 4: (hi, lo) halves at chunk 32 + sub / 4, pair sub % 4
        const int sub = lane >> 2;
        const __half hi = __float2half_rn(sum);
        const __half2 hl = __halves2half2(hi, __float2half_rn(sum - __half2float(hi)));
        reinterpret_cast<__half2*>(&tile[32 + (sub >> 2)][w])[sub & 3] = hl;
    }
    __syncthreads();
    uint4* dst = xw + (size_t)pass * units * WIDE_CHUNKS * per_pass + (size_t)blk * WIDE_CHUNKS * n_pad;
    for (int i = threadIdx.x; i < WIDE_CHUNKS * 8; i += 256) {
        const int c = i >> 3, t = i & 7;
        dst[(size_t)c * n_pad + grp * 8 + t] = tile[c][t];
    }
}

// One box of the weight matrix (128 rows x one 144-byte block) lands as 128 consecutive 144-byte rows: a lane stride
// of nine 16-byte units, so the 128-bit loads of 32 consecutive rows do not collide.
__device__ __forceinline__ void tensor_g2s_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// ROUNDS: how many 16-column read-backs cover a warp's share of the accumulator columns (n_pad / 4 <= 16 * ROUNDS)
template <int ROUNDS>
__global__ void __launch_bounds__(WIDE_THREADS, 1)
    gemm_wide_q4k_kernel(const __grid_constant__ CUtensorMap wmap, int64_t rows, int units, const uint4* __restrict__ xw, int n_pad,
                         int tokens, void* __restrict__ y, int64_t y_stride, int y_f32, int n_whole, int ksplit, float* __restrict__ part,
                         uint32_t* __restrict__ err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    WideBars* bars = reinterpret_cast<WideBars*>(smem);
    // accumulator sets and the depth of the activation ring follow the pass's width (see the file header)
    const uint32_t n_sets = n_pad <= WIDE_NDUAL ? 2u : 1u;
    const uint32_t n_bst = n_pad <= WIDE_NDUAL ? 3u : 2u;
    uint8_t* raw_ring = smem + 1024;
    uint8_t* min_ring = raw_ring + WIDE_RAW_STAGES * WIDE_RAW_BYTES;
    uint8_t* b_ring = min_ring + 2 * WIDE_MIN_BYTES;
    const int b_stage_bytes = WIDE_CHUNKS * n_pad * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef TSB_WIDE_TRACE
    unsigned long long* const wtrc = blockIdx.x == 0 ? g_wide_trace : nullptr;
#endif
    // Work items, dealt round-robin to the CTAs: the first n_whole tiles (a multiple of the grid) go whole; each of the
    // remaining tiles - fewer than CTAs - is cut into `ksplit` runs of its blocks so that the last wave fills the
    // device too.  A run leaves its partial sums in `part` (after 1024 ticket words); the CTA that finishes a tile's last
    // run adds them in run order and writes the tile.
    const int n_tiles = (int)(rows / WM);
    const int n_items = n_whole + (n_tiles - n_whole) * ksplit;
    const int upk = (units + ksplit - 1) / ksplit;  // blocks per run
    struct Item {
        int tile, b0, nblk, ks;  // ks < 0: a whole tile
    };
    auto item_of = [&](int item) {
        Item it;
        if (item < n_whole) {
            it.tile = item, it.b0 = 0, it.nblk = units, it.ks = -1;
        } else {
            const int t = item - n_whole;
            it.tile = n_whole + t / ksplit, it.ks = ksplit > 1 ? t % ksplit : -1;
            it.b0 = (t % ksplit) * upk;
            it.nblk = max(0, min(units, it.b0 + upk) - it.b0);
        }
        return it;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < WIDE_RAW_STAGES; i++) mbar_init(&bars->raw_full[i], 1), mbar_init(&bars->raw_empty[i], WIDE_DEQ_WARPS);
        for (int i = 0; i < WIDE_B_STAGES; i++) mbar_init(&bars->b_full[i], 1), mbar_init(&bars->b_empty[i], 1);
        for (int i = 0; i < 2; i++) mbar_init(&bars->a_full[i], WIDE_DEQ_WARPS), mbar_init(&bars->mma_done[i], 1);
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
    const uint32_t tmem_a0 = tmem;                       // two A slots of WIDE_A_COLS columns
    const uint32_t tmem_acc = tmem + 2 * WIDE_A_COLS;    // set s: D1 (quants) at s * 2 * n_pad, D2 (mins) n_pad columns further
    pdl_wait();

    if (warp == WIDE_DEQ_WARPS) {
        // ---- producer of the raw blocks: one tensor copy (128 rows x 144 bytes) per block
        if (lane == 0) {
            uint32_t nb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item wi = item_of(item);
                const int b0 = wi.b0, nblk = wi.nblk, row0 = wi.tile * WM;
                for (int blk = 0; blk < nblk && ok; blk++, nb++) {
                    const uint32_t s = nb % WIDE_RAW_STAGES;
                    if (nb >= WIDE_RAW_STAGES) ok = mbar_wait(&bars->raw_empty[s], ((nb / WIDE_RAW_STAGES) - 1) & 1, err);
                    if (!ok) break;
                    mbar_expect_tx(&bars->raw_full[s], (uint32_t)WIDE_RAW_BYTES);
                    tensor_g2s_2d(raw_ring + s * WIDE_RAW_BYTES, &wmap, (b0 + blk) * 36, row0, &bars->raw_full[s]);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (warp == WIDE_DEQ_WARPS + 2) {
        // ---- producer of the activation chunks: its own warp, so a full activation ring never holds up the weights
        if (lane == 0) {
            uint32_t nb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item wi = item_of(item);
                const int b0 = wi.b0, nblk = wi.nblk;
                (void)b0;
                for (int blk = 0; blk < nblk && ok; blk++, nb++) {
                    const uint32_t bs = nb % n_bst;
                    if (nb >= n_bst) ok = mbar_wait(&bars->b_empty[bs], ((nb / n_bst) - 1) & 1, err);
                    if (!ok) break;
                    mbar_expect_tx(&bars->b_full[bs], (uint32_t)b_stage_bytes);
                    bulk_g2s(b_ring + bs * b_stage_bytes, xw + (size_t)(b0 + blk) * WIDE_CHUNKS * n_pad, (uint32_t)b_stage_bytes, &bars->b_full[bs]);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (warp == WIDE_DEQ_WARPS + 1) {
        // ---- MMA issue: the warp walks the blocks together, lane 0 issues
        {
            const uint32_t leader = lane == 0 ? 1u : 0u;
            // instruction descriptor: f32 accumulate, f16 A and B, both K-major, N = n_pad, M = 128
            const uint32_t idesc = (1u << 4) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(WM >> 4) << 24);
            // shared-memory matrix descriptor of B without the start address: leading-byte-offset = chunk stride,
            // stride-byte-offset = 128 (eight tokens of 16 bytes), descriptor version 1, no swizzle
            const uint64_t desc_hi = ((uint64_t)((uint32_t)(n_pad * 16) >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
            // the mins tile: chunk stride 128 rows x 16 bytes, eight rows of 16 bytes per row group
            const uint64_t desc_min_hi = ((uint64_t)((uint32_t)(WM * 16) >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
            uint32_t nb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item wi = item_of(item);
                const int nblk = wi.nblk;
                for (int blk = 0; blk < nblk && ok; blk++, nb++) {
                    const uint32_t as = nb & 1, bs = nb % n_bst, set = nb % n_sets;
                    // a_full also says that the block this one's accumulator set held before is folded: every warp folds
                    // before it arrives
                    ok = mbar_wait(&bars->a_full[as], (nb >> 1) & 1, err) && mbar_wait(&bars->b_full[bs], (nb / n_bst) & 1, err);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    WTRC(nb, 8);
                    tc_fence_after();
                    const uint32_t a_col = tmem_a0 + as * WIDE_A_COLS;
                    const uint32_t d1 = tmem_acc + set * 2 * (uint32_t)n_pad, d2 = d1 + (uint32_t)n_pad;
                    // consecutive K steps are two chunks apart: the descriptor's address field (16-byte units) moves by 2 * n_pad
                    const uint64_t desc0 = desc_hi | (uint64_t)((smem_u32(b_ring + bs * b_stage_bytes) >> 4) & 0x3FFFu);
                    const uint64_t step = (uint64_t)(2 * n_pad);
                    tc_mma_ts<false>(leader, d1, a_col, desc0, idesc);
#pragma unroll
                    for (int j = 1; j < 16; j++) tc_mma_ts<true>(leader, d1, a_col + 8 * j, desc0 + (uint64_t)j * step, idesc);
                    tc_mma_ss<false>(leader, d2, desc_min_hi | (uint64_t)((smem_u32(min_ring + as * WIDE_MIN_BYTES) >> 4) & 0x3FFFu), desc0 + 16 * step,
                                     idesc);
                    tc_commit_if(leader, &bars->mma_done[as]);
                    tc_commit_if(leader, &bars->b_empty[bs]);
                    WTRC(nb, 9);
                }
            }
            if (!ok && lane == 0) bars->failed = 1;
        }
    } else {
        // ---- dequantisation warps (also the epilogue): thread = (row of the tile, group g of the block)
        const int q4 = warp & 3, g = warp >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        uint32_t nb = 0;
        bool ok = true;
        // the accumulator columns (token rows) are dealt evenly to the four warps of a lane quadrant: n_pad / 4 each
        const int cpw = n_pad >> 2;
        const uint32_t lag = n_sets;  // a block is folded `lag` blocks after it was written
        // fold block `which`'s accumulators into the registers: acc += d * D1 - dmin * D2
        auto drain = [&](uint32_t which, float d, float dmin, float (&acc)[16 * ROUNDS]) {
            const uint32_t set = which % n_sets;
            if (ok) ok = mbar_wait(&bars->mma_done[which & 1], (which >> 1) & 1, err);
            if (ok) {
                tc_fence_after();
                const uint32_t d1 = tmem_acc + set * 2 * (uint32_t)n_pad + lane_base + g * cpw, d2 = d1 + (uint32_t)n_pad;
#pragma unroll
                for (int h = 0; h < ROUNDS; h++)
                    if (16 * h < cpw) {
                        // sixteen columns per round trip; columns past this warp's share are read and dropped
                        uint32_t a16[16], b16[16];
                        tc_ld16(d1 + 16 * h, a16);
                        tc_ld16(d2 + 16 * h, b16);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            acc[16 * h + i] = fmaf(d, __uint_as_float(a16[i]), fmaf(-dmin, __uint_as_float(b16[i]), acc[16 * h + i]));
                    }
                tc_fence_before();
            }
        };
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const Item wi = item_of(item);
            const int nblk = wi.nblk, tile = wi.tile, ks = wi.ks;
            const int64_t tail_rows = (int64_t)(n_tiles - n_whole) * WM;
            float acc[16 * ROUNDS];
#pragma unroll
            for (int i = 0; i < 16 * ROUNDS; i++) acc[i] = 0.f;
            float d_p1 = 0.f, dmin_p1 = 0.f, d_p2 = 0.f, dmin_p2 = 0.f;  // scales of the last and the last-but-one block
            for (int blk = 0; blk < nblk; blk++, nb++) {
                const uint32_t s = nb % WIDE_RAW_STAGES, as = nb & 1;
                if (warp == 0) WTRC(nb, 5);
                if (ok) ok = mbar_wait(&bars->raw_full[s], (nb / WIDE_RAW_STAGES) & 1, err);
                if (warp == 0) WTRC(nb, 6);
                uint4 hdr = make_uint4(0, 0, 0, 0), qa = hdr, qb = hdr;
                if (ok) {
                    const uint8_t* bp = raw_ring + s * WIDE_RAW_BYTES + row * 144;
                    hdr = *reinterpret_cast<const uint4*>(bp);
                    qa = *reinterpret_cast<const uint4*>(bp + 16 + 32 * g);
                    qb = *reinterpret_cast<const uint4*>(bp + 32 + 32 * g);
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&bars->raw_empty[s]);  // the block sits in registers now
                if (warp == 0) WTRC(nb, 0);
                if (ok && nb >= 2) ok = mbar_wait(&bars->mma_done[as], ((nb >> 1) - 1) & 1, err);
                if (warp == 0) WTRC(nb, 1);
                float d = 0.f, dmin = 0.f;
                if (ok) {
                    tc_fence_after();
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
                    tc_st32(tmem_a0 + as * WIDE_A_COLS + lane_base + 32 * g, r);
                    // K positions 4g .. 4g+3 of the mins step: (m, m) against the (hi, lo) sums of sub-blocks 2g, 2g+1
                    *reinterpret_cast<uint2*>(min_ring + as * WIDE_MIN_BYTES + (g >> 1) * (WM * 16) + row * 16 + (g & 1) * 8) = make_uint2(m0, m1);
                }
                if (warp == 0) WTRC(nb, 2);
                // while the stores to tensor memory are in flight: an earlier block's products are ready by now
                // (its MMAs ran under the dequantisation since)
                if (lag == 1) {
                    if (blk >= 1) drain(nb - 1, d_p1, dmin_p1, acc);
                } else {
                    if (blk >= 2) drain(nb - 2, d_p2, dmin_p2, acc);
                }
                if (warp == 0) WTRC(nb, 3);
                if (ok) {
                    tc_wait_st();
                    tc_fence_before();
                    fence_proxy_async_smem();
                }
                __syncwarp();
                if (warp == 0) WTRC(nb, 4);
                if (warp == 15) WTRC(nb, 13);
                if (warp == 6) WTRC(nb, 14);
                if (lane == 0 && ok) mbar_arrive(&bars->a_full[as]);
                d_p2 = d_p1, dmin_p2 = dmin_p1;
                d_p1 = d, dmin_p1 = dmin;
            }
            // the item's last block(s)
            if (lag == 2 && nblk >= 2) drain(nb - 2, d_p2, dmin_p2, acc);
            if (nblk >= 1) drain(nb - 1, d_p1, dmin_p1, acc);
            const int64_t orow = (int64_t)tile * WM + row;
            if (ks < 0) {
                if (ok) {
#pragma unroll
                    for (int i = 0; i < 16 * ROUNDS; i++) {
                        const int n = g * cpw + i;
                        if (i < cpw && n < tokens) {
                            if (y_f32)
                                reinterpret_cast<float*>(y)[(size_t)n * y_stride + orow] = acc[i];
                            else
                                reinterpret_cast<__half*>(y)[(size_t)n * y_stride + orow] = __float2half_rn(acc[i]);
                        }
                    }
                }
            } else {
                // a run of a cut tile: leave the partial sums, take a ticket; whoever holds the last one adds the runs in
                // run order (so the result does not depend on who that is) and puts the counter back to zero
                uint32_t* tickets = reinterpret_cast<uint32_t*>(part);
                float* pdata = part + 1024;
                const int64_t trow = orow - (int64_t)n_whole * WM;
#pragma unroll
                for (int i = 0; i < 16 * ROUNDS; i++) {
                    const int n = g * cpw + i;
                    if (i < cpw && n < tokens) pdata[((size_t)ks * tokens + n) * tail_rows + trow] = ok ? acc[i] : 0.f;
                }
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(WIDE_DEQ_WARPS * 32) : "memory");
                if (threadIdx.x == 0) {
                    const uint32_t t = atomicAdd(&tickets[tile - n_whole], 1u);
                    if (t == (uint32_t)ksplit - 1) tickets[tile - n_whole] = 0;
                    bars->ticket = t;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(WIDE_DEQ_WARPS * 32) : "memory");
                if (bars->ticket == (uint32_t)ksplit - 1) {
                    __threadfence();
                    // run by run, every column of the run loaded before the adds: the loads of a run are in flight together
#pragma unroll
                    for (int i = 0; i < 16 * ROUNDS; i++) acc[i] = 0.f;
                    for (int k = 0; k < ksplit; k++) {
                        float v[16 * ROUNDS];
#pragma unroll
                        for (int i = 0; i < 16 * ROUNDS; i++) {
                            const int n = g * cpw + i;
                            v[i] = (i < cpw && n < tokens) ? __ldcg(&pdata[((size_t)k * tokens + n) * tail_rows + trow]) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 16 * ROUNDS; i++) acc[i] += v[i];
                    }
#pragma unroll
                    for (int i = 0; i < 16 * ROUNDS; i++) {
                        const int n = g * cpw + i;
                        if (i < cpw && n < tokens) {
                            if (y_f32)
                                reinterpret_cast<float*>(y)[(size_t)n * y_stride + orow] = acc[i];
                            else
                                reinterpret_cast<__half*>(y)[(size_t)n * y_stride + orow] = __float2half_rn(acc[i]);
                        }
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(WIDE_DEQ_WARPS * 32) : "memory");  // the ticket word is reused by the next cut tile
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

}  // namespace

bool gemm_wide_supported(int qtype, int64_t rows, int64_t cols, int tokens) {
    return qtype == TSB_Q4_K && rows % WM == 0 && cols % 256 == 0 && tokens >= 1;
}

// How a matrix's 128-row tiles are dealt to the CTAs: whole tiles while they fill complete waves, the rest cut into
// `ksplit` runs of blocks.  ksplit minimises the longest CTA's time in units of one block (18 KB of weights): a run
// of a cut tile also writes its 128 x n_pad partial sums and the tile's last run reads them all back, which at 128
// token rows costs as much as seven blocks, plus one block's worth of fixed work.  The plan must not depend on the
// token count - the order in which a row's sums are added, and so its bits, would change with its batch mates - so
// the cost is taken at 96 token rows whatever the pass carries.
struct WidePlan {
    int n_whole, ksplit;
    int64_t tail_rows;
};
static WidePlan wide_plan(int sm_count, int64_t rows, int units) {
    constexpr int n_pad = 96;
    const int tiles = (int)(rows / WM), grid = sm_count;
    WidePlan p;
    p.n_whole = tiles / grid * grid;
    const int tail = tiles - p.n_whole;
    p.ksplit = 1;
    p.tail_rows = (int64_t)tail * WM;
    if (tail == 0) return p;
    const float per_run = 1.f + (float)n_pad / 18.f;
    float best = (float)((tail + grid - 1) / grid) * (float)units;
    for (int k = 2; k <= units && k <= 16; k++) {
        const int upk = (units + k - 1) / k;
        const float load = (float)((tail * k + grid - 1) / grid) * ((float)upk + per_run);
        if (load < best - 1e-3f) best = load, p.ksplit = k;
    }
    if (const char* env = getenv("TSB_WIDE_KSPLIT")) p.ksplit = std::max(1, std::min(units, atoi(env)));  // experiments
    const int upk = (units + p.ksplit - 1) / p.ksplit;
    p.ksplit = (units + upk - 1) / upk;  // no empty runs: every run of a tile takes a ticket
    return p;
}
// the operand copy of every pass of a call with `tokens` token rows
size_t gemm_wide_workspace_bytes(int64_t cols, int tokens) {
    const int passes = (tokens + WIDE_NMAX - 1) / WIDE_NMAX;
    return (size_t)(passes < 1 ? 1 : passes) * (size_t)(cols / 256) * WIDE_CHUNKS * WIDE_NMAX * 16;
}
size_t gemm_wide_partial_bytes_for(int sm_count, int64_t rows, int64_t cols) {
    const WidePlan p = wide_plan(sm_count, rows, (int)(cols / 256));
    return p.ksplit > 1 ? 4096 + (size_t)p.ksplit * WIDE_NMAX * p.tail_rows * sizeof(float) : 0;
}
size_t gemm_wide_partial_bytes(const tsb_ctx* ctx, int64_t rows, int64_t cols) {
    return gemm_wide_partial_bytes_for(ctx->sm_count, rows, cols);
}

static size_t wide_smem_bytes(int n_pad) {
    const size_t b_stages = n_pad <= WIDE_NDUAL ? 3 : 2;
    return 1024 + (size_t)WIDE_RAW_STAGES * WIDE_RAW_BYTES + 2 * WIDE_MIN_BYTES + b_stages * WIDE_CHUNKS * (size_t)n_pad * 16;
}

// The tensor map of a weight matrix: 2-D over 32-bit words, [rows][units * 36], box 128 rows x 36 words (one block).
// Encoding goes through the driver entry point (no link against libcuda); maps are kept per (address, shape).
static cudaError_t wide_weight_map(const uint8_t* w, int64_t rows, int units, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static EncodeFn encode = nullptr;
    struct Key {
        const void* p;
        int64_t rows;
        int units;
        bool operator<(const Key& o) const { return p != o.p ? p < o.p : rows != o.rows ? rows < o.rows : units < o.units; }
    };
    static std::map<Key, CUtensorMap> cache;
    std::lock_guard<std::mutex> lock(mu);
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const Key key{w, rows, units};
    auto it = cache.find(key);
    if (it == cache.end()) {
        if (cache.size() > 8192) cache.clear();
        CUtensorMap m;
        const cuuint64_t gdim[2] = {(cuuint64_t)units * 36, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)units * 144};
        const cuuint32_t box[2] = {36, (cuuint32_t)WM};
        const cuuint32_t estride[2] = {1, 1};
        if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(w), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return cudaSuccess;
}

#ifdef TSB_WIDE_TRACE
extern "C" __attribute__((visibility("default"))) void tsb_debug_set_wide_trace(void* p) {
    unsigned long long* q = static_cast<unsigned long long*>(p);
    cudaMemcpyToSymbol(g_wide_trace, &q, sizeof(q));
}
#endif

cudaError_t launch_gemm_wide_q4k(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int64_t cols, const __half* x,
                                 int64_t x_stride, int tokens, void* y, int64_t y_stride, bool y_f32, void* workspace, void* partials) {
    const int units = (int)(cols / 256);
    static SmemOptIn configured1, configured2;
    const size_t smem_max = std::max(wide_smem_bytes(WIDE_NDUAL), wide_smem_bytes(WIDE_NMAX));
    if (cudaError_t e = tsb_opt_in_smem(ctx, gemm_wide_q4k_kernel<1>, smem_max, configured1); e != cudaSuccess) return e;
    if (cudaError_t e = tsb_opt_in_smem(ctx, gemm_wide_q4k_kernel<2>, smem_max, configured2); e != cudaSuccess) return e;
    CUtensorMap wmap;
    if (cudaError_t e = wide_weight_map(w, rows, units, &wmap); e != cudaSuccess) return e;
    // token rows go through in equal passes of at most WIDE_NMAX; one launch lays out the operand of every pass
    const int passes = (tokens + WIDE_NMAX - 1) / WIDE_NMAX;
    const int per_pass = ((tokens + passes - 1) / passes + 15) / 16 * 16;
    const size_t pass_chunks = (size_t)units * WIDE_CHUNKS * per_pass;
    uint4* xw_all = static_cast<uint4*>(workspace);
    if (!workspace)
        if (cudaError_t e = cudaMallocAsync((void**)&xw_all, pass_chunks * passes * 16, st); e != cudaSuccess) return e;
    cudaError_t e = tsb_launch(ctx, wide_prepare_kernel, dim3((unsigned)units, (unsigned)(passes * (per_pass >> 3))), dim3(256), 0, st, true, x,
                               x_stride, tokens, per_pass, units, xw_all);
    for (int t0 = 0, pass = 0; t0 < tokens && e == cudaSuccess; t0 += per_pass, pass++) {
        const int nt = min(per_pass, tokens - t0);
        const int n_pad = (nt + 15) / 16 * 16;
        const uint4* xw = xw_all + pass * pass_chunks;
        const WidePlan plan = wide_plan(ctx->sm_count, rows, units);
        const int ksplit = plan.ksplit;
        if (e == cudaSuccess) {
            // one CTA per SM: the kernel wants the whole tensor memory and most of the shared memory
            const size_t smem = wide_smem_bytes(n_pad);
            const int n_items = plan.n_whole + ((int)(rows / WM) - plan.n_whole) * ksplit;
            dim3 grid((unsigned)min(n_items, ctx->sm_count));
            uint8_t* yp = static_cast<uint8_t*>(y) + (size_t)t0 * y_stride * (y_f32 ? 4 : 2);
            float* part = static_cast<float*>(partials);
            if (ksplit > 1 && !part) {
                e = cudaMallocAsync((void**)&part, 4096 + (size_t)ksplit * nt * plan.tail_rows * sizeof(float), st);
                if (e == cudaSuccess) e = cudaMemsetAsync(part, 0, 4096, st);  // the ticket words start at zero
            }
            if (e == cudaSuccess) {
                if (n_pad <= 64)
                    e = tsb_launch(ctx, gemm_wide_q4k_kernel<1>, grid, dim3(WIDE_THREADS), smem, st, true, wmap, rows, units, (const uint4*)xw,
                                   n_pad, nt, (void*)yp, y_stride, (int)(y_f32 ? 1 : 0), plan.n_whole, ksplit, part, ctx->dev_error);
                else
                    e = tsb_launch(ctx, gemm_wide_q4k_kernel<2>, grid, dim3(WIDE_THREADS), smem, st, true, wmap, rows, units, (const uint4*)xw,
                                   n_pad, nt, (void*)yp, y_stride, (int)(y_f32 ? 1 : 0), plan.n_whole, ksplit, part, ctx->dev_error);
            }
            if (ksplit > 1 && !partials && part) cudaFreeAsync(part, st);
        }
    }
    if (!workspace) cudaFreeAsync(xw_all, st);
    return e;
}
