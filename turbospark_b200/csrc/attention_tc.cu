// Split-KV attention for passes with many queries per (stream, kv head) - a speculative tree's 65 rows x the head
// group, or a prefill chunk - on the fifth-generation tensor cores.  head_dim 128.
//
// A CTA owns one (stream, kv head, 128-query tile, KV chunk) and walks the chunk in 128-token tiles (one
// tcgen05.mma costs about a hundred cycles however narrow it is: 94 with both operands in shared memory and N <= 128,
// 111 with A in tensor memory, 128 = the full rate only at N = 256 - so the tiles are as wide as tensor memory allows):
//   warps 0-7  two softmax warpgroups.  Thread t of group w is query t of the tile - it owns lane t of tensor memory -
//              and takes tokens 64 w .. 64 w + 63 of every tile: it reads its half row of S = Q K^T (tcgen05.ld),
//              applies the tree mask, meets the other group's half-row maximum through shared memory, and writes
//              P = 2^(S * scale - m) as f16 back to tensor memory over the tile's scores, the A operand of the second
//              product.  O stays in tensor memory and the tensor core accumulates into it; m is a reference, not the
//              exact maximum: it moves only when a tile's maximum exceeds it by more than 8 (P then stays below 2^8,
//              far inside f16), and only then the groups rescale O in place, 64 columns each (tcgen05.ld, multiply,
//              tcgen05.st)
//   warp 8     loader: one thread issues tensor copies (cp.async.bulk.tensor, a 2-D map over the whole K/V pool) of the
//              tile's K and V rows, page by page, into the 128-byte-swizzled operand layout (rows of 128 bytes = 64
//              columns, two column blocks per tile), which serves K as a K-major B operand (N = tokens, K = head_dim)
//              and V as an MN-major one (N = head_dim, K = tokens).  (16-byte cp.async copies from two warps took
//              1.4 us per tile to issue and were the bottleneck; without the swizzle the tensor core fetched its
//              operands at about a third of the rate.)
//   warp 9     one thread issues tcgen05.mma: S(i) = Q K_i^T (both operands in shared memory, 8 steps of K = 16) into
//              score accumulator i & 1 (128 columns), and O += P V_i (A from tensor memory, 8 steps) into the 128-column
//              output accumulator; S(i+2) is issued right behind (P V)(i), so the tensor pipe works on the next
//              tile's scores while the softmax warps are busy with this one's
// Every CTA leaves one partial (m, l, O[128]) per query in memory, in the layout of the few-query kernel, and the same
// merge launch finishes the rows.  All waits are bounded; a wait that runs
// out marks the launch failed, the roles leave their loops, tensor memory is freed and the kernel returns.
//
// Masking as in the few-query kernel: positions below the row's `base` are the committed prefix; position base + j is
// in-flight slot j, visible iff bit j of the row's 128-bit mask is set.
#include <cuda.h>

#include <map>
#include <mutex>

#include "attention.cuh"
#include "tc05.cuh"

namespace {

constexpr int TC_HD = 128;
constexpr int TC_QM = 128;      // queries per CTA (UMMA M)
constexpr int TC_TN = 128;      // tokens per tile
constexpr int TC_STAGES = 3;    // K/V tiles in flight
constexpr int TC_SOFTMAX_WARPS = 8, TC_LOAD_WARPS = 1;  // two softmax warpgroups; one thread of the loader warp issues the tensor copies
constexpr int TC_THREADS = (TC_SOFTMAX_WARPS + TC_LOAD_WARPS + 1) * 32;
constexpr int TC_Q_BYTES = TC_QM * TC_HD * 2;
constexpr int TC_TILE_BYTES = TC_TN * TC_HD * 2;  // K or V of one tile
constexpr int TC_STAGE_BYTES = 2 * TC_TILE_BYTES;
constexpr int TC_HEADER_BYTES = 3072;  // barriers, then (at 1024) the row maxima the two softmax warpgroups exchange
constexpr int TC_SMEM_BYTES = TC_HEADER_BYTES + TC_Q_BYTES + TC_STAGES * TC_STAGE_BYTES;  // 227 KB: all there is
constexpr int TC_MAX_SPLITS = 64;  // KV chunks = shares per query
// tensor-memory columns: two score accumulators of 128 columns (P, 128 f16 = 64 columns, is written over the first half
// of a tile's scores once they are in registers) and the output accumulator (128 columns)
constexpr uint32_t TC_COL_S = 0, TC_COL_PV = 256, TC_TMEM_COLS = 512;

#ifdef TSB_ATTN_TC_TRACE
// development builds: nanosecond stamps of CTA (0, 0, 0), eight per tile for the first 64 tiles
__device__ unsigned long long g_tc_trace[64 * 8];
#define TTRC(t, i) do { if (trace_on && (t) < 64) g_tc_trace[(t) * 8 + (i)] = global_timer_ns(); } while (0)
#else
#define TTRC(t, i)
#endif

struct TcBars {
    uint64_t kv_full[TC_STAGES], kv_empty[TC_STAGES];
    uint64_t s_full[2], p_full[2], mx_full[2];
    uint64_t pv_full, fin_full;
    uint32_t tmem_base, failed;
};

// One box of the K/V pool - 64 columns (128 bytes) x box_rows token rows - lands 128-byte-swizzled, row after row.
__device__ __forceinline__ void tc_tensor_g2s_2d(uint32_t dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2_tc(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// Byte offset of 16-byte chunk c (0..15) of row r in a 128-byte-swizzled tile of `rows` rows x 128 f16: two column
// blocks of 64 elements, `rows` * 128 bytes apart; inside a block a row is 128 bytes and its eight chunks are XORed with
// the row index mod 8 (the hardware's SWIZZLE_128B pattern; the tile starts on a 1024-byte boundary).  The same bytes
// serve as a K-major operand (rows = M or N, 64 K elements per block: Q and K) and as an MN-major one (rows = K,
// 64 N elements per block: V).
__device__ __forceinline__ uint32_t sw128_off(int r, int c, int rows) {
    return (uint32_t)((c >> 3) * (rows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

__global__ void __launch_bounds__(TC_THREADS, 1)
    attn_tc_partial_kernel(const __grid_constant__ CUtensorMap kvmap, int box_rows, KvView kv, int layer, const __half* __restrict__ q,
                           int64_t q_stride, const tsb_row_desc* __restrict__ rows, int rows_per_seq, int n_q_heads, float scale_log2e, int chunk, float* __restrict__ part_o,
                           float2* __restrict__ part_ml, uint32_t* __restrict__ err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    TcBars* bars = reinterpret_cast<TcBars*>(smem);
    float* xbuf = reinterpret_cast<float*>(smem + 1024);  // [2 tiles in turn][2 warpgroups][128 queries]
    uint8_t* q_tile = smem + TC_HEADER_BYTES;
    uint8_t* ring = q_tile + TC_Q_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = n_q_heads / kv.kv_heads;
    const int n_queries = rows_per_seq * G;
    const int n_qtiles = (n_queries + TC_QM - 1) / TC_QM;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / n_qtiles, qtile = blockIdx.y % n_qtiles;
    const int row_first = blockIdx.z * rows_per_seq;
#ifdef TSB_ATTN_TC_TRACE
    const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0;
#endif

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_STAGES; i++) mbar_init(&bars->kv_full[i], 1), mbar_init(&bars->kv_empty[i], 1);
        for (int i = 0; i < 2; i++) mbar_init(&bars->s_full[i], 1), mbar_init(&bars->p_full[i], TC_SOFTMAX_WARPS), mbar_init(&bars->mx_full[i], TC_SOFTMAX_WARPS);
        mbar_init(&bars->pv_full, 1), mbar_init(&bars->fin_full, TC_SOFTMAX_WARPS);
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == TC_SOFTMAX_WARPS + TC_LOAD_WARPS) {  // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the row descriptors and the page table were written before the pass began
    const tsb_row_desc rd0 = rows[row_first];
    const int seq = rd0.seq, base = rd0.base;
    const bool seq_ok = seq >= 0 && seq < kv.max_seqs;
    const int L = base + rows_per_seq;
    const int t_begin = split * chunk;
    const int t_end = min(L, t_begin + chunk);
    const int n_tiles = (seq_ok && t_end > t_begin) ? (t_end - t_begin + TC_TN - 1) / TC_TN : 0;
    if (!seq_ok && threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);

    pdl_wait();  // q, and the K/V rows of this pass, come from the preceding kernel

    // ---- the query tile, K-major, 128-byte swizzle: row = query of the tile, 16 chunks of 8 columns
    for (int i = threadIdx.x; i < TC_QM * 16; i += TC_THREADS) {
        const int ql = i >> 4, c = i & 15;
        const int qi = qtile * TC_QM + ql;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qi < n_queries)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(row_first + qi / G) * q_stride + (size_t)(kvh * G + qi % G) * TC_HD + c * 8);
        *reinterpret_cast<uint4*>(q_tile + sw128_off(ql, c, TC_QM)) = v;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp >= TC_SOFTMAX_WARPS && warp < TC_SOFTMAX_WARPS + TC_LOAD_WARPS) {
        // ---- loader: one thread issues the tensor copies of a tile - per box_rows token rows (a page, or 128 rows of a
        // larger page) and per 64-column block one copy for K and one for V - all counted on the stage's barrier.
        // Rows past the end of the stream are masked later; a part that lies wholly past the end is read from the
        // page of the stream's last position, so that no stale shared memory meets the tensor core.
        if (lane == 0) {
            bool ok = true;
            const int64_t rows_per_plane = (int64_t)kv.num_pages * kv.page_tokens;  // token rows of one layer's K (or V)
            for (int tile = 0; tile < n_tiles && ok; tile++) {
                const int st = tile % TC_STAGES;
                if (tile >= TC_STAGES) ok = mbar_wait(&bars->kv_empty[st], ((tile / TC_STAGES) - 1) & 1, err);
                if (!ok) break;
                TTRC(tile, 7);
                const uint32_t kdst = smem_u32(ring + st * TC_STAGE_BYTES), vdst = kdst + TC_TILE_BYTES;
                mbar_expect_tx(&bars->kv_full[st], (uint32_t)TC_STAGE_BYTES);
                for (int part = 0; part * box_rows < TC_TN; part++) {
                    int pos = t_begin + tile * TC_TN + part * box_rows;
                    if (pos >= t_end) pos = (t_end - 1) & ~(box_rows - 1);
                    const int lp = pos >> kv.page_shift;
                    int page = lp < kv.max_pages_per_seq ? kv.page_table[(size_t)seq * kv.max_pages_per_seq + lp] : -1;
                    if (page < 0) {  // not a reserved position: flagged; the copy reads page 0 so that the byte count stays whole
                        atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
                        page = 0;
                    }
                    const int64_t row_k = (int64_t)(2 * layer) * rows_per_plane + (int64_t)page * kv.page_tokens + (pos & (kv.page_tokens - 1));
                    const int64_t row_v = row_k + rows_per_plane;
                    const uint32_t off = (uint32_t)(part * box_rows * 128);
#pragma unroll
                    for (int b = 0; b < 2; b++) {
                        tc_tensor_g2s_2d(kdst + b * (TC_TN * 128) + off, &kvmap, kvh * TC_HD + b * 64, (int)row_k, &bars->kv_full[st]);
                        tc_tensor_g2s_2d(vdst + b * (TC_TN * 128) + off, &kvmap, kvh * TC_HD + b * 64, (int)row_v, &bars->kv_full[st]);
                    }
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (warp == TC_SOFTMAX_WARPS + TC_LOAD_WARPS) {
        // ---- MMA issue: the warp walks the tiles together, lane 0 issues
        const uint32_t leader = lane == 0 ? 1u : 0u;
        // instruction descriptors: f32 accumulate, f16 A and B, M = 128; scores N = 128 tokens, both operands K-major;
        // P V N = 128 columns with B (V) MN-major
        const uint32_t idesc_s = (1u << 4) | ((uint32_t)(TC_TN >> 3) << 17) | ((uint32_t)(TC_QM >> 4) << 24);
        const uint32_t idesc_pv = (1u << 4) | (1u << 16) | ((uint32_t)(TC_HD >> 3) << 17) | ((uint32_t)(TC_QM >> 4) << 24);
        // shared-memory matrix descriptors without the start address (version 1, 128-byte swizzle).  K-major (Q, K):
        // eight-row groups 1024 bytes apart (stride byte offset), the leading offset is not used; a K = 16 step moves
        // the start address by 32 bytes inside the 64-element block, the second block starts rows * 128 bytes later.
        // MN-major (V): eight-token groups 1024 bytes apart (stride), the two 64-column blocks a block's size apart (leading)
        constexpr uint64_t SW128 = 2ull << 61;
        const uint64_t desc_kmaj = ((uint64_t)1u << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | SW128;
        const uint64_t desc_mnmaj = ((uint64_t)((uint32_t)(TC_TN * 128) >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | SW128;
        const uint64_t desc_q = desc_kmaj | (uint64_t)((smem_u32(q_tile) >> 4) & 0x3FFFu);
        bool ok = true;
        auto scores = [&](int t) {  // S(t) into accumulator t & 1
            const int st = t % TC_STAGES;
            ok = mbar_wait(&bars->kv_full[st], (t / TC_STAGES) & 1, err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            tc_fence_after();
            const uint64_t desc_k = desc_kmaj | (uint64_t)((smem_u32(ring + st * TC_STAGE_BYTES) >> 4) & 0x3FFFu);
            const uint32_t d = tmem + TC_COL_S + (uint32_t)(t & 1) * TC_TN;
            tc_mma_ss<false>(leader, d, desc_q, desc_k, idesc_s);
#pragma unroll
            for (int ks = 1; ks < TC_HD / 16; ks++) {  // address units of 16 bytes: 32 bytes per step, a block per four steps
                const uint32_t in_block = (uint32_t)(ks & 3) * 2u;
                tc_mma_ss<true>(leader, d, desc_q + (uint64_t)((uint32_t)(ks >> 2) * (TC_QM * 128 / 16) + in_block),
                                desc_k + (uint64_t)((uint32_t)(ks >> 2) * (TC_TN * 128 / 16) + in_block), idesc_s);
            }
            tc_commit_if(leader, &bars->s_full[t & 1]);
        };
        if (n_tiles > 0) scores(0);
        if (ok && n_tiles > 1) scores(1);
        for (int t = 0; t < n_tiles && ok; t++) {
            const int st = t % TC_STAGES;
            ok = mbar_wait(&bars->p_full[t & 1], (t >> 1) & 1, err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            TTRC(t, 1);
            tc_fence_after();
            const uint64_t desc_v = desc_mnmaj | (uint64_t)((smem_u32(ring + st * TC_STAGE_BYTES + TC_TILE_BYTES) >> 4) & 0x3FFFu);
            const uint32_t d = tmem + TC_COL_PV;
            const uint32_t a = tmem + TC_COL_S + (uint32_t)(t & 1) * TC_TN;  // P sits where the tile's scores were
            if (t == 0) tc_mma_ts<false>(leader, d, a, desc_v, idesc_pv);  // the first tile starts the output
            else tc_mma_ts<true>(leader, d, a, desc_v, idesc_pv);
#pragma unroll
            for (int kt = 1; kt < TC_TN / 16; kt++)  // sixteen tokens per step: two 1024-byte token groups = 128 address units
                tc_mma_ts<true>(leader, d, a + 8 * kt, desc_v + (uint64_t)(128 * kt), idesc_pv);
            tc_commit_if(leader, &bars->pv_full);
            tc_commit_if(leader, &bars->kv_empty[st]);
            TTRC(t, 0);
            if (t + 2 < n_tiles) scores(t + 2);
            TTRC(t, 2);
        }
        if (!ok && lane == 0) bars->failed = 1;
    } else {
        // ---- softmax warpgroups: thread = (query ql of the tile = tensor-memory lane ql, half wg of every tile's 128 tokens).
        // A failed wait does not leave the loop: the other group's barriers still get their arrivals, nobody is left waiting.
        const int wg = warp >> 2;
        const int ql = threadIdx.x & (TC_QM - 1);
        const int qi = qtile * TC_QM + ql;
        const bool valid = qi < n_queries;
        const int row = valid ? qi / G : 0, head = kvh * G + (valid ? qi % G : 0);
        uint64_t mask[2] = {0, 0};
        if (valid) mask[0] = rows[row_first + row].mask[0], mask[1] = rows[row_first + row].mask[1];
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t col_o = tmem + lane_base + TC_COL_PV + (uint32_t)wg * (TC_HD / 2);  // this group's half of the output columns
        float m_ref = -INFINITY, l_run = 0.f;  // l_run: over this group's tokens only
        bool ok = true;
        for (int t = 0; t < n_tiles; t++) {
            const int buf = t & 1;
            const uint32_t c = (uint32_t)(t >> 1);  // completion index on the barriers of buffer `buf`
            const uint32_t col_s = tmem + lane_base + TC_COL_S + (uint32_t)buf * TC_TN;
            if ((warp & 3) == 0) TTRC(t, 3 + wg);
            if (ok) ok = mbar_wait(&bars->s_full[buf], c & 1u, err);
            tc_fence_after();
            // this group's 64 scores of the row
            float s[64];
            {
                uint32_t r0[16], r1[16], r2[16], r3[16];
                tc_ld16(col_s + 64 * wg, r0);
                tc_ld16(col_s + 64 * wg + 16, r1);
                tc_ld16(col_s + 64 * wg + 32, r2);
                tc_ld16(col_s + 64 * wg + 48, r3);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    s[i] = __uint_as_float(r0[i]);
                    s[16 + i] = __uint_as_float(r1[i]);
                    s[32 + i] = __uint_as_float(r2[i]);
                    s[48 + i] = __uint_as_float(r3[i]);
                }
            }
            const int pos0 = t_begin + t * TC_TN + 64 * wg;
            if (pos0 + 64 > base) {  // the half tile reaches in-flight slots (or the end of the stream): mask
#pragma unroll
                for (int j2 = 0; j2 < 64; j2++) {
                    const int j = pos0 + j2 - base;
                    bool vis = j < 0;
                    if (j >= 0 && j < 128) vis = (mask[j >> 6] >> (j & 63)) & 1ull;
                    if (!vis) s[j2] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j2 = 0; j2 < 64; j2 += 4) {
                mx4[0] = fmaxf(mx4[0], s[j2]), mx4[1] = fmaxf(mx4[1], s[j2 + 1]);
                mx4[2] = fmaxf(mx4[2], s[j2 + 2]), mx4[3] = fmaxf(mx4[3], s[j2 + 3]);
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the row's maximum over the whole tile: the two groups exchange their halves' maxima.  Arriving also says
            // that this warp has its scores in registers, so the other group may write P over them.
            xbuf[(buf * 2 + wg) * TC_QM + ql] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->mx_full[buf]);
            if (ok) ok = mbar_wait(&bars->mx_full[buf], c & 1u, err);
            mx = fmaxf(mx, xbuf[(buf * 2 + (wg ^ 1)) * TC_QM + ql]) * scale_log2e;  // the scale is positive
            if ((warp & 3) == 0 && wg == 0) TTRC(t, 5);
            // the reference moves only when the tile's maximum is more than 8 above it (or it was -inf); both groups
            // take the same decision from the same numbers
            const bool grow = mx > m_ref + 8.f;
            const float m_new = grow ? mx : m_ref;
            const float alpha = grow ? exp2f(m_ref - m_new) : 1.f;  // 0 when nothing was visible before
            const bool rescale = grow && m_ref != -INFINITY;
            if (__any_sync(0xffffffffu, rescale)) {
                // the output so far is rescaled in place, this group's 64 columns of it: the previous tile's product
                // has to be complete first (completion t - 1 of the barrier; nothing newer can have completed yet)
                if (ok && t > 0) ok = mbar_wait(&bars->pv_full, (uint32_t)(t - 1) & 1u, err);
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < TC_HD / 2; c0 += 32) {
                    uint32_t a16[16], b16[16], w32[32];
                    tc_ld16(col_o + c0, a16);
                    tc_ld16(col_o + c0 + 16, b16);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        w32[i] = __float_as_uint(__uint_as_float(a16[i]) * alpha);
                        w32[16 + i] = __float_as_uint(__uint_as_float(b16[i]) * alpha);
                    }
                    tc_st32(col_o + c0, w32);
                }
            }
            // P = 2^(S * scale - m) as f16 pairs: this group's 64 tokens are columns 32 wg .. 32 wg + 31 of the buffer
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int j2 = 0; j2 < 64; j2 += 4) {
                const float p0 = ex2_approx(fmaf(s[j2], scale_log2e, -m_use)), p1 = ex2_approx(fmaf(s[j2 + 1], scale_log2e, -m_use));
                const float p2 = ex2_approx(fmaf(s[j2 + 2], scale_log2e, -m_use)), p3 = ex2_approx(fmaf(s[j2 + 3], scale_log2e, -m_use));
                rs4[0] += p0, rs4[1] += p1, rs4[2] += p2, rs4[3] += p3;
                pk[j2 >> 1] = pack_half2_tc(p0, p1);
                pk[(j2 >> 1) + 1] = pack_half2_tc(p2, p3);
            }
            l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            m_ref = m_new;
            tc_st32(col_s + 32 * wg, pk);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if ((warp & 3) == 0 && wg == 0) TTRC(t, 6);
            if (lane == 0) mbar_arrive(&bars->p_full[buf]);
        }
        // the last product, the other group's share of the row sum, then the query's share: (m, l, O)
        if (ok && n_tiles > 0) ok = mbar_wait(&bars->pv_full, (uint32_t)(n_tiles - 1) & 1u, err);
        tc_fence_after();
        xbuf[wg * TC_QM + ql] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->fin_full);
        if (ok) ok = mbar_wait(&bars->fin_full, 0u, err);
        const float l_all = l_run + xbuf[(wg ^ 1) * TC_QM + ql];
        if (!ok) bars->failed = 1;
        pdl_launch_dependents();
        const size_t pi = ((size_t)(row_first + row) * n_q_heads + head) * gridDim.x + blockIdx.x;
        float4* po = reinterpret_cast<float4*>(part_o + pi * TC_HD + wg * (TC_HD / 2));
        if (ok && n_tiles > 0) {
#pragma unroll
            for (int c0 = 0; c0 < TC_HD / 2; c0 += 32) {
                uint32_t a16[16], b16[16];
                tc_ld16(col_o + c0, a16);
                tc_ld16(col_o + c0 + 16, b16);
                tc_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        po[(c0 >> 2) + i] = make_float4(__uint_as_float(a16[4 * i]), __uint_as_float(a16[4 * i + 1]), __uint_as_float(a16[4 * i + 2]),
                                                        __uint_as_float(a16[4 * i + 3]));
                        po[(c0 >> 2) + 4 + i] = make_float4(__uint_as_float(b16[4 * i]), __uint_as_float(b16[4 * i + 1]),
                                                            __uint_as_float(b16[4 * i + 2]), __uint_as_float(b16[4 * i + 3]));
                    }
                }
            }
            if (valid && wg == 0) part_ml[pi] = make_float2(m_ref, l_all);
        } else if (ok && valid) {  // no tile in this chunk: an empty share
#pragma unroll
            for (int i = 0; i < TC_HD / 8; i++) po[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (wg == 0) part_ml[pi] = make_float2(-INFINITY, 0.f);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_SOFTMAX_WARPS + TC_LOAD_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// How the context is cut: one CTA per SM at a time (a CTA holds 225 KB of shared memory and all of tensor memory).
// Fewer CTAs than SMs: as many chunks per (stream, kv head, query tile) as fill the device.  More: the cut whose waves
// come out most even (a CTA costs its tiles plus about three tiles' time of fixed work).  Planned for the length rounded
// up to 512, so the cut does not move with every row.
struct TcPlan {
    int n_qtiles, groups, n_splits, chunk;
};
TcPlan attn_tc_plan(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads, int max_len) {
    TcPlan p;
    const int G = n_q_heads / kv->view.kv_heads;
    p.n_qtiles = (rows_per_seq * G + TC_QM - 1) / TC_QM;
    p.groups = rows / rows_per_seq;
    const int planned = max_len > 0 ? (max_len + 511) / 512 * 512 : 512;
    const int tiles_total = planned / TC_TN;
    const int base_ctas = p.groups * kv->view.kv_heads * p.n_qtiles;
    const int resident = ctx->sm_count > 0 ? ctx->sm_count : 1;
    int splits = resident / (base_ctas > 0 ? base_ctas : 1);
    if (splits < 1) {
        float best = 1e30f;
        for (int s = 1; s <= 8 && s <= tiles_total; s++) {
            const int waves = (base_ctas * s + resident - 1) / resident;
            const float cost = (float)waves * ((float)((tiles_total + s - 1) / s) + 3.f);
            if (cost < best - 1e-3f) best = cost, splits = s;
        }
    }
    if (splits > TC_MAX_SPLITS) splits = TC_MAX_SPLITS;
    if (splits > tiles_total) splits = tiles_total;
    if (splits < 1) splits = 1;
    const int tiles_per = (tiles_total + splits - 1) / splits;
    p.chunk = tiles_per * TC_TN;
    p.n_splits = (tiles_total + tiles_per - 1) / tiles_per;
    return p;
}

// The tensor map of a K/V pool: 2-D over f16, [layers * 2 * pages * page_tokens token rows][kv_heads * head_dim], box
// 64 columns x box_rows rows, 128-byte swizzle.  Encoding goes through the driver entry point (no link against libcuda);
// maps are kept per (pool, shape).
cudaError_t tc_kv_map(const KvView& v, int box_rows, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static EncodeFn encode = nullptr;
    struct Key {
        const void* p;
        int64_t rows;
        int cols, box;
        bool operator<(const Key& o) const {
            return p != o.p ? p < o.p : rows != o.rows ? rows < o.rows : cols != o.cols ? cols < o.cols : box < o.box;
        }
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
    const int cols = v.kv_heads * v.head_dim;
    const int64_t rows = (int64_t)v.layers * 2 * v.num_pages * v.page_tokens;
    const Key key{v.pool, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it == cache.end()) {
        if (cache.size() > 1024) cache.clear();
        CUtensorMap m;
        const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)cols * sizeof(__half)};
        const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
        const cuuint32_t estride[2] = {1, 1};
        if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, v.pool, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return cudaSuccess;
}

}  // namespace

bool attn_tc_applicable(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads) {
    static int enabled = -1, min_queries = 65;  // TSB_ATTN_TC=0 keeps every pass on the mma.sync kernel (experiments)
    if (enabled < 0) {
        const char* env = getenv("TSB_ATTN_TC");
        enabled = env ? (atoi(env) != 0) : 1;
        env = getenv("TSB_ATTN_TC_MINQ");  // queries per (stream, kv head) from which the tensor-memory kernel is taken
        if (env && atoi(env) > 0) min_queries = atoi(env);
    }
    if (!enabled || kv->view.head_dim != TC_HD || kv->view.kv_heads <= 0 || n_q_heads % kv->view.kv_heads != 0) return false;
    // the tensor copies take whole boxes of a page: pages of 8, 16, ... token rows, all rows of the pool within 32-bit coordinates
    const int pt = kv->view.page_tokens;
    if (pt < 8 || (pt & (pt - 1)) != 0 || (int64_t)kv->view.layers * 2 * kv->view.num_pages * pt >= (int64_t)1 << 31) return false;
    if (rows_per_seq * (n_q_heads / kv->view.kv_heads) >= min_queries) return true;
    // few queries per stream but many streams: when streams x kv heads fill the device, a CTA per SM that streams its K/V
    // through tensor copies is the faster one (64 streams x 6 rows at context 4096: 262 vs 316 us per layer); below
    // that the few-query kernel wins, whose smaller CTAs overlap the neighbouring matmuls' prologues
    return rows_per_seq > 0 && (rows / rows_per_seq) * kv->view.kv_heads >= ctx->sm_count;
}

cudaError_t launch_attn_tc_partials(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                    const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int n_q_heads, float scale, int max_len,
                                    void* scratch, const float** part_o_out, const float2** part_ml_out, int* n_splits_out) {
    const TcPlan p = attn_tc_plan(ctx, kv, rows, rows_per_seq, n_q_heads, max_len);
    float* part_o = reinterpret_cast<float*>(scratch);
    float2* part_ml = reinterpret_cast<float2*>(part_o + (size_t)rows * n_q_heads * p.n_splits * TC_HD);
    *part_o_out = part_o, *part_ml_out = part_ml, *n_splits_out = p.n_splits;
    const int box_rows = kv->view.page_tokens < TC_TN ? kv->view.page_tokens : TC_TN;
    CUtensorMap kvmap;
    if (cudaError_t e = tc_kv_map(kv->view, box_rows, &kvmap); e != cudaSuccess) return e;
    static SmemOptIn configured;
    if (cudaError_t e = tsb_opt_in_smem(ctx, attn_tc_partial_kernel, (size_t)TC_SMEM_BYTES, configured); e != cudaSuccess) return e;
    dim3 grid((unsigned)p.n_splits, (unsigned)(kv->view.kv_heads * p.n_qtiles), (unsigned)p.groups);
    return tsb_launch(ctx, attn_tc_partial_kernel, grid, dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, st, true, kvmap, box_rows, kv->view, layer, q, q_stride,
                      rows_dev, rows_per_seq, n_q_heads, scale * 1.4426950408889634f, p.chunk, part_o, part_ml, ctx->dev_error);
}

#ifdef TSB_ATTN_TC_TRACE
extern "C" __attribute__((visibility("default"))) int tsb_debug_get_tc_trace(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_tc_trace, sizeof(unsigned long long) * 64 * 8);
}
#endif
