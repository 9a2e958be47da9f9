// Split-KV ("flash-decoding") attention over the paged fp16 cache for a batch of
// verify rows, with the speculative tree's ancestor mask.
//
// Rows come grouped per stream (rows_per_seq each, ordered by in-flight slot).
// A CTA owns one (stream, kv head, 32-query tile, KV chunk): the queries are the
// stream's rows x the kv head's group of q heads, so every K/V byte is read once
// for the whole group (GQA-shared) and once for all rows of the round.  Inside
// the CTA four warps split the work 2 x 2: two 16-query mma tiles x two halves
// of each 64-token K/V tile.  Scores S = Q K^T and O += P V run on mma.sync
// m16n8k16 (f16 in, f32 accumulate) with K/V staged in shared memory by
// cp.async (three stages), 16-byte-chunk XOR swizzle, fragments pulled with
// ldmatrix.  The online softmax keeps (m, l, O) per query in registers; row max
// and sum are combined across the four lanes of a quad with warp shuffles.
// Each CTA writes one partial (m, l, O[head_dim]) per query; the last CTA of a
// (stream, kv head, query tile) to finish - decided by a ticket counter, nobody
// waits - merges the partials of all chunks with warp shuffles and emits f16
// rows and/or the o_proj matmul's activation operand.
//
// Masking: positions below the row's `base` are the committed prefix (always
// visible); position base + j is in-flight slot j and is visible iff bit j of
// the row's 128-bit mask is set (a chain row m has bits 0..m, a tree row its
// root path).  HBM-bound: bytes = context * kv_heads * head_dim * 2 (K and V) * 2 B per layer.
#include "attention.cuh"
#include <cooperative_groups.h>
#include <mutex>
namespace cg = cooperative_groups;

namespace {

constexpr int ATT_THREADS = 128;
constexpr int TILE_TOKENS = 64;
constexpr int MAX_SPLITS = 64;
constexpr int NST = 3;  // K/V tile stages in shared memory
constexpr int ATTN_MAX_DEVICES = 64;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// byte offset of 16-byte chunk `c` of token row `r` inside a swizzled [64][HD] f16 tile
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}

// MT = query m-tiles per CTA (1 -> 16 queries, 4 warps; 2 -> 32 queries, 8 warps; 4 -> 64 queries, 16 warps).  Whatever MT is, a warp owns one
// m-tile and one 16-token slice of every 64-token tile, so the arithmetic done for a query - the order of its
// running maxima, sums and merges - does not depend on how many other rows are in flight: a row verified in a
// batch of six comes out bit-identical to the same row decoded alone.
// Grid: x = KV chunks (a multiple of the cluster size; the CTAs of a cluster hold consecutive chunks of the same
// queries), y = kv head * query tiles, z = streams.
template <int HD, int MT>
__global__ void __maxnreg__(128)
    attn_partial_kernel(KvView kv, int layer, const __half* __restrict__ q, int64_t q_stride,
                        const tsb_row_desc* __restrict__ rows, int rows_per_seq, int n_q_heads, float scale_log2e,
                        int chunk, int cluster_size, float* __restrict__ part_o, float2* __restrict__ part_ml,
                        uint32_t* __restrict__ tickets, __half* __restrict__ out, ActOut act, uint32_t* __restrict__ err,
                        int defer_merge) {
    constexpr int CH = HD / 8;         // 16-byte chunks per token row
    constexpr int KS = HD / 16;        // k steps of S = Q K^T
    constexpr int NO = HD / 8;         // n tiles of O
    constexpr int QT = 16 * MT;        // queries per CTA
    constexpr int NTHR = ATT_THREADS * MT;
    constexpr int SL = 4;              // token slices of a tile (one per warp of an m-tile)
    constexpr int WTOK = TILE_TOKENS / SL;  // tokens of a tile one warp covers
    constexpr int NT8 = WTOK / 8, KK = WTOK / 16;
    constexpr int TILE_BYTES = TILE_TOKENS * HD * 2;
    extern __shared__ __align__(128) uint8_t smem[];  // [NST stages][K tile | V tile]; later the warps' partials
    __shared__ int s_last;
    cg::cluster_group cluster = cg::this_cluster();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int mt = warp % MT, sl = warp / MT;
    const int nkv = kv.kv_heads, G = n_q_heads / nkv;
#ifdef TSB_ATTN_TRACE
    unsigned long long* trc = defer_merge && tickets ? reinterpret_cast<unsigned long long*>(tickets) + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 : nullptr;
#define TRC(i) if (trc && threadIdx.x == 0) trc[i] = global_timer_ns()
#else
#define TRC(i)
#endif
    TRC(0);
    const int n_queries = rows_per_seq * G;
    const int n_qtiles = (n_queries + QT - 1) / QT;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / n_qtiles, qtile = blockIdx.y % n_qtiles;
    const int row_first = blockIdx.z * rows_per_seq;

    // The row descriptors and page table were written before the pass began and cache rows below `base` in
    // earlier passes, so they may be touched before the preceding kernel has finished.
    const tsb_row_desc rd0 = rows[row_first];
    const int seq = rd0.seq, base = rd0.base;
    const int L = base + rows_per_seq;
    const int t_begin = split * chunk;
    const int t_end = min(L, t_begin + chunk);
    if (seq < 0 || seq >= kv.max_seqs) {  // the same for every CTA of the cluster: all leave together
        if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_BAD_INDEX);
        return;
    }
    const int n_tiles = t_end > t_begin ? (t_end - t_begin + TILE_TOKENS - 1) / TILE_TOKENS : 0;

    const uint32_t smem_base = smem_u32(smem);
    // a thread copies half a token row (K and V) of every tile: one page-table lookup per thread per tile
    auto issue_tile = [&](int tile, int stage) {
        const int t0 = t_begin + tile * TILE_TOKENS;
        const uint32_t kdst = smem_base + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
        constexpr int TPR = NTHR / TILE_TOKENS;  // threads sharing a token row
        const int r = threadIdx.x / TPR, c0 = (threadIdx.x % TPR) * (CH / TPR);
        const int pos = t0 + r;
        const bool valid = pos < t_end;
        const __half* kr = valid ? kv_row(kv, layer, 0, seq, pos) : nullptr;
        const bool ok = kr != nullptr;
        const __half* ksrc = ok ? kr + (size_t)kvh * HD : kv.pool;
        const __half* vsrc = ok ? ksrc + kv.kv_stride : kv.pool;  // V sits one kv_stride after K in the same layer
#pragma unroll
        for (int i = 0; i < CH / TPR; i++) {
            const int c = c0 + i;
            const uint32_t off = tile_off<HD>(r, c);
            cp_async16_zfill(kdst + off, ok ? (const void*)(ksrc + c * 8) : (const void*)kv.pool, ok);
            cp_async16_zfill(vdst + off, ok ? (const void*)(vsrc + c * 8) : (const void*)kv.pool, ok);
        }
        cp_async_commit();
    };
    auto prologue = [&]() {  // every stage of the ring starts filled
#pragma unroll
        for (int i = 0; i < NST; i++) {
            if (i < n_tiles) issue_tile(i, i);
            else cp_async_commit();
        }
    };
    // tiles made only of committed rows can start moving while the kernel that produces q is still running
    const bool early = t_begin + NST * TILE_TOKENS <= base;
    if (early) prologue();
    TRC(1);
    pdl_wait();
    TRC(2);
    if (!early) prologue();

    // ---- this lane's two queries (rows gid and gid+8 of the warp's mma tile)
    const int q0 = qtile * QT + mt * 16 + gid, q1 = q0 + 8;
    const bool v0 = q0 < n_queries, v1 = q1 < n_queries;
    const int r0 = v0 ? q0 / G : 0, r1 = v1 ? q1 / G : 0;
    const int h0 = kvh * G + (v0 ? q0 % G : 0), h1 = kvh * G + (v1 ? q1 % G : 0);
    uint64_t mask0[2] = {0, 0}, mask1[2] = {0, 0};
    if (v0) mask0[0] = rows[row_first + r0].mask[0], mask0[1] = rows[row_first + r0].mask[1];
    if (v1) mask1[0] = rows[row_first + r1].mask[0], mask1[1] = rows[row_first + r1].mask[1];

    uint32_t qa[KS][4];
    {
        const __half* p0 = q + (size_t)(row_first + r0) * q_stride + (size_t)h0 * HD;
        const __half* p1 = q + (size_t)(row_first + r1) * q_stride + (size_t)h1 * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(p0 + 16 * ks + 2 * tig);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(p1 + 16 * ks + 2 * tig);
            qa[ks][2] = *reinterpret_cast<const uint32_t*>(p0 + 16 * ks + 8 + 2 * tig);
            qa[ks][3] = *reinterpret_cast<const uint32_t*>(p1 + 16 * ks + 8 + 2 * tig);
        }
    }

    float o[NO][4];
#pragma unroll
    for (int n = 0; n < NO; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[n][i] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // NST-deep cp.async ring: a stage is refilled as soon as every warp is done with it
    for (int tile = 0; tile < n_tiles; tile++) {
        const int stage = tile % NST;
        cp_async_wait<NST - 1>();  // all but the NST - 1 youngest groups have landed: tile `tile` is here
        __syncthreads();
        if (tile == 0) { TRC(3); }
        const uint32_t ktile = smem_base + stage * 2 * TILE_BYTES, vtile = ktile + TILE_BYTES;
        const int tok0 = sl * WTOK;  // this warp's tokens of the tile
        const int pos0 = t_begin + tile * TILE_TOKENS + tok0;

        // ---- S = Q K^T for 16 queries x WTOK tokens
        float s[NT8][4];
#pragma unroll
        for (int nt = 0; nt < NT8; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) s[nt][i] = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT8; nt++) {
#pragma unroll
            for (int kp = 0; kp < KS / 2; kp++) {
                uint32_t b[4];
                const int r = tok0 + nt * 8 + (lane & 7);
                const int c = kp * 4 + (lane >> 3);
                ldmatrix_x4(b, ktile + tile_off<HD>(r, c));
                const uint32_t b01[2] = {b[0], b[1]}, b23[2] = {b[2], b[3]};
                mma_16816(s[nt], qa[2 * kp], b01);
                mma_16816(s[nt], qa[2 * kp + 1], b23);
            }
        }
        // ---- scale, mask, online softmax
        const bool need_mask = pos0 + WTOK > base;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NT8; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v = s[nt][i] * scale_log2e;
                if (need_mask) {
                    const int p = pos0 + nt * 8 + 2 * tig + (i & 1);
                    const int j = p - base;
                    bool vis = j < 0;
                    if (j >= 0 && j < 128) {
                        const uint64_t w = (i < 2) ? mask0[j >> 6] : mask1[j >> 6];
                        vis = (w >> (j & 63)) & 1ull;
                    }
                    if (!vis) v = -INFINITY;
                }
                s[nt][i] = v;
                mx[i >> 1] = fmaxf(mx[i >> 1], v);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[h] = exp2f(m_run[h] - m_use[h]);  // 0 when m_run is -inf
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pa[KK][4];
#pragma unroll
        for (int nt = 0; nt < NT8; nt++) {
            const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
            const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_half2(p0, p1);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_half2(p2, p3);
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l_run[h] = l_run[h] * alpha[h] + rs[h];
        }
#pragma unroll
        for (int n = 0; n < NO; n++) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            o[n][2] *= alpha[1];
            o[n][3] *= alpha[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < KK; kk++) {
#pragma unroll
            for (int np = 0; np < NO / 2; np++) {
                uint32_t b[4];
                const int r = tok0 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int c = np * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, vtile + tile_off<HD>(r, c));
                const uint32_t b01[2] = {b[0], b[1]}, b23[2] = {b[2], b[3]};
                mma_16816(o[2 * np], pa[kk], b01);
                mma_16816(o[2 * np + 1], pa[kk], b23);
            }
        }
        __syncthreads();  // a stage is rewritten only after every warp is done with it
        if (tile + NST < n_tiles) issue_tile(tile + NST, stage);
        else cp_async_commit();
    }
    cp_async_wait<0>();
    TRC(4);
    pdl_launch_dependents();

    // ---- every warp leaves its (m, l, O) for its 16 queries in shared memory: wo[warp][16][HDP], wml[warp][16]
    // (rows padded by four floats: the eight query rows a warp stores at once land in different banks)
    constexpr int HDP = HD + 4;
    float* wo = reinterpret_cast<float*>(smem);
    float2* wml = reinterpret_cast<float2*>(smem + (size_t)4 * MT * 16 * HDP * sizeof(float));
    {
        float* dst = wo + (size_t)warp * 16 * HDP;
#pragma unroll
        for (int n = 0; n < NO; n++) {
            *reinterpret_cast<float2*>(dst + gid * HDP + n * 8 + 2 * tig) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(dst + (gid + 8) * HDP + n * 8 + 2 * tig) = make_float2(o[n][2], o[n][3]);
        }
        if (tig == 0) {
            wml[warp * 16 + gid] = make_float2(m_run[0], l_run[0]);
            wml[warp * 16 + gid + 8] = make_float2(m_run[1], l_run[1]);
        }
    }
    __syncthreads();

    // ---- merges:  out = sum_c O_c 2^(m_c - m) / sum_c l_c 2^(m_c - m)   (crates/gpu/src/shaders/attention.metal:983-1031)
    // first the four token slices inside the CTA, then the CTAs of the cluster through distributed shared memory,
    // then (if the context needed more than one cluster) the clusters through memory.  A thread owns a run of
    // eight columns of one query.
    constexpr int TPH = HD / 8;             // 8-column runs per head
    constexpr int QPP = NTHR / TPH;         // queries finished per pass over the threads
    float* co = wo + (size_t)4 * MT * 16 * HDP + 2 * 4 * MT * 16;  // [QT][HD] after wo and wml
    float2* cml = reinterpret_cast<float2*>(co + (size_t)QT * HD);
    const int part = threadIdx.x % TPH;
#pragma unroll
    for (int ql0 = 0; ql0 < QT; ql0 += QPP) {
        const int ql = ql0 + threadIdx.x / TPH;
        const int w0 = ql / 16, qq = ql % 16;  // warp (m-tile) and row that held the query
        float m = -INFINITY, den = 0.f, accv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < SL; s2++) m = fmaxf(m, wml[(s2 * MT + w0) * 16 + qq].x);
        const float mu = (m == -INFINITY) ? 0.f : m;
#pragma unroll
        for (int s2 = 0; s2 < SL; s2++) {
            const int w = s2 * MT + w0;
            const float2 v = wml[w * 16 + qq];
            const float wgt = exp2f(v.x - mu);
            den += v.y * wgt;
            const float4* po = reinterpret_cast<const float4*>(wo + ((size_t)w * 16 + qq) * HDP + part * 8);
            const float4 a = po[0], b2 = po[1];
            accv[0] += a.x * wgt, accv[1] += a.y * wgt, accv[2] += a.z * wgt, accv[3] += a.w * wgt;
            accv[4] += b2.x * wgt, accv[5] += b2.y * wgt, accv[6] += b2.z * wgt, accv[7] += b2.w * wgt;
        }
        if (defer_merge) {
            // partials-only launch (no cluster): the CTA's share goes straight to memory, the merge launch takes over
            const int qi = qtile * QT + ql;
            if (qi < n_queries) {
                const size_t pi = ((size_t)(row_first + qi / G) * n_q_heads + (kvh * G + qi % G)) * gridDim.x + blockIdx.x;
                float4* po = reinterpret_cast<float4*>(part_o + pi * HD + part * 8);
                po[0] = make_float4(accv[0], accv[1], accv[2], accv[3]);
                po[1] = make_float4(accv[4], accv[5], accv[6], accv[7]);
                if (part == 0) part_ml[pi] = make_float2(m, den);
            }
            continue;
        }
        float4* dst = reinterpret_cast<float4*>(co + (size_t)ql * HD + part * 8);
        dst[0] = make_float4(accv[0], accv[1], accv[2], accv[3]);
        dst[1] = make_float4(accv[4], accv[5], accv[6], accv[7]);
        if (part == 0) cml[ql] = make_float2(m, den);
    }
    if (defer_merge) {
        TRC(6);
        return;
    }
    if (cluster_size > 1) cluster.sync();
    else __syncthreads();
    TRC(5);

    // CTA `rank` of the cluster finishes queries rank, rank + cluster_size, ... of the tile
    const int rank = cluster_size > 1 ? (int)cluster.block_rank() : 0;
    const int n_clusters = gridDim.x / cluster_size, cl = blockIdx.x / cluster_size;
    const int n_own = (QT - rank + cluster_size - 1) / cluster_size;  // queries rank, rank + cs, ... below QT
    for (int j0 = 0; j0 < n_own; j0 += QPP) {  // uniform trip count per CTA
        const int j = j0 + threadIdx.x / TPH;
        const int ql = rank + j * cluster_size;  // query within the tile
        const int qi = qtile * QT + ql;
        const bool active = j < n_own && qi < n_queries;
        float m = -INFINITY, den = 0.f, accv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] = 0.f;
        if (active) {
            // members in rank order, eight at a time (all loads of a batch are in flight together)
            for (int c = 0; c < cluster_size; c++) {
                const float2* rml = cluster_size > 1 ? cluster.map_shared_rank(cml, c) : cml;
                m = fmaxf(m, rml[ql].x);
            }
            const float mu = (m == -INFINITY) ? 0.f : m;
            for (int c0 = 0; c0 < cluster_size; c0 += 8) {
                float2 ml[8];
                float4 va[8], vb[8];
#pragma unroll
                for (int c = 0; c < 8; c++)
                    if (c0 + c < cluster_size) {
                        const float2* rml = cluster_size > 1 ? cluster.map_shared_rank(cml, c0 + c) : cml;
                        const float* ro = cluster_size > 1 ? cluster.map_shared_rank(co, c0 + c) : co;
                        ml[c] = rml[ql];
                        const float4* po = reinterpret_cast<const float4*>(ro + (size_t)ql * HD + part * 8);
                        va[c] = po[0], vb[c] = po[1];
                    }
#pragma unroll
                for (int c = 0; c < 8; c++)
                    if (c0 + c < cluster_size) {
                        const float wgt = exp2f(ml[c].x - mu);
                        den += ml[c].y * wgt;
                        accv[0] += va[c].x * wgt, accv[1] += va[c].y * wgt, accv[2] += va[c].z * wgt, accv[3] += va[c].w * wgt;
                        accv[4] += vb[c].x * wgt, accv[5] += vb[c].y * wgt, accv[6] += vb[c].z * wgt, accv[7] += vb[c].w * wgt;
                    }
            }
        }
        const int row = row_first + (active ? qi / G : 0), head = kvh * G + (active ? qi % G : 0);
        const int e0 = head * HD + part * 8;
        if (n_clusters == 1 && !defer_merge) {
            const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) accv[i] *= inv;
            if (out && active) {
                uint4 pk;
                __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
                for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(accv[i]);
                *reinterpret_cast<uint4*>(out + (size_t)row * n_q_heads * HD + e0) = pk;
            }
            if (act.xp) act_store8(accv, act.xp, act.xs, row, e0, (n_q_heads * HD) >> 8, active);
        } else if (active) {  // this cluster's share goes to memory; the last CTA of all clusters finishes the job
            const size_t pi = ((size_t)row * n_q_heads + head) * n_clusters + cl;
            float4* po = reinterpret_cast<float4*>(part_o + pi * HD + part * 8);
            po[0] = make_float4(accv[0], accv[1], accv[2], accv[3]);
            po[1] = make_float4(accv[4], accv[5], accv[6], accv[7]);
            if (part == 0) part_ml[pi] = make_float2(m, den);
        }
    }
    // nobody may leave while a neighbour still reads its shared memory: arrive now, wait just before leaving, so the
    // barrier's latency hides behind the ticket and the last merge
    TRC(6);
    if (cluster_size > 1) cluster.barrier_arrive();
    if (n_clusters == 1 || defer_merge) {  // deferred: whoever runs next merges the shares left in memory
        if (cluster_size > 1) cluster.barrier_wait();
        return;
    }

    // ---- the last CTA to finish among all clusters of this (stream, kv head, query tile) merges the clusters'
    // shares.  A ticket counter decides who is last; nobody waits on anybody.
    const int ticket_id = (blockIdx.z * nkv + kvh) * n_qtiles + qtile;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(&tickets[ticket_id], 1u);
        s_last = old == gridDim.x - 1;
        if (s_last) tickets[ticket_id] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) {
        if (cluster_size > 1) cluster.barrier_wait();
        return;
    }
    __threadfence();
    for (int ql0 = 0; ql0 < QT; ql0 += QPP) {
        const int ql = ql0 + threadIdx.x / TPH;
        const int qi = qtile * QT + ql;
        const bool active = ql < QT && qi < n_queries;
        const int row = row_first + (active ? qi / G : 0), head = kvh * G + (active ? qi % G : 0);
        const size_t pi = ((size_t)row * n_q_heads + head) * n_clusters;
        float m = -INFINITY, den = 0.f, accv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] = 0.f;
        if (active) {
            for (int c = 0; c < n_clusters; c++) m = fmaxf(m, __ldcg(&part_ml[pi + c]).x);
            const float mu = (m == -INFINITY) ? 0.f : m;
#pragma unroll 4
            for (int c = 0; c < n_clusters; c++) {
                const float2 v = __ldcg(&part_ml[pi + c]);
                const float wgt = exp2f(v.x - mu);
                den += v.y * wgt;
                const float4* po = reinterpret_cast<const float4*>(part_o + (pi + c) * HD + part * 8);
                const float4 a = __ldcg(po), b2 = __ldcg(po + 1);
                accv[0] += a.x * wgt, accv[1] += a.y * wgt, accv[2] += a.z * wgt, accv[3] += a.w * wgt;
                accv[4] += b2.x * wgt, accv[5] += b2.y * wgt, accv[6] += b2.z * wgt, accv[7] += b2.w * wgt;
            }
        }
        const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] *= inv;
        const int e0 = head * HD + part * 8;
        if (out && active) {
            uint4 pk;
            __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
            for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(accv[i]);
            *reinterpret_cast<uint4*>(out + (size_t)row * n_q_heads * HD + e0) = pk;
        }
        if (act.xp) act_store8(accv, act.xp, act.xs, row, e0, (n_q_heads * HD) >> 8, active);
    }
    if (cluster_size > 1) cluster.barrier_wait();
}

// ---- merge of the split-KV shares left by a partials-only launch: one CTA per (row, head).
// out = sum_c O_c 2^(m_c - m) / sum_c l_c 2^(m_c - m)   (crates/gpu/src/shaders/attention.metal:983-1031)
// The CTA's threads are (split group, eight-column part): a group folds its splits c = g, g + n_groups, ... in that
// order into one (m, l, O) share, the shares meet in shared memory, and the first group combines them in group order -
// a fixed summation tree that depends only on the number of splits.
constexpr int MERGE_THREADS = 256;
__global__ void __launch_bounds__(MERGE_THREADS)
    attn_merge_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml, int n_splits, int n_q_heads, int head_dim,
                      __half* __restrict__ out, ActOut act) {
    __shared__ float sh_o[MERGE_THREADS * 8];
    __shared__ float2 sh_ml[MERGE_THREADS];
    const int lpi = head_dim >> 3;              // threads per group (one per eight columns)
    const int n_groups = MERGE_THREADS / lpi;   // split groups
    const int grp = threadIdx.x / lpi, part = threadIdx.x % lpi;
    const int item = blockIdx.x;                // row * n_q_heads + head
    pdl_wait();
    const size_t pi = (size_t)item * n_splits;
    float m = -INFINITY, den = 0.f, accv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) accv[i] = 0.f;
    // a group has at most MAX_SPLITS / 16 = 4 splits: all their loads are issued together (one round trip to L2
    // instead of two dependent ones), then folded in split order exactly as a loop over them would
    {
        constexpr int PER = 4;
        float2 ml[PER];
        float4 va[PER], vb[PER];
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int c = grp + k * n_groups;
            ml[k] = make_float2(-INFINITY, 0.f), va[k] = vb[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < n_splits) {
                ml[k] = __ldcg(&part_ml[pi + c]);
                const float4* po = reinterpret_cast<const float4*>(part_o + (pi + c) * head_dim + part * 8);
                va[k] = __ldcg(po), vb[k] = __ldcg(po + 1);
            }
        }
#pragma unroll
        for (int k = 0; k < PER; k++) m = fmaxf(m, ml[k].x);
        for (int c = grp + PER * n_groups; c < n_splits; c += n_groups) m = fmaxf(m, __ldcg(&part_ml[pi + c]).x);  // never taken at <= 64 splits
        const float mu = (m == -INFINITY) ? 0.f : m;
#pragma unroll
        for (int k = 0; k < PER; k++)
            if (grp + k * n_groups < n_splits) {
                const float wgt = exp2f(ml[k].x - mu);
                den += ml[k].y * wgt;
                accv[0] += va[k].x * wgt, accv[1] += va[k].y * wgt, accv[2] += va[k].z * wgt, accv[3] += va[k].w * wgt;
                accv[4] += vb[k].x * wgt, accv[5] += vb[k].y * wgt, accv[6] += vb[k].z * wgt, accv[7] += vb[k].w * wgt;
            }
        for (int c = grp + PER * n_groups; c < n_splits; c += n_groups) {
            const float2 v = __ldcg(&part_ml[pi + c]);
            const float wgt = exp2f(v.x - mu);
            den += v.y * wgt;
            const float4* po = reinterpret_cast<const float4*>(part_o + (pi + c) * head_dim + part * 8);
            const float4 a = __ldcg(po), b2 = __ldcg(po + 1);
            accv[0] += a.x * wgt, accv[1] += a.y * wgt, accv[2] += a.z * wgt, accv[3] += a.w * wgt;
            accv[4] += b2.x * wgt, accv[5] += b2.y * wgt, accv[6] += b2.z * wgt, accv[7] += b2.w * wgt;
        }
    }
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < 8; i++) sh_o[threadIdx.x * 8 + i] = accv[i];
    sh_ml[threadIdx.x] = make_float2(m, den);
    __syncthreads();
    if (threadIdx.x >= 32 && threadIdx.x >= lpi) return;  // the first warp finishes (its lanes past lpi only take part in the shuffles)
    const bool active = threadIdx.x < lpi;
    float mm = -INFINITY, dd = 0.f, o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = 0.f;
    if (active) {
        for (int g = 0; g < n_groups; g++) mm = fmaxf(mm, sh_ml[g * lpi + part].x);
        const float mu = (mm == -INFINITY) ? 0.f : mm;
        for (int g = 0; g < n_groups; g++) {
            const float2 v = sh_ml[g * lpi + part];
            const float wgt = exp2f(v.x - mu);
            dd += v.y * wgt;
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] += sh_o[(g * lpi + part) * 8 + i] * wgt;
        }
        const float inv = dd > 0.f ? 1.0f / dd : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] *= inv;
    }
    const int row = item / n_q_heads, head = item % n_q_heads;
    const int e0 = head * head_dim + part * 8;
    if (out && active) {
        uint4 pk;
        __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(o[i]);
        *reinterpret_cast<uint4*>(out + (size_t)row * n_q_heads * head_dim + e0) = pk;
    }
    if (act.xp) act_store8(o, act.xp, act.xs, row, active ? e0 : 0, (n_q_heads * head_dim) >> 8, active);
}

// The same merge for at most four splits: a thread is (query row x head, eight-column part) and folds the query's
// shares itself, in split order, all loads in one round trip - no shared memory, no barrier, sixteen (head_dim 128) or
// thirty-two (64) queries per CTA.  Passes over many rows cut the context into few chunks and have tens of thousands of
// queries to finish; one CTA per query, most of whose threads have no split to fold, took 40 us there.
template <int HD>
__global__ void __launch_bounds__(MERGE_THREADS)
    attn_merge_few_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml, int n_splits, int n_items, int n_q_heads,
                          __half* __restrict__ out, ActOut act) {
    constexpr int LPI = HD / 8;
    const int item = blockIdx.x * (MERGE_THREADS / LPI) + threadIdx.x / LPI, part = threadIdx.x % LPI;
    const bool active = item < n_items;
    pdl_wait();
    float2 ml[4];
    float4 va[4], vb[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        ml[k] = make_float2(-INFINITY, 0.f), va[k] = vb[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active && k < n_splits) {
            const size_t pi = (size_t)item * n_splits + k;
            ml[k] = __ldcg(&part_ml[pi]);
            const float4* po = reinterpret_cast<const float4*>(part_o + pi * HD + part * 8);
            va[k] = __ldcg(po), vb[k] = __ldcg(po + 1);
        }
    }
    pdl_launch_dependents();
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; k++) m = fmaxf(m, ml[k].x);
    const float mu = (m == -INFINITY) ? 0.f : m;
    float den = 0.f, o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++)
        if (k < n_splits) {
            const float wgt = exp2f(ml[k].x - mu);
            den += ml[k].y * wgt;
            o[0] += va[k].x * wgt, o[1] += va[k].y * wgt, o[2] += va[k].z * wgt, o[3] += va[k].w * wgt;
            o[4] += vb[k].x * wgt, o[5] += vb[k].y * wgt, o[6] += vb[k].z * wgt, o[7] += vb[k].w * wgt;
        }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] *= inv;
    const int row = active ? item / n_q_heads : 0, head = active ? item % n_q_heads : 0;
    const int e0 = head * HD + part * 8;
    if (out && active) {
        uint4 pk;
        __half* pp = reinterpret_cast<__half*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; i++) pp[i] = __float2half_rn(o[i]);
        *reinterpret_cast<uint4*>(out + (size_t)row * n_q_heads * HD + e0) = pk;
    }
    if (act.xp) act_store8(o, act.xp, act.xs, row, e0, (n_q_heads * HD) >> 8, active);
}

}  // namespace

// Dynamic shared memory of a CTA: the K/V ring, or - four m-tiles - the larger area the warps' partials are merged in.
static size_t attn_smem_bytes(int hd, int mt) {
    const size_t ring = (size_t)NST * 2 * TILE_TOKENS * hd * sizeof(__half);
    const size_t merge = ((size_t)4 * mt * 16 * (hd + 4) + 2 * 4 * mt * 16 + (size_t)16 * mt * hd + 2 * 16 * mt) * sizeof(float);
    return ring > merge ? ring : merge;
}

// How many clusters of `cs` CTAs of the kernel can be resident at once (cached per shape and device).
template <int HD, int MT>
static int max_clusters_t(int device, int cs) {
    static int cache[ATTN_MAX_DEVICES][5] = {};
    const int slot = cs == 16 ? 4 : cs == 8 ? 3 : cs == 4 ? 2 : cs == 2 ? 1 : 0;
    if (device < 0 || device >= ATTN_MAX_DEVICES) return 0;
    if (cache[device][slot]) return cache[device][slot] > 0 ? cache[device][slot] : 0;
    const size_t smem = attn_smem_bytes(HD, MT);
    if (cudaFuncSetAttribute(attn_partial_kernel<HD, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
    // clusters of sixteen are beyond the portable size: allowed on this part, the occupancy query says whether they fit
    if (cudaFuncSetAttribute(attn_partial_kernel<HD, MT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        if (cs > 8) return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs * 64, 1, 1);
    cfg.blockDim = dim3(ATT_THREADS * MT);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cs > 1 ? 1 : 0;
    int n = 0;
    if (cs > 1) {
        if (cudaOccupancyMaxActiveClusters(&n, attn_partial_kernel<HD, MT>, &cfg) != cudaSuccess) n = 0;
    } else {
        int per_sm = 0, sms = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_partial_kernel<HD, MT>, ATT_THREADS * MT, smem);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        n = per_sm * sms;
    }
    cudaGetLastError();
    cache[device][slot] = n > 0 ? n : (cs > 1 ? -1 : 1);  // -1: clusters of this size do not fit at all
    return cache[device][slot] > 0 ? cache[device][slot] : 0;
}
static int max_clusters(int device, int hd, int mt, int cs) {
    if (hd == 128) return mt == 4 ? max_clusters_t<128, 4>(device, cs) : mt == 2 ? max_clusters_t<128, 2>(device, cs) : max_clusters_t<128, 1>(device, cs);
    return mt == 4 ? max_clusters_t<64, 4>(device, cs) : mt == 2 ? max_clusters_t<64, 2>(device, cs) : max_clusters_t<64, 1>(device, cs);
}

AttnPlan attn_plan(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads, int max_len) {
    AttnPlan p;
    const int G = n_q_heads / kv->view.kv_heads;
    const int n_queries = rows_per_seq * G;
    p.mt = n_queries <= 16 ? 1 : 2;
    p.n_qtiles = (n_queries + 16 * p.mt - 1) / (16 * p.mt);
    p.groups = rows / rows_per_seq;
    // the split is planned for the length rounded up to 512, so calls whose lengths differ by a few rows (a row
    // verified in a batch, then decoded alone) cut the context at the same places and sum in the same order
    const int planned = max_len > 0 ? (max_len + 511) / 512 * 512 : 512;
    const int tiles_total = planned / TILE_TOKENS;
    const int base_ctas = p.groups * kv->view.kv_heads * p.n_qtiles;
    // one wave: as many chunks per (stream, kv head, query tile) as the device can hold at once, in clusters of
    // up to four CTAs (larger clusters leave SMs of a GPC unused)
    int cand_splits[5] = {1, 0, 0, 0, 0}, most = 1;  // for cluster sizes 1, 2, 4, 8, 16
    static int per_sm = 0, max_cs_log2 = -1;  // TSB_ATTN_CTAS_PER_SM, TSB_ATTN_MAX_CLUSTER override (experiments)
    if (!per_sm) {
        const char* env = getenv("TSB_ATTN_CTAS_PER_SM");
        per_sm = env ? atoi(env) : 2;
        if (per_sm < 1) per_sm = 1;
        env = getenv("TSB_ATTN_MAX_CLUSTER");
        const int v = env ? atoi(env) : 4;  // larger clusters measured slower: fewer of them fit, and their barriers cost more
        max_cs_log2 = v >= 16 ? 4 : v >= 8 ? 3 : v >= 4 ? 2 : (v >= 2 ? 1 : 0);
    }
    for (int i = 0; i <= max_cs_log2; i++) {
        const int cs = 1 << i;
        int resident = max_clusters(ctx->device, kv->view.head_dim, p.mt, cs);  // clusters
        if (resident > ctx->sm_count * per_sm / cs) resident = ctx->sm_count * per_sm / cs;
        int clusters_per = resident / base_ctas;  // per (stream, head, tile)
        if (clusters_per < 1) {
            if (cs > 1) continue;  // clusters of this size would not all be resident: a second wave costs more than it saves
            clusters_per = 1;
        }
        if (clusters_per > MAX_SPLITS) clusters_per = MAX_SPLITS;
        int splits = clusters_per * cs;
        if (splits > tiles_total) splits = (tiles_total / cs) * cs;
        cand_splits[i] = splits;  // 0 when a cluster would be longer than the context
        if (splits > most) most = splits;
    }
    // the largest cluster that keeps at least 4/5 of the parallelism: fewer shares travel through memory
    int best_splits = cand_splits[0] > 0 ? cand_splits[0] : 1, best_cs = 1;
    bool chosen = false;
    for (int i = max_cs_log2; i >= 1 && !chosen; i--)
        if (cand_splits[i] * 5 >= most * 4 && cand_splits[i] > 0) best_splits = cand_splits[i], best_cs = 1 << i, chosen = true;
    p.cluster_size = best_cs;
    p.n_splits = best_splits;
    const int tiles_per = (tiles_total + p.n_splits - 1) / p.n_splits;
    p.chunk = (tiles_per < 1 ? 1 : tiles_per) * TILE_TOKENS;
    return p;
}

size_t attn_scratch_bytes(int rows, int n_q_heads, int head_dim) {
    // chunk partials (O and (m, l)) plus one ticket word per (stream, kv head, query tile), which is at most
    // rows * n_q_heads words; the tickets must be zero before the first launch and reset themselves
    return (size_t)rows * n_q_heads * MAX_SPLITS * ((size_t)head_dim * sizeof(float) + sizeof(float2)) +
           (size_t)rows * n_q_heads * sizeof(uint32_t);
}

template <int HD, int MT>
static cudaError_t launch_attn_t(tsb_ctx* ctx, cudaStream_t st, const AttnPlan& p, dim3 grid, size_t smem, KvView view, int layer,
                                 const __half* q, int64_t q_stride, const tsb_row_desc* rows_dev, int rows_per_seq,
                                 int n_q_heads, float scale_log2e, float* part_o, float2* part_ml, uint32_t* tickets,
                                 __half* out, ActOut act, int defer_merge = 0) {
    static SmemOptIn configured;
    if (cudaError_t e = tsb_opt_in_smem(ctx, attn_partial_kernel<HD, MT>, smem, configured); e != cudaSuccess) return e;
    return tsb_launch_cluster(ctx, attn_partial_kernel<HD, MT>, grid, dim3(ATT_THREADS * MT), smem, st, true,
                              (unsigned)p.cluster_size, view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads,
                              scale_log2e, p.chunk, p.cluster_size, part_o, part_ml, tickets, out, act, ctx->dev_error, defer_merge);
}

// TSB_ATTN_MODE=0 keeps the single launch whose CTAs merge through clusters and a ticket; the default (1) is the
// partials launch followed by the merge launch.
static bool attn_split_merge_mode() {
    static int mode = -1;
    if (mode < 0) {
        const char* env = getenv("TSB_ATTN_MODE");
        mode = env ? atoi(env) : 1;
    }
    return mode == 1;
}

// The merge launch that follows a partials launch: the per-query kernel, or - few splits - the many-queries-per-CTA one.
static cudaError_t launch_attn_merge(tsb_ctx* ctx, cudaStream_t st, const float* part_o, const float2* part_ml, int n_splits, int rows,
                                     int n_q_heads, int head_dim, __half* out, ActOut act) {
    const int items = rows * n_q_heads;
    if (n_splits <= 4 && (head_dim == 128 || head_dim == 64)) {
        const int per_cta = MERGE_THREADS / (head_dim / 8);
        const dim3 grid((unsigned)((items + per_cta - 1) / per_cta));
        if (head_dim == 128)
            return tsb_launch(ctx, attn_merge_few_kernel<128>, grid, dim3(MERGE_THREADS), 0, st, true, part_o, part_ml, n_splits, items, n_q_heads, out, act);
        return tsb_launch(ctx, attn_merge_few_kernel<64>, grid, dim3(MERGE_THREADS), 0, st, true, part_o, part_ml, n_splits, items, n_q_heads, out, act);
    }
    return tsb_launch(ctx, attn_merge_kernel, dim3((unsigned)items), dim3(MERGE_THREADS), 0, st, true, part_o, part_ml, n_splits, n_q_heads,
                      head_dim, out, act);
}

cudaError_t launch_attn_decode_rows(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                    __half* out, ActOut act, const tsb_row_desc* rows_dev, int rows, int rows_per_seq,
                                    int n_q_heads, float scale, int max_len, void* scratch, int rows_cap) {
    if (attn_split_merge_mode()) {
        // every chunk CTA leaves its share in memory and a second, wide launch merges them (one CTA per row and head)
        const float* part_o;
        const float2* part_ml;
        int n_splits;
        if (attn_tc_applicable(ctx, kv, rows, rows_per_seq, n_q_heads)) {
            // many queries per (stream, kv head), or streams enough to fill the device: the tensor-memory kernel; its shares
            // always go through the merge
            cudaError_t e = launch_attn_tc_partials(ctx, st, kv, layer, q, q_stride, rows_dev, rows, rows_per_seq, n_q_heads, scale, max_len,
                                                    scratch, &part_o, &part_ml, &n_splits);
            if (e != cudaSuccess) return e;
            return launch_attn_merge(ctx, st, part_o, part_ml, n_splits, rows, n_q_heads, kv->view.head_dim, out, act);
        }
        cudaError_t e = launch_attn_partials(ctx, st, kv, layer, q, q_stride, rows_dev, rows, rows_per_seq, n_q_heads, scale, max_len, scratch,
                                             &part_o, &part_ml, &n_splits, out, act);
        if (e != cudaSuccess || n_splits == 1) return e;  // a single split wrote the output itself
        return launch_attn_merge(ctx, st, part_o, part_ml, n_splits, rows, n_q_heads, kv->view.head_dim, out, act);
    }
    const AttnPlan p = attn_plan(ctx, kv, rows, rows_per_seq, n_q_heads, max_len);
    const int hd = kv->view.head_dim;
    const int n_clusters = p.n_splits / p.cluster_size;
    float* part_o = reinterpret_cast<float*>(scratch);
    float2* part_ml = reinterpret_cast<float2*>(part_o + (size_t)rows * n_q_heads * n_clusters * hd);
    // tickets sit at the very end of the scratch area, whatever the split count of this call
    uint32_t* tickets = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(scratch) +
                                                    (size_t)rows_cap * n_q_heads * MAX_SPLITS * ((size_t)hd * sizeof(float) + sizeof(float2)));
    const float scale_log2e = scale * 1.4426950408889634f;
    dim3 grid((unsigned)p.n_splits, (unsigned)(kv->view.kv_heads * p.n_qtiles), (unsigned)p.groups);
    const size_t smem = (size_t)NST * 2 * TILE_TOKENS * hd * sizeof(__half);
    if (hd == 128) {
        if (p.mt == 2)
            return launch_attn_t<128, 2>(ctx, st, p, grid, smem, kv->view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads,
                                         scale_log2e, part_o, part_ml, tickets, out, act);
        return launch_attn_t<128, 1>(ctx, st, p, grid, smem, kv->view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads,
                                     scale_log2e, part_o, part_ml, tickets, out, act);
    }
    if (p.mt == 2)
        return launch_attn_t<64, 2>(ctx, st, p, grid, smem, kv->view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads,
                                    scale_log2e, part_o, part_ml, tickets, out, act);
    return launch_attn_t<64, 1>(ctx, st, p, grid, smem, kv->view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads,
                                scale_log2e, part_o, part_ml, tickets, out, act);
}

// The split plan of the partials-only launch: no clusters, as many KV chunks per (stream, kv head, query tile) as
// the device holds CTAs at once, up to two per SM (at most MAX_SPLITS): one wave, and with two tiles or fewer per
// CTA every K/V byte of a chunk is in flight from the first instruction.  Like attn_plan it is made for the length rounded up
// to 512 and does not depend on the row count while the queries fit one tile, so a row gets the same chunks - and
// the same sums - whether it is verified in a batch or decoded alone.
static AttnPlan attn_plan_partials(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads, int max_len) {
    AttnPlan p;
    const int G = n_q_heads / kv->view.kv_heads;
    const int n_queries = rows_per_seq * G;
    // every query tile of a (stream, kv head) streams that head's K and V again, so many queries (a tree's rows x the
    // group's heads) go 64 to a CTA
    p.mt = n_queries <= 16 ? 1 : n_queries <= 64 ? 2 : 4;
    p.n_qtiles = (n_queries + 16 * p.mt - 1) / (16 * p.mt);
    p.groups = rows / rows_per_seq;
    p.cluster_size = 1;
    const int planned = max_len > 0 ? (max_len + 511) / 512 * 512 : 512;
    const int tiles_total = planned / TILE_TOKENS;
    const int base_ctas = p.groups * kv->view.kv_heads * p.n_qtiles;
    int resident = max_clusters(ctx->device, kv->view.head_dim, p.mt, 1);  // CTAs the device holds at once
    if (resident > ctx->sm_count * 2) resident = ctx->sm_count * 2;
    if (resident < 1) resident = ctx->sm_count;
    int splits = resident / (base_ctas > 0 ? base_ctas : 1);
    if (splits < 1) {
        // more CTAs than the device holds: cut the context so that the waves come out even (a CTA costs its tiles
        // plus about four tiles' time of fixed work)
        float best = 1e30f;
        for (int s = 1; s <= 8 && s <= tiles_total; s++) {
            const int waves = (base_ctas * s + resident - 1) / resident;
            const float cost = (float)waves * ((float)((tiles_total + s - 1) / s) + 4.f);
            if (cost < best - 1e-3f) best = cost, splits = s;
        }
    }
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits > tiles_total) splits = tiles_total;
    const int tiles_per = (tiles_total + splits - 1) / splits;
    p.chunk = tiles_per * TILE_TOKENS;
    p.n_splits = (tiles_total + tiles_per - 1) / tiles_per;
    return p;
}

#ifdef TSB_ATTN_TRACE
static uint32_t* g_attn_trace = nullptr;
extern "C" __attribute__((visibility("default"))) void tsb_debug_set_attn_trace(void* p) { g_attn_trace = (uint32_t*)p; }
#define ATTN_TICKETS g_attn_trace
#else
#define ATTN_TICKETS nullptr
#endif
cudaError_t launch_attn_partials(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                 const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int n_q_heads, float scale, int max_len,
                                 void* scratch, const float** part_o_out, const float2** part_ml_out, int* n_splits_out, __half* out_single,
                                 ActOut act_single) {
    const AttnPlan p = attn_plan_partials(ctx, kv, rows, rows_per_seq, n_q_heads, max_len);
    const int hd = kv->view.head_dim;
    float* part_o = reinterpret_cast<float*>(scratch);
    float2* part_ml = reinterpret_cast<float2*>(part_o + (size_t)rows * n_q_heads * p.n_splits * hd);
    *part_o_out = part_o, *part_ml_out = part_ml, *n_splits_out = p.n_splits;
    const float scale_log2e = scale * 1.4426950408889634f;
    dim3 grid((unsigned)p.n_splits, (unsigned)(kv->view.kv_heads * p.n_qtiles), (unsigned)p.groups);
    const size_t smem = attn_smem_bytes(hd, p.mt);
    // one split: nothing to merge - the CTAs finish their queries themselves and write the output (the same arithmetic
    // as a merge of one share: weight 2^0, one division)
    const bool single = p.n_splits == 1;
    const ActOut none{nullptr, nullptr};
    __half* out = single ? out_single : nullptr;
    const ActOut act = single ? act_single : none;
    const int defer = single ? 0 : 1;
#define TSB_ATTN_LAUNCH(HDV, MTV)                                                                                                          \
    return launch_attn_t<HDV, MTV>(ctx, st, p, grid, smem, kv->view, layer, q, q_stride, rows_dev, rows_per_seq, n_q_heads, scale_log2e, part_o, \
                                   part_ml, ATTN_TICKETS, out, act, defer)
    if (hd == 128) {
        if (p.mt == 4) TSB_ATTN_LAUNCH(128, 4);
        if (p.mt == 2) TSB_ATTN_LAUNCH(128, 2);
        TSB_ATTN_LAUNCH(128, 1);
    }
    if (p.mt == 4) TSB_ATTN_LAUNCH(64, 4);
    if (p.mt == 2) TSB_ATTN_LAUNCH(64, 2);
    TSB_ATTN_LAUNCH(64, 1);
#undef TSB_ATTN_LAUNCH
}

extern "C" {

size_t tsb_attn_scratch_bytes(int32_t rows, int32_t n_q_heads, int32_t head_dim) {
    if (rows <= 0 || n_q_heads <= 0 || head_dim <= 0) return 0;
    return attn_scratch_bytes(rows, n_q_heads, head_dim);
}

int32_t tsb_attn_decode_rows(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, const void* q_f16, int64_t q_stride,
                             void* out_f16, const tsb_row_desc* rows_dev, int32_t rows, int32_t rows_per_seq,
                             int32_t n_q_heads, float scale, int32_t max_len, void* scratch, size_t scratch_bytes) {
    if (!ctx || !kv) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, q_f16 && out_f16 && rows_dev && scratch, "null buffer");
    TSB_REQUIRE(ctx, rows > 0 && rows_per_seq > 0 && rows % rows_per_seq == 0, "rows must be a whole number of streams");
    TSB_REQUIRE(ctx, rows_per_seq <= 128, "at most 128 in-flight rows per stream (mask width), got %d", rows_per_seq);
    TSB_REQUIRE(ctx, layer >= 0 && layer < kv->view.layers, "layer %d outside 0..%d", layer, kv->view.layers);
    TSB_REQUIRE(ctx, n_q_heads > 0 && n_q_heads % kv->view.kv_heads == 0, "n_q_heads must be a multiple of the kv heads");
    TSB_REQUIRE(ctx, (n_q_heads * kv->view.head_dim) % 256 == 0, "n_q_heads * head_dim must be a multiple of 256");
    TSB_REQUIRE(ctx, q_stride >= (int64_t)n_q_heads * kv->view.head_dim && q_stride % 2 == 0, "q_stride smaller than a row");
    // the longest stream bounds what the kernel may read; computed in 64 bits so it cannot wrap
    const int64_t reach = (int64_t)max_len;
    TSB_REQUIRE(ctx, reach >= rows_per_seq && reach <= (int64_t)kv->view.max_pages_per_seq * kv->view.page_tokens,
                "max_len %lld outside the cache (%lld positions per stream)", (long long)reach,
                (long long)kv->view.max_pages_per_seq * kv->view.page_tokens);
    TSB_REQUIRE(ctx, scratch_bytes >= attn_scratch_bytes(rows, n_q_heads, kv->view.head_dim), "scratch too small");
    DeviceGuard g(ctx);
    // the ticket words at the end of the caller's scratch are not known to be zero
    TSB_CUDA(ctx, cudaMemsetAsync(reinterpret_cast<uint8_t*>(scratch) + attn_scratch_bytes(rows, n_q_heads, kv->view.head_dim) -
                                      (size_t)rows * n_q_heads * sizeof(uint32_t),
                                  0, (size_t)rows * n_q_heads * sizeof(uint32_t), (cudaStream_t)s));
    TSB_CUDA(ctx, launch_attn_decode_rows(ctx, (cudaStream_t)s, kv, layer, (const __half*)q_f16, q_stride, (__half*)out_f16,
                                          ActOut{nullptr, nullptr}, rows_dev, rows, rows_per_seq, n_q_heads, scale, max_len,
                                          scratch, rows));
    return TSB_OK;
}


// ---- attention without a scratch argument ---------------------------------------------------------------
// Some callers cannot hand over a scratch buffer: a host that owns no device allocator of its own (an FFI
// binding that only forwards the buffers it was given), or one that must not allocate at the point of the
// call (inside a latency-critical loop where an allocation could block on other work of the device).  For
// them the chunk partials live in a fixed array that is part of the loaded module.
namespace {
constexpr size_t ATTN_STATIC_BYTES = TSB_ATTN_STATIC_SCRATCH_BYTES;
__device__ __align__(256) unsigned char g_attn_static_scratch[ATTN_STATIC_BYTES];
constexpr int ATTN_STATIC_MAX_DEVICES = 64;
void* g_attn_static_ptr[ATTN_STATIC_MAX_DEVICES] = {};  // per device: address of its copy of the array
std::mutex g_attn_static_mutex;

// Address of the array on the context's device (which must be current).  The first call per device asks the
// runtime for it; later calls read the table.
cudaError_t attn_static_scratch(const tsb_ctx* ctx, void** out) {
    if (ctx->device < 0 || ctx->device >= ATTN_STATIC_MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_attn_static_mutex);
    void*& slot = g_attn_static_ptr[ctx->device];
    if (!slot) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess) return e;
        slot = p;
    }
    *out = slot;
    return cudaSuccess;
}
}  // namespace

int32_t tsb_attn_decode_rows_static(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, const void* q_f16,
                                    int64_t q_stride, void* out_f16, const tsb_row_desc* rows_dev, int32_t rows,
                                    int32_t rows_per_seq, int32_t n_q_heads, float scale, int32_t max_len) {
    if (!ctx || !kv) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, rows > 0 && n_q_heads > 0, "rows and n_q_heads must be positive");
    const size_t need = attn_scratch_bytes(rows, n_q_heads, kv->view.head_dim);
    if (need > ATTN_STATIC_BYTES)
        return tsb_fail(ctx, TSB_ERR_INVALID,
                        "tsb_attn_decode_rows_static: %d rows x %d heads x head_dim %d need %zu bytes of scratch, the built-in "
                        "area holds %zu; use tsb_attn_decode_rows with a caller buffer",
                        rows, n_q_heads, kv->view.head_dim, need, (size_t)ATTN_STATIC_BYTES);
    DeviceGuard g(ctx);
    void* scratch = nullptr;
    TSB_CUDA(ctx, attn_static_scratch(ctx, &scratch));
    // same checks, same ticket clearing, same kernel as the entry point with a caller buffer
    return tsb_attn_decode_rows(ctx, s, kv, layer, q_f16, q_stride, out_f16, rows_dev, rows, rows_per_seq, n_q_heads, scale,
                                max_len, scratch, need);
}

}  // extern "C"
