// Fused dequantise + matmul over verbatim GGUF blocks (Q4_K, Q6_K, MXFP4).
//
// One kernel shape serves the M = 1 draft step and the K+1 verify batch:
// weights stream HBM -> shared memory through 1-D bulk async copies
// (cp.async.bulk, mbarrier completion) issued by a producer warp into a ring of
// stages; eight consumer warps rebuild f16 operands from the packed nibbles in
// registers and feed mma.sync m16n8k16 with the weights as the 16-row A operand
// and up to eight tokens as the B operand, fp32 accumulation.  A token is one B
// column, so its result does not depend on how many other tokens share the call
// (decode and verify agree bit for bit per token).
//
// The kernel is HBM-bound for tokens <= 8: per 16x256 weight tile it moves 2304
// bytes (Q4_K) and issues ~200 warp instructions, about half the SM's issue
// slots at full memory bandwidth.
//
// A CTA owns 16 weight rows over the whole reduction dimension; its eight
// consumer warps take one 256-column block each per stage and the partial sums
// meet in shared memory in a fixed order (deterministic).
//
// Programmatic dependent launch: the weight prefetch does not depend on the
// previous kernel, so the producer warp starts before griddepcontrol.wait; only
// the consumers (which read activations and write y) wait.
#include "gemm_blocks.cuh"

namespace {

// 1/rms of every token from the partial sums of x^2 its producer left (one warp).  Per token the lanes add their
// partials in index order and meet in a butterfly - the order does not depend on the token count - but the loads of
// four tokens are issued before the first sum, so the warp pays one memory latency per four tokens, not per token.
__device__ __forceinline__ void token_inv_rms(const EpiArgs& epi, int tokens, int tok0, int lane, float* inv_rms) {
    constexpr int TB = 4, PL = 8;  // tokens per batch, partials per lane per token (covers 256 partials)
    const int parts = epi.ss_parts;
    for (int t0 = 0; t0 < tokens; t0 += TB) {
        float v[TB][PL];
#pragma unroll
        for (int tt = 0; tt < TB; tt++)
#pragma unroll
            for (int j = 0; j < PL; j++) {
                const int i = lane + 32 * j;
                v[tt][j] = (t0 + tt < tokens && i < parts) ? epi.ss_in[(size_t)(tok0 + t0 + tt) * parts + i] : 0.f;
            }
#pragma unroll
        for (int tt = 0; tt < TB; tt++) {
            if (t0 + tt >= tokens) break;
            float sacc = 0.f;
#pragma unroll
            for (int j = 0; j < PL; j++) sacc += v[tt][j];
            for (int i = lane + 32 * PL; i < parts; i += 32) sacc += epi.ss_in[(size_t)(tok0 + t0 + tt) * parts + i];  // wider models
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
            if (lane == 0) inv_rms[t0 + tt] = 1.0f / sqrtf(sacc / (float)epi.d_in + epi.eps);
        }
    }
}

// GROUPED: one launch over many matrices of one shape (the experts of a routed feed-forward).  Work item =
// (matrix m, row group g); matrix m sits at W + m * w_stride, multiplies count[m] token rows whose operand tiles
// start at tile tile_start[m] of `act`, and its outputs are indexed from token tile_start[m] * 8.  A launch covers
// token rows [chunk0, chunk0 + 8 NT) of every matrix; matrices with fewer rows are skipped.  Producer and consumers
// walk the same compacted list, so the stage ring stays in step.  The token-tile width of a
// launch is fixed (8 NT): `tokens` is recomputed per matrix as min(8 NT, count - chunk0).
constexpr int GROUPED_MAX_MATS = 512;
struct GroupedArgs {
    const int32_t* count = nullptr;
    const int32_t* tile_start = nullptr;
    int n_mats = 0;
    int chunk0 = 0;
    int lo = 0, hi = 0x7fffffff;  // only matrices with lo < count <= hi take part in this launch
    int64_t w_stride = 0;
#ifdef TSB_GEMM_TRACE
    unsigned long long* trace = nullptr;  // development builds: eight nanosecond stamps per CTA
#endif
};

// Resident CTAs per SM the kernel is compiled for (register cap) and launched with.
#ifndef TSB_GEMM_CTAS_NT1
#define TSB_GEMM_CTAS_NT1 2
#endif
template <int QT, int NT>
constexpr int gemm_ctas_per_sm() {
    return NT == 1 && QT == TSB_Q4_K ? TSB_GEMM_CTAS_NT1 : (NT <= 2 ? 2 : 1);
}

template <int QT, int NT, int EPI, bool GROUPED = false>
__global__ void __launch_bounds__(GEMM_THREADS, (gemm_ctas_per_sm<QT, NT>()))
    gemm_quant_kernel(const uint8_t* __restrict__ W0, int64_t rows, int units /*256-col units per row*/,
                      ActOperand act, int tokens, int tok0, EpiArgs epi, uint32_t* __restrict__ err, GroupedArgs grp) {
    constexpr int UB = Fmt<QT>::UNIT_BYTES;
    constexpr int ROW_STRIDE = row_stride_for(UB);
    constexpr int STAGE_BYTES = TILE_ROWS * ROW_STRIDE;
    constexpr int NTOK = NT * 8;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + NUM_STAGES;
    float* inv_rms = reinterpret_cast<float*>(smem + 64);                                  // [NTOK] (<= 64 floats)
    float* red = reinterpret_cast<float*>(smem + 64 + 256);                                // [2][8 warps][NT][4][32]
    float* tile_out0 = red + 2 * CONSUMER_WARPS * NT * 4 * 32;                             // [2 groups in turn][2][NTOK][16]
    // Single-tile epilogues work element by element with the thread-to-element mapping of the sum loop (thread idx sums
    // and finishes element idx), so they alternate between two reduction buffers and keep one barrier per tile; the
    // paired ones park both tiles' partial sums first and need a second barrier before the buffers are reused.
    constexpr bool ELEMWISE = EPI == EPI_PLAIN || EPI == EPI_SCALE || EPI == EPI_RESID_NORM;
    uint8_t* stages = reinterpret_cast<uint8_t*>(tile_out0 + 4 * NTOK * 16);
    constexpr bool NEEDS_INV = EPI == EPI_SCALE || EPI == EPI_SILU || EPI == EPI_ROPE_STORE;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef TSB_GEMM_TRACE
    unsigned long long* trc = grp.trace ? grp.trace + (size_t)blockIdx.x * 8 : nullptr;
#define GTRC(i) if (trc && threadIdx.x == 0) trc[i] = global_timer_ns()
    if (trc && threadIdx.x == CONSUMER_WARPS * 32) trc[7] = global_timer_ns();
#else
#define GTRC(i)
#endif
    GTRC(0);
    const int n_tiles = (int)((rows + TILE_ROWS - 1) / TILE_ROWS);
    const int n_groups = num_groups<EPI>(n_tiles, epi);
    const int iters = (units + STAGE_UNITS - 1) / STAGE_UNITS;  // stages per row tile
    const int64_t row_bytes = (int64_t)units * UB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NUM_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    // GROUPED: the matrices that take part in this launch, compacted once per CTA (index, row count, first tile), so
    // the item walk touches no global memory and the items spread evenly over the CTAs
    __shared__ int grp_mat[GROUPED ? GROUPED_MAX_MATS : 1], grp_cnt[GROUPED ? GROUPED_MAX_MATS : 1], grp_tile[GROUPED ? GROUPED_MAX_MATS : 1];
    __shared__ int grp_active;
    if constexpr (GROUPED) {
        if (warp == 0) {
            int base = 0;
            for (int c = 0; c < grp.n_mats; c += 32) {
                const int mt = c + lane;
                const int cnt = mt < grp.n_mats ? grp.count[mt] : 0;
                const bool on = cnt > grp.lo && cnt <= grp.hi && cnt > grp.chunk0;
                const uint32_t mask = __ballot_sync(0xffffffffu, on);
                if (on) {
                    const int at = base + __popc(mask & ((1u << lane) - 1u));
                    grp_mat[at] = mt, grp_cnt[at] = cnt, grp_tile[at] = grp.tile_start[mt];
                }
                base += __popc(mask);
            }
            if (lane == 0) grp_active = base;
        }
    }
    __syncthreads();
    const int n_items = GROUPED ? n_groups * grp_active : n_groups;

    // The CTA is persistent: it walks groups blockIdx.x, +gridDim.x, ... and the stage ring runs on across
    // tile boundaries, so weight bytes stay in flight while the consumers reduce and store a finished tile.
    if (warp == CONSUMER_WARPS) {
        // ---- producer: one bulk copy per row per stage; sources are rounded down to 16 bytes (formats whose
        // rows are not 16-byte multiples) and the consumer skips the same slack.
        uint32_t n = 0;
        bool inv_done = !NEEDS_INV;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            int g = item;
            const uint8_t* W = W0;
            if constexpr (GROUPED) {
                const int a = item / n_groups;
                g = item - a * n_groups;
                W = W0 + (int64_t)grp_mat[a] * grp.w_stride;
            }
            const Group gr = group_of<EPI>(g, n_tiles, epi);
            for (int ti = 0; ti < gr.n; ti++) {
                const int64_t row0 = (int64_t)(ti ? gr.tile1 : gr.tile0) * TILE_ROWS;
                const int nrows = (int)min((int64_t)TILE_ROWS, rows - row0);
                for (int it = 0; it < iters; it++, n++) {
                    const uint32_t s = n % NUM_STAGES;
                    if (n >= NUM_STAGES) {
                        if (!inv_done) {
                            // the ring is primed: before blocking on it, turn the predecessor's partial sums of
                            // x^2 into 1/rms per token for the epilogue (the consumers pick it up at barrier 2)
                            pdl_wait();
                            token_inv_rms(epi, tokens, tok0, lane, inv_rms);
                            __syncwarp();
                            asm volatile("bar.arrive 2, %0;" ::"n"(GEMM_THREADS) : "memory");
                            inv_done = true;
                        }
                        if (!mbar_wait(&empty[s], ((n / NUM_STAGES) - 1) & 1, err)) return;
                    }
                    const int nun = min(STAGE_UNITS, units - it * STAGE_UNITS);
                    uint32_t bytes = 0;
                    const uint8_t* src = nullptr;
                    if (lane < nrows) {
                        const uint8_t* p = W + (row0 + lane) * row_bytes + (int64_t)it * STAGE_UNITS * UB;
                        const uint32_t slack = (uint32_t)(reinterpret_cast<uintptr_t>(p) & 15u);
                        src = p - slack;
                        bytes = (slack + (uint32_t)nun * UB + 15u) & ~15u;
                    }
                    uint32_t total = bytes;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                    if (lane == 0) mbar_expect_tx(&full[s], total);
                    __syncwarp();
                    if (lane < nrows) bulk_g2s(stages + s * STAGE_BYTES + lane * ROW_STRIDE, src, bytes, &full[s]);
                }
            }
        }
        if (!inv_done) {
            pdl_wait();
            token_inv_rms(epi, tokens, tok0, lane, inv_rms);
            __syncwarp();
            asm volatile("bar.arrive 2, %0;" ::"n"(GEMM_THREADS) : "memory");
        }
        // the dependents are released by the consumers, which have waited for the predecessor by then: a kernel
        // never lets its successor start before its own predecessor has finished
        return;
    }

    // ---- consumers
    const int gid = lane >> 2, tig = lane & 3;
    LaneAct<NT> la;
    la.nblk = units;
    for (int nt = 0; nt < NT; nt++) {
        la.xp[nt] = act.xp + (size_t)nt * units * 256 + lane;
        la.xs[nt] = act.xs + (size_t)nt * units * 32 + lane;
    }
    pdl_wait();  // activations come from the previous kernel
    GTRC(1);
    const ActOperand act0 = act;

    bool ok = true, have_inv = !NEEDS_INV;
    uint32_t n = 0, tile_no = 0, group_no = 0;
    uint32_t stage = 0, phase = 0;  // ring position of block n: n % NUM_STAGES and the parity of n / NUM_STAGES
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        if (item + (int)gridDim.x >= n_items) pdl_launch_dependents();  // last item of this CTA
        int g = item;
        const uint8_t* W = W0;
        if constexpr (GROUPED) {
            const int a = item / n_groups;
            g = item - a * n_groups;
            const int cnt = grp_cnt[a];
            W = W0 + (int64_t)grp_mat[a] * grp.w_stride;
            const int tile0 = grp_tile[a] + grp.chunk0 / 8;
            tokens = min(NT * 8, cnt - grp.chunk0);
            tok0 = tile0 * 8;
            act.xp = act0.xp + (size_t)tile0 * units * 256;
            act.xs = act0.xs + (size_t)tile0 * units * 32;
            for (int nt = 0; nt < NT; nt++) {
                la.xp[nt] = act.xp + (size_t)nt * units * 256 + lane;
                la.xs[nt] = act.xs + (size_t)nt * units * 32 + lane;
            }
        }
        const Group gr = group_of<EPI>(g, n_tiles, epi);
        // finished tiles alternate between two buffers, so a group's epilogue may still be reading its tiles while
        // the next group's sums are written: no barrier after the epilogue
        float* tile_out = tile_out0 + (group_no++ & 1u) * (2 * NTOK * 16);
        for (int ti = 0; ti < gr.n; ti++) {
            const int64_t row0 = (int64_t)(ti ? gr.tile1 : gr.tile0) * TILE_ROWS;
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;
            // formats whose block rows are 16-byte multiples (Q4_K) start every row on a 16-byte boundary: no slack
            constexpr bool ALIGNED_ROWS = (UB % 16) == 0;
            const uint32_t slackA = ALIGNED_ROWS ? 0u : (uint32_t)(reinterpret_cast<uintptr_t>(W + (row0 + gid) * row_bytes) & 15u);
            const uint32_t slackB = ALIGNED_ROWS ? 0u : (uint32_t)(reinterpret_cast<uintptr_t>(W + (row0 + gid + 8) * row_bytes) & 15u);

            for (int it = 0; it < iters; it++, n++) {
                const uint32_t s = stage;
                if (ok) ok = mbar_wait(&full[s], phase, err);
                if (++stage == NUM_STAGES) stage = 0, phase ^= 1u;
                if (n == 0) { GTRC(2); }
                const int nun = min(STAGE_UNITS, units - it * STAGE_UNITS);
                if (ok && warp < nun) {
                    // slack of this stage's source address: the row start's slack plus the stage offset
                    const uint32_t stA = ALIGNED_ROWS ? 0u : (slackA + (uint32_t)((int64_t)it * STAGE_UNITS * UB)) & 15u;
                    const uint32_t stB = ALIGNED_ROWS ? 0u : (slackB + (uint32_t)((int64_t)it * STAGE_UNITS * UB)) & 15u;
                    const uint8_t* rA = stages + s * STAGE_BYTES + gid * ROW_STRIDE + stA + warp * UB;
                    const uint8_t* rB = stages + s * STAGE_BYTES + (gid + 8) * ROW_STRIDE + stB + warp * UB;
                    const int unit = it * STAGE_UNITS + warp;
                    if constexpr (QT == TSB_Q4_K)
                        q4k_block<NT>(reinterpret_cast<const uint4*>(rA), reinterpret_cast<const uint4*>(rB), la, unit, tig, acc);
                    if constexpr (QT == TSB_MXFP4) mxfp4_unit<NT>(rA, rB, act, units, unit, gid, tig, acc);
                    if constexpr (QT == TSB_Q6_K) q6k_block<NT>(rA, rB, act, units, unit, gid, tig, acc);
                    if constexpr (QT == TSB_Q5_K) q5k_block<NT>(rA, rB, act, units, unit, gid, tig, acc);
                    if constexpr (QT == TSB_Q8_0) q8_0_unit<NT>(rA, rB, act, units, unit, gid, tig, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }

            // ---- fixed-order reduction over the eight consumer warps into tile_out[ti].  Single-tile epilogues take the
            // two reduction buffers in turn (one barrier per tile); the paired ones park the first tile's partial sums
            // in buffer 0, the second's in buffer 1, and reduce both behind one pair of barriers.
            if (item == (int)blockIdx.x && ti == 0) { GTRC(3); }
            constexpr int RED_FLOATS = CONSUMER_WARPS * NT * 4 * 32;
            float* redb = red + (ELEMWISE ? (tile_no++ & 1u) : (uint32_t)ti) * RED_FLOATS;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) redb[((warp * NT + nt) * 4 + i) * 32 + lane] = acc[nt][i];
            if (!ELEMWISE && ti + 1 < gr.n) continue;  // the pair's second tile first
            epilogue_prefetch<EPI, NT>(epi, gr, rows, tokens, tok0);
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            for (int t2 = ELEMWISE ? ti : 0; t2 <= ti; t2++) {
                const float* rsrc = ELEMWISE ? redb : red + t2 * RED_FLOATS;
                for (int idx = threadIdx.x; idx < NTOK * 16; idx += CONSUMER_WARPS * 32) {
                    const int tok = idx >> 4, row = idx & 15;
                    const int nt = tok >> 3, nn = tok & 7;
                    const int src_lane = (row & 7) * 4 + (nn >> 1);
                    const int i = ((row >> 3) << 1) | (nn & 1);
                    float sum = 0.f;
#pragma unroll
                    for (int w = 0; w < CONSUMER_WARPS; w++) sum += rsrc[((w * NT + nt) * 4 + i) * 32 + src_lane];
                    tile_out[t2 * NTOK * 16 + idx] = sum;
                }
            }
            if constexpr (!ELEMWISE)
                asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");  // red reusable
        }
        if (!have_inv) {
            asm volatile("bar.sync 2, %0;" ::"n"(GEMM_THREADS) : "memory");  // 1/rms per token from the producer warp
            have_inv = true;
        }
        // (run_epilogue reads tile_out[idx] with the same idx -> thread mapping as the sum loop: no barrier between)
        if (item == (int)blockIdx.x) { GTRC(4); }
        if (ok) run_epilogue<EPI, NT>(epi, gr, tile_out, inv_rms, rows, tokens, tok0, err);
        if (item == (int)blockIdx.x) { GTRC(5); }
    }
    GTRC(6);
    if (!have_inv) asm volatile("bar.sync 2, %0;" ::"n"(GEMM_THREADS) : "memory");
}

#ifdef TSB_GEMM_TRACE
unsigned long long* g_gemm_trace = nullptr;
size_t g_gemm_trace_cap = 0, g_gemm_trace_used = 0;
#endif

template <int QT, int NT>
constexpr size_t gemm_smem_bytes() {
    return 64 + 256 + (size_t)2 * CONSUMER_WARPS * NT * 4 * 32 * sizeof(float) + (size_t)4 * NT * 8 * 16 * sizeof(float) +
           (size_t)NUM_STAGES * TILE_ROWS * row_stride_for(Fmt<QT>::UNIT_BYTES) + 128;
}

template <int QT, int NT, int EPI, bool GROUPED = false>
cudaError_t launch_one(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int units, ActOperand act, int tokens,
                       int tok0, const EpiArgs& args, const GroupedArgs& grp = GroupedArgs()) {
    auto kern = gemm_quant_kernel<QT, NT, EPI, GROUPED>;
    static SmemOptIn configured;  // per instantiation and per device
    constexpr size_t smem = gemm_smem_bytes<QT, NT>();
    if (cudaError_t e = tsb_opt_in_smem(ctx, kern, smem, configured); e != cudaSuccess) return e;
    const int n_tiles = (int)((rows + TILE_ROWS - 1) / TILE_ROWS);
    int groups = n_tiles;
    if (EPI == EPI_SILU || EPI == EPI_MOE_ACT) groups = n_tiles / 2;
    if (EPI == EPI_ROPE_STORE) {
        const int tph = args.head_dim / 16;
        groups = (args.n_q_heads + args.n_kv_heads) * (tph / 2) + (args.n_v_heads < 0 ? args.n_kv_heads : args.n_v_heads) * tph;
    }
    const int per_sm = gemm_ctas_per_sm<QT, NT>();
    if (GROUPED) groups *= grp.n_mats;
    dim3 grid((unsigned)min(groups, ctx->sm_count * per_sm));
#ifdef TSB_GEMM_TRACE
    GroupedArgs g2 = grp;
    if (g_gemm_trace && (g_gemm_trace_used + 1) * 2400 <= g_gemm_trace_cap) g2.trace = g_gemm_trace + (g_gemm_trace_used++) * 2400;
    return tsb_launch(ctx, kern, grid, dim3(GEMM_THREADS), smem, st, true, w, rows, units, act, tokens, tok0, args, ctx->dev_error, g2);
#else
    return tsb_launch(ctx, kern, grid, dim3(GEMM_THREADS), smem, st, true, w, rows, units, act, tokens, tok0, args, ctx->dev_error, grp);
#endif
}

// The matrices are binned by their row count, one launch per bin with the token-tile width that fits it: a matrix
// with three rows is not run through the 64-column variant because another one has forty.
template <int QT, int EPI>
cudaError_t launch_grouped_nt(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int units, ActOperand act, int max_tokens,
                              const EpiArgs& args, GroupedArgs grp) {
    cudaError_t e;
    grp.chunk0 = 0, grp.lo = 0, grp.hi = 8;
    if ((e = launch_one<QT, 1, EPI, true>(ctx, st, w, rows, units, act, 8, 0, args, grp)) != cudaSuccess || max_tokens <= 8) return e;
    grp.lo = 8, grp.hi = 16;
    if ((e = launch_one<QT, 2, EPI, true>(ctx, st, w, rows, units, act, 16, 0, args, grp)) != cudaSuccess || max_tokens <= 16) return e;
    grp.lo = 16, grp.hi = 32;
    if ((e = launch_one<QT, 4, EPI, true>(ctx, st, w, rows, units, act, 32, 0, args, grp)) != cudaSuccess || max_tokens <= 32) return e;
    grp.lo = 32, grp.hi = 0x7fffffff;
    for (int t0 = 0; t0 < max_tokens; t0 += 64) {
        grp.chunk0 = t0;
        if ((e = launch_one<QT, 8, EPI, true>(ctx, st, w, rows, units, act, 64, 0, args, grp)) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

template <int QT>
cudaError_t launch_grouped_epi(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int units, ActOperand act, int tokens,
                               int epi, const EpiArgs& args, const GroupedArgs& grp) {
    if (epi == EPI_MOE_ACT) return launch_grouped_nt<QT, EPI_MOE_ACT>(ctx, st, w, rows, units, act, tokens, args, grp);
    if (epi == EPI_PLAIN) return launch_grouped_nt<QT, EPI_PLAIN>(ctx, st, w, rows, units, act, tokens, args, grp);
    return cudaErrorInvalidValue;
}

template <int QT, int EPI>
cudaError_t launch_nt(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int units, ActOperand act, int tokens,
                      int tok0, const EpiArgs& args) {
    if (tokens <= 8) return launch_one<QT, 1, EPI>(ctx, st, w, rows, units, act, tokens, tok0, args);
    if (tokens <= 16) return launch_one<QT, 2, EPI>(ctx, st, w, rows, units, act, tokens, tok0, args);
    if (tokens <= 32) return launch_one<QT, 4, EPI>(ctx, st, w, rows, units, act, tokens, tok0, args);
    return launch_one<QT, 8, EPI>(ctx, st, w, rows, units, act, tokens, tok0, args);
}

template <int QT>
cudaError_t launch_epi(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int units, ActOperand act, int tokens,
                       int tok0, int epi, const EpiArgs& args) {
    switch (epi) {
        case EPI_PLAIN: return launch_nt<QT, EPI_PLAIN>(ctx, st, w, rows, units, act, tokens, tok0, args);
        case EPI_SCALE: return launch_nt<QT, EPI_SCALE>(ctx, st, w, rows, units, act, tokens, tok0, args);
        case EPI_RESID_NORM: return launch_nt<QT, EPI_RESID_NORM>(ctx, st, w, rows, units, act, tokens, tok0, args);
        case EPI_SILU: return launch_nt<QT, EPI_SILU>(ctx, st, w, rows, units, act, tokens, tok0, args);
        case EPI_MOE_ACT: return launch_nt<QT, EPI_MOE_ACT>(ctx, st, w, rows, units, act, tokens, tok0, args);
        case EPI_ROPE_STORE: return launch_nt<QT, EPI_ROPE_STORE>(ctx, st, w, rows, units, act, tokens, tok0, args);
        default: return cudaErrorInvalidValue;
    }
}

// x natural -> fragment-major operand + 16-column sums
__global__ void act_prepare_kernel(const __half* __restrict__ x, int64_t x_stride, const int32_t* __restrict__ src_rows, int tokens,
                                   int cols, uint4* __restrict__ xp, uint4* __restrict__ xs) {
    pdl_wait();
    const int per_row = cols >> 3;
    const int padded = ((tokens + 7) >> 3) << 3;  // slots of the last tile are zero-filled
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = idx < (int64_t)padded * per_row;
    const int t = active ? (int)(idx / per_row) : 0;
    const int e0 = active ? (int)(idx % per_row) * 8 : 0;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = 0.f;
    if (active && t < tokens) {
        const int src = src_rows ? src_rows[t] : t;
        if (src >= 0) {  // a negative source row is a padding slot: zeros
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)src * x_stride + e0);
            const __half* hp = reinterpret_cast<const __half*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __half2float(hp[i]);
        }
    }
    pdl_launch_dependents();
    act_store8(v, xp, xs, t, e0, cols >> 8, active);
}

}  // namespace

cudaError_t launch_act_prepare(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, int tokens, int cols,
                               uint4* xp, uint4* xs) {
    const int64_t n = (int64_t)act_tiles(tokens) * 8 * (cols / 8);
    const int threads = 256;  // even, and cols/8 is even, so the 16-column pairs never straddle rows
    return tsb_launch(ctx, act_prepare_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, st, true,
                      x, x_stride, (const int32_t*)nullptr, tokens, cols, xp, xs);
}

cudaError_t launch_act_prepare_gather(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, const int32_t* src_rows,
                                      int tokens, int cols, uint4* xp, uint4* xs) {
    const int64_t n = (int64_t)act_tiles(tokens) * 8 * (cols / 8);
    const int threads = 256;
    return tsb_launch(ctx, act_prepare_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, st, true,
                      x, x_stride, src_rows, tokens, cols, xp, xs);
}

cudaError_t launch_gemm_fused(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, int tokens, int epi, const EpiArgs& args) {
    const int units = (int)(cols / 256);
    // more than 64 tokens: passes of 64 (each pass re-streams the weights)
    for (int t0 = 0; t0 < tokens; t0 += 64) {
        const int nt = min(64, tokens - t0);
        ActOperand a = {act.xp + (size_t)(t0 / 8) * units * 256, act.xs + (size_t)(t0 / 8) * units * 32};
        cudaError_t e;
        switch (qtype) {
            case TSB_Q4_K: e = launch_epi<TSB_Q4_K>(ctx, st, w, rows, units, a, nt, t0, epi, args); break;
            case TSB_Q6_K: e = launch_epi<TSB_Q6_K>(ctx, st, w, rows, units, a, nt, t0, epi, args); break;
            case TSB_MXFP4: e = launch_epi<TSB_MXFP4>(ctx, st, w, rows, units, a, nt, t0, epi, args); break;
            case TSB_Q5_K: e = launch_epi<TSB_Q5_K>(ctx, st, w, rows, units, a, nt, t0, epi, args); break;
            case TSB_Q8_0: e = launch_epi<TSB_Q8_0>(ctx, st, w, rows, units, a, nt, t0, epi, args); break;
            default: return cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t launch_gemm_grouped(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t w_stride, int n_mats,
                                int64_t rows, int64_t cols, ActOperand act, const int32_t* count, const int32_t* tile_start,
                                int max_tokens, int epi, const EpiArgs& args) {
    const int units = (int)(cols / 256);
    GroupedArgs grp;
    grp.count = count, grp.tile_start = tile_start, grp.n_mats = n_mats, grp.w_stride = w_stride;
    switch (qtype) {
        case TSB_Q4_K: return launch_grouped_epi<TSB_Q4_K>(ctx, st, w, rows, units, act, max_tokens, epi, args, grp);
        case TSB_Q6_K: return launch_grouped_epi<TSB_Q6_K>(ctx, st, w, rows, units, act, max_tokens, epi, args, grp);
        case TSB_MXFP4: return launch_grouped_epi<TSB_MXFP4>(ctx, st, w, rows, units, act, max_tokens, epi, args, grp);
        case TSB_Q5_K: return launch_grouped_epi<TSB_Q5_K>(ctx, st, w, rows, units, act, max_tokens, epi, args, grp);
        case TSB_Q8_0: return launch_grouped_epi<TSB_Q8_0>(ctx, st, w, rows, units, act, max_tokens, epi, args, grp);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemm_quant(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, void* y, int64_t y_stride, int tokens, bool y_f32) {
    EpiArgs a;
    a.y = y, a.y_stride = y_stride, a.y_f32 = y_f32 ? 1 : 0;
    return launch_gemm_fused(ctx, st, qtype, w, rows, cols, act, tokens, EPI_PLAIN, a);
}

// 24 token rows and more of a supported matrix dequantise every weight once per 128-row tile on the tensor-memory path
static bool gemm_takes_wide(int qtype, int64_t rows, int64_t cols, int tokens) {
    static int wide_min = -1;
    if (wide_min < 0) {
        const char* env = getenv("TSB_WIDE_MIN");
        wide_min = env ? atoi(env) : 24;
    }
    return tokens >= wide_min && gemm_wide_supported(qtype, rows, cols, tokens);
}

// ------------------------------------------------------------------ C ABI
extern "C" {
#ifdef TSB_GEMM_TRACE
__attribute__((visibility("default"))) void tsb_debug_set_gemm_trace(void* p, size_t n_u64) {
    g_gemm_trace = static_cast<unsigned long long*>(p), g_gemm_trace_cap = n_u64, g_gemm_trace_used = 0;
}
#endif

int32_t tsb_gemm_quant(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off, int64_t rows,
                       int64_t cols, const void* x_f16, void* y, int32_t tokens, int32_t y_f32) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, region && x_f16 && y, "null buffer");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST, "unknown block format %d", qtype);
    TSB_REQUIRE(ctx, rows > 0 && cols > 0 && tokens > 0, "rows, cols and tokens must be positive");
    if (cols % 256 != 0)
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED,
                        "cols (%lld) is not a whole number of 256-element superblocks", (long long)cols);
    TSB_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_f16) & 15u) == 0, "x must be 16-byte aligned");
    if (qtype == TSB_Q4_K || qtype == TSB_Q5_K || qtype == TSB_Q8_0)  // formats whose 256-column units are 16-byte multiples
        TSB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(region) + w_off) & 15u) == 0, "rows of this format must start on a 16-byte boundary");
    if (qtype == TSB_MXFP4)  // the resident file aligns every tensor to 4 bytes (crates/repack/src/resident_writer.rs:401-405)
        TSB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(region) + w_off) & 3u) == 0, "MXFP4 rows must start on a 4-byte boundary");
    DeviceGuard g(ctx);
    cudaStream_t st = (cudaStream_t)s;
    if (gemm_takes_wide(qtype, rows, cols, tokens)) {  // many token rows: the tensor-memory path
        TSB_CUDA(ctx, launch_gemm_wide_q4k(ctx, st, static_cast<const uint8_t*>(region) + w_off, rows, cols, (const __half*)x_f16, cols,
                                           tokens, y, rows, y_f32 != 0));
        return TSB_OK;
    }
    const size_t xp_bytes = (act_xp_bytes(tokens, cols) + 255) & ~(size_t)255;
    uint8_t* tmp = nullptr;
    TSB_CUDA(ctx, cudaMallocAsync((void**)&tmp, xp_bytes + act_xs_bytes(tokens, cols), st));
    uint4* xp = reinterpret_cast<uint4*>(tmp);
    uint4* xs = reinterpret_cast<uint4*>(tmp + xp_bytes);
    cudaError_t e = launch_act_prepare(ctx, st, (const __half*)x_f16, cols, tokens, (int)cols, xp, xs);
    if (e == cudaSuccess)
        e = launch_gemm_quant(ctx, st, qtype, (const uint8_t*)region + w_off, rows, cols, ActOperand{xp, xs}, y,
                              rows, tokens, y_f32 != 0);
    cudaError_t e2 = cudaFreeAsync(tmp, st);
    TSB_CUDA(ctx, e);
    TSB_CUDA(ctx, e2);
    return TSB_OK;
}

// ---- the same operator with the caller's workspace: no allocation, and the operand conversion on its own
// the operand copy of the many-row path, 256-byte aligned, then its partial sums (sized for the current device)
static size_t wide_operand_bytes(int64_t cols, int tokens) { return (gemm_wide_workspace_bytes(cols, tokens) + 255) & ~(size_t)255; }

size_t tsb_gemm_workspace_bytes(int32_t qtype, int64_t rows, int64_t cols, int32_t tokens) {
    if (tokens <= 0 || cols <= 0 || cols % 256 != 0) return 0;
    if (gemm_takes_wide(qtype, rows, cols, tokens)) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
        return wide_operand_bytes(cols, tokens) + gemm_wide_partial_bytes_for(sms, rows, cols) + 256;
    }
    return ((act_xp_bytes(tokens, cols) + 255) & ~(size_t)255) + act_xs_bytes(tokens, cols) + 256;
}

int32_t tsb_gemm_prepare(tsb_ctx* ctx, tsb_stream s, int32_t qtype, int64_t rows, int64_t cols, const void* x_f16, int32_t tokens,
                         void* workspace, size_t workspace_bytes) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, x_f16 && workspace, "null buffer");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST && rows > 0 && cols > 0 && cols % 256 == 0 && tokens > 0, "bad shape or format");
    TSB_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_f16) & 15u) == 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, "x must be 16-byte, the workspace 256-byte aligned");
    TSB_REQUIRE(ctx, workspace_bytes >= tsb_gemm_workspace_bytes(qtype, rows, cols, tokens), "workspace too small");
    DeviceGuard g(ctx);
    if (gemm_takes_wide(qtype, rows, cols, tokens)) {
        // that path converts inside its own launch sequence; the ticket words of its partial sums start at zero
        if (gemm_wide_partial_bytes(ctx, rows, cols) > 0)
            TSB_CUDA(ctx, cudaMemsetAsync(static_cast<uint8_t*>(workspace) + wide_operand_bytes(cols, tokens), 0, 4096, (cudaStream_t)s));
        return TSB_OK;
    }
    const size_t xp_bytes = (act_xp_bytes(tokens, cols) + 255) & ~(size_t)255;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    TSB_CUDA(ctx, launch_act_prepare(ctx, (cudaStream_t)s, (const __half*)x_f16, cols, tokens, (int)cols, reinterpret_cast<uint4*>(ws),
                                     reinterpret_cast<uint4*>(ws + xp_bytes)));
    return TSB_OK;
}

int32_t tsb_gemm_quant_prepared(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off, int64_t rows, int64_t cols,
                                const void* x_f16, void* workspace, void* y, int32_t tokens, int32_t y_f32) {
    if (!ctx) return TSB_ERR_INVALID;
    TSB_REQUIRE(ctx, region && x_f16 && workspace && y, "null buffer");
    TSB_REQUIRE(ctx, qtype >= TSB_Q4_K && qtype <= TSB_QTYPE_LAST && rows > 0 && cols > 0 && cols % 256 == 0 && tokens > 0, "bad shape or format");
    if (qtype == TSB_Q4_K || qtype == TSB_Q5_K || qtype == TSB_Q8_0)
        TSB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(region) + w_off) & 15u) == 0, "rows of this format must start on a 16-byte boundary");
    if (qtype == TSB_MXFP4) TSB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(region) + w_off) & 3u) == 0, "MXFP4 rows must start on a 4-byte boundary");
    DeviceGuard g(ctx);
    cudaStream_t st = (cudaStream_t)s;
    const uint8_t* w = static_cast<const uint8_t*>(region) + w_off;
    if (gemm_takes_wide(qtype, rows, cols, tokens)) {
        const bool cut = gemm_wide_partial_bytes(ctx, rows, cols) > 0;
        TSB_CUDA(ctx, launch_gemm_wide_q4k(ctx, st, w, rows, cols, (const __half*)x_f16, cols, tokens, y, rows, y_f32 != 0, workspace,
                                           cut ? static_cast<uint8_t*>(workspace) + wide_operand_bytes(cols, tokens) : nullptr));
        return TSB_OK;
    }
    const size_t xp_bytes = (act_xp_bytes(tokens, cols) + 255) & ~(size_t)255;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    TSB_CUDA(ctx, launch_gemm_quant(ctx, st, qtype, w, rows, cols, ActOperand{reinterpret_cast<uint4*>(ws), reinterpret_cast<uint4*>(ws + xp_bytes)}, y,
                                    rows, tokens, y_f32 != 0));
    return TSB_OK;
}

int32_t tsb_gemv_q4k(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                     void* y) {
    return tsb_gemm_quant(c, s, TSB_Q4_K, r, o, rows, cols, x, y, 1, 0);
}
int32_t tsb_gemv_q6k(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                     void* y) {
    return tsb_gemm_quant(c, s, TSB_Q6_K, r, o, rows, cols, x, y, 1, 0);
}
int32_t tsb_gemv_mxfp4(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                       void* y) {
    return tsb_gemm_quant(c, s, TSB_MXFP4, r, o, rows, cols, x, y, 1, 0);
}
int32_t tsb_gemm_q4k(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                     void* y, int32_t t) {
    return tsb_gemm_quant(c, s, TSB_Q4_K, r, o, rows, cols, x, y, t, 0);
}
int32_t tsb_gemm_q6k(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                     void* y, int32_t t) {
    return tsb_gemm_quant(c, s, TSB_Q6_K, r, o, rows, cols, x, y, t, 0);
}
int32_t tsb_gemm_mxfp4(tsb_ctx* c, tsb_stream s, const void* r, uint64_t o, int64_t rows, int64_t cols, const void* x,
                       void* y, int32_t t) {
    return tsb_gemm_quant(c, s, TSB_MXFP4, r, o, rows, cols, x, y, t, 0);
}

}  // extern "C"
