// A chain of dependent quantized matmuls as ONE cooperative launch.
//
// A decoder layer's matmuls (o_proj -> gate|up -> down -> the next layer's q|k|v, or the head) are a few megabytes
// each: launched one by one, every kernel pays its own ramp-up, tail and launch gap, and the weight stream stops at
// each boundary.  Here the same persistent CTAs walk the phases of the chain in order.  The producer warp of a CTA
// knows the whole schedule in advance (weights are static), so its bulk-copy ring runs straight through the phase
// boundaries: while the consumer warps sit in a grid-wide barrier, the next phase's blocks are already landing in
// shared memory.  Consumers synchronise between phases with an arrival counter in global memory (all CTAs are
// co-resident: the launch is cooperative), after which the previous phase's outputs - written by other CTAs of this
// launch - are read with plain (coherent) loads.
//
// The arithmetic of every phase is the stand-alone matmul kernel's: the same block routine, the same fixed-order
// reduction over the eight consumer warps, the same epilogues.  A chain therefore gives bit-identical results to
// the same matmuls launched separately.
//
// A chain may start with the merge of the attention kernel's split-KV partials (phase kind MERGE): every
// (row, head) is finished by one half-warp somewhere in the grid, which spreads what used to be a serial tail of
// the attention kernel over all SMs.
#include "gemm_blocks.cuh"
#include "gemm_fused.cuh"

namespace {

constexpr int UB = Fmt<TSB_Q4_K>::UNIT_BYTES;
constexpr int ROW_STRIDE = row_stride_for(UB);
constexpr int STAGE_BYTES = TILE_ROWS * ROW_STRIDE;

// Wait on a ring barrier; gives up when the CTA's abort flag is up or the time bound runs out.
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity, uint32_t* state, volatile int* abort_flag) {
    unsigned long long t0 = 0, limit_ns = 0;
    for (uint32_t i = 1;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                const uint32_t us = *reinterpret_cast<volatile uint32_t*>(state + 1);
                limit_ns = (unsigned long long)(us ? us : 1000000u) * 1000ull;
            } else if (now - t0 > limit_ns) {
                break;
            }
        }
    }
    atomicCAS(state, 0u, (uint32_t)TSB_DEV_BARRIER_TIMEOUT);
    return false;
}

// Grid-wide barrier, called by ONE thread per CTA after the CTA's own threads have met.  The counter only grows:
// arrival number `old` belongs to barrier old / per_barrier, so no reset is needed between barriers or launches
// (every launch adds a whole number of barriers; the host zeroes the counter after a failed launch).
__device__ __forceinline__ bool grid_arrive_and_wait(uint32_t* state, unsigned arrive_inc, unsigned per_barrier) {
    unsigned long long* ctr = reinterpret_cast<unsigned long long*>(state + 2);
    __threadfence();
    const unsigned long long old = atomicAdd(ctr, (unsigned long long)arrive_inc);
    const unsigned long long target = (old / per_barrier + 1ull) * per_barrier;
    unsigned long long t0 = 0, limit_ns = 0;
    for (uint32_t i = 1;; i++) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
        if (v >= target) break;
        if ((i & 15u) == 0) {
            if (*reinterpret_cast<volatile uint32_t*>(state) != 0u) return false;  // somebody else gave up
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                const uint32_t us = *reinterpret_cast<volatile uint32_t*>(state + 1);
                limit_ns = (unsigned long long)(us ? us : 1000000u) * 1000ull;
            } else if (now - t0 > limit_ns) {
                atomicCAS(state, 0u, (uint32_t)TSB_DEV_BARRIER_TIMEOUT);
                return false;
            }
        }
    }
    __threadfence();
    return true;
}

struct Ring {
    uint64_t* full;
    uint64_t* empty;
    uint8_t* stages;
    uint32_t n;  // stages issued (producer) / consumed (consumers) so far, across phases
};

// ---- producer side of one matmul phase: the bulk copies of this CTA's row tiles, in the consumers' order
template <int EPI>
__device__ __forceinline__ bool produce_phase(const FusedPhase& ph, Ring& ring, uint32_t* state, volatile int* abort_flag, int lane) {
    const int64_t rows = ph.rows;
    const int units = ph.units;
    const int n_tiles = (int)((rows + TILE_ROWS - 1) / TILE_ROWS);
    const int n_groups = num_groups<EPI>(n_tiles, ph.e);
    const int iters = (units + STAGE_UNITS - 1) / STAGE_UNITS;
    const int64_t row_bytes = (int64_t)units * UB;
    for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const Group gr = group_of<EPI>(g, n_tiles, ph.e);
        for (int ti = 0; ti < gr.n; ti++) {
            const int64_t row0 = (int64_t)(ti ? gr.tile1 : gr.tile0) * TILE_ROWS;
            const int nrows = (int)min((int64_t)TILE_ROWS, rows - row0);
            for (int it = 0; it < iters; it++, ring.n++) {
                const uint32_t s = ring.n % NUM_STAGES;
                if (ring.n >= NUM_STAGES && !ring_wait(&ring.empty[s], ((ring.n / NUM_STAGES) - 1) & 1, state, abort_flag)) return false;
                const int nun = min(STAGE_UNITS, units - it * STAGE_UNITS);
                const uint32_t bytes = lane < nrows ? (uint32_t)nun * UB : 0u;  // Q4_K rows are 16-byte multiples: no slack
                uint32_t total = bytes;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                if (lane == 0) mbar_expect_tx(&ring.full[s], total);
                __syncwarp();
                if (lane < nrows)
                    bulk_g2s(ring.stages + s * STAGE_BYTES + lane * ROW_STRIDE, ph.w + (row0 + lane) * row_bytes + (int64_t)it * STAGE_UNITS * UB,
                             bytes, &ring.full[s]);
            }
        }
    }
    return true;
}

// ---- consumer side of one matmul phase
template <int NT, int EPI>
__device__ __forceinline__ bool consume_phase(const FusedPhase& ph, int tokens, Ring& ring, float* inv_rms, float* red, float* tile_out0,
                                              uint32_t& tile_no, uint32_t& group_no, uint32_t* state, volatile int* abort_flag) {
    constexpr int NTOK = NT * 8;
    constexpr bool ELEMWISE = EPI == EPI_PLAIN || EPI == EPI_SCALE;
    constexpr bool NEEDS_INV = EPI == EPI_SCALE || EPI == EPI_SILU || EPI == EPI_ROPE_STORE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tig = lane & 3;
    const int64_t rows = ph.rows;
    const int units = ph.units;
    const int n_tiles = (int)((rows + TILE_ROWS - 1) / TILE_ROWS);
    const int n_groups = num_groups<EPI>(n_tiles, ph.e);
    const int iters = (units + STAGE_UNITS - 1) / STAGE_UNITS;
    const EpiArgs& epi = ph.e;

    if constexpr (NEEDS_INV) {
        // 1/rms per token from the partial sums of x^2 the producing phase left (same order of additions as the
        // stand-alone kernel: a lane-strided pass, then a butterfly)
        for (int t = warp; t < tokens; t += CONSUMER_WARPS) {
            float sacc = 0.f;
            for (int i = lane; i < epi.ss_parts; i += 32) sacc += *reinterpret_cast<const volatile float*>(&epi.ss_in[(size_t)t * epi.ss_parts + i]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
            if (lane == 0) inv_rms[t] = 1.0f / sqrtf(sacc / (float)epi.d_in + epi.eps);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
    }

    LaneAct<NT> la;
    la.nblk = units;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        la.xp[nt] = ph.act.xp + (size_t)nt * units * 256 + lane;
        la.xs[nt] = ph.act.xs + (size_t)nt * units * 32 + lane;
    }
    bool ok = true;
    for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const Group gr = group_of<EPI>(g, n_tiles, epi);
        float* tile_out = tile_out0 + (group_no++ & 1u) * (2 * NTOK * 16);
        for (int ti = 0; ti < gr.n; ti++) {
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;
            for (int it = 0; it < iters; it++, ring.n++) {
                const uint32_t s = ring.n % NUM_STAGES;
                if (ok) ok = ring_wait(&ring.full[s], (ring.n / NUM_STAGES) & 1, state, abort_flag);
                const int nun = min(STAGE_UNITS, units - it * STAGE_UNITS);
                if (ok && warp < nun) {
                    const int gid = lane >> 2;
                    const uint8_t* rA = ring.stages + s * STAGE_BYTES + gid * ROW_STRIDE + warp * UB;
                    const uint8_t* rB = ring.stages + s * STAGE_BYTES + (gid + 8) * ROW_STRIDE + warp * UB;
                    q4k_block<NT, false>(reinterpret_cast<const uint4*>(rA), reinterpret_cast<const uint4*>(rB), la, it * STAGE_UNITS + warp, tig, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&ring.empty[s]);
            }
            constexpr int RED_FLOATS = CONSUMER_WARPS * NT * 4 * 32;
            float* redb = red + (ELEMWISE ? (tile_no++ & 1u) : (uint32_t)ti) * RED_FLOATS;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) redb[((warp * NT + nt) * 4 + i) * 32 + lane] = acc[nt][i];
            if (!ELEMWISE && ti + 1 < gr.n) continue;
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
            if constexpr (!ELEMWISE) asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
        }
        if (ok) run_epilogue<EPI, NT>(epi, gr, tile_out, inv_rms, rows, tokens, 0, state);
    }
    return ok;
}

// ---- merge of the attention kernel's split-KV partials into the o_proj operand
// out = sum_c O_c 2^(m_c - m) / sum_c l_c 2^(m_c - m), splits in order (crates/gpu/src/shaders/attention.metal:983-1031).
// hd / 8 neighbouring threads finish one (row, head); each owns eight columns.
__device__ __forceinline__ void merge_phase(const MergeArgs& mg) {
    const int lpi = mg.head_dim >> 3;  // threads per (row, head)
    const int gthreads = gridDim.x * CONSUMER_WARPS * 32;
    const int n_items = mg.rows * mg.n_q_heads;
    const int gtid = blockIdx.x * (CONSUMER_WARPS * 32) + threadIdx.x;
    const int part = gtid % lpi;
    for (int base = 0; base < n_items; base += gthreads / lpi) {  // uniform trip count
        const int item = base + gtid / lpi;
        const bool active = item < n_items;
        float m = -INFINITY, den = 0.f, accv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] = 0.f;
        if (active) {
            const size_t pi = (size_t)item * mg.n_splits;
            for (int c = 0; c < mg.n_splits; c++) m = fmaxf(m, __ldcg(&mg.part_ml[pi + c]).x);
            const float mu = (m == -INFINITY) ? 0.f : m;
#pragma unroll 4
            for (int c = 0; c < mg.n_splits; c++) {
                const float2 v = __ldcg(&mg.part_ml[pi + c]);
                const float wgt = exp2f(v.x - mu);
                den += v.y * wgt;
                const float4* po = reinterpret_cast<const float4*>(mg.part_o + (pi + c) * mg.head_dim + part * 8);
                const float4 a = __ldcg(po), b2 = __ldcg(po + 1);
                accv[0] += a.x * wgt, accv[1] += a.y * wgt, accv[2] += a.z * wgt, accv[3] += a.w * wgt;
                accv[4] += b2.x * wgt, accv[5] += b2.y * wgt, accv[6] += b2.z * wgt, accv[7] += b2.w * wgt;
            }
        }
        const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) accv[i] *= inv;
        const int row = active ? item / mg.n_q_heads : 0, head = active ? item % mg.n_q_heads : 0;
        act_store8(accv, mg.out.xp, mg.out.xs, row, head * mg.head_dim + part * 8, (mg.n_q_heads * mg.head_dim) >> 8, active);
    }
}

template <int NT>
__global__ void __launch_bounds__(GEMM_THREADS, (NT <= 2 ? 2 : 1)) fused_chain_kernel(const __grid_constant__ FusedArgs a) {
    constexpr int NTOK = NT * 8;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + NUM_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 48);  // a wait gave up: everybody drains and leaves
    volatile uint32_t* prod_n = reinterpret_cast<volatile uint32_t*>(smem + 52);  // stages the producer issued, valid once prod_done
    volatile int* prod_done = reinterpret_cast<volatile int*>(smem + 56);
    float* inv_rms = reinterpret_cast<float*>(smem + 64);
    float* red = reinterpret_cast<float*>(smem + 64 + 256);
    float* tile_out0 = red + 2 * CONSUMER_WARPS * NT * 4 * 32;
    uint8_t* stages = reinterpret_cast<uint8_t*>(tile_out0 + 4 * NTOK * 16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NUM_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_fence_init();
        *abort_flag = 0;
        *prod_done = 0;
    }
    __syncthreads();
    Ring ring{full, empty, stages, 0u};
    uint32_t* state = a.state;

    if (warp == CONSUMER_WARPS) {
        // ---- producer: every matmul phase's copies back to back; it never waits for a grid barrier
        bool ok = true;
        for (int p = 0; p < a.n_phases && ok; p++) {
            const FusedPhase& ph = a.ph[p];
            if (ph.kind != FUSED_GEMM) continue;
            switch (ph.epi) {
                case EPI_RESID_NORM: ok = produce_phase<EPI_RESID_NORM>(ph, ring, state, abort_flag, lane); break;
                case EPI_SILU: ok = produce_phase<EPI_SILU>(ph, ring, state, abort_flag, lane); break;
                case EPI_ROPE_STORE: ok = produce_phase<EPI_ROPE_STORE>(ph, ring, state, abort_flag, lane); break;
                default: ok = produce_phase<EPI_SCALE>(ph, ring, state, abort_flag, lane); break;
            }
        }
        if (lane == 0) {
            *prod_n = ring.n;
            __threadfence_block();
            *prod_done = 1;
        }
        return;
    }
    // After a wait gave up the consumers stop reading the ring, but copies the producer issued still land in this
    // CTA's shared memory: one thread waits (bounded) for the producer to stop and for its last copies to arrive.
    auto drain = [&]() {
        if (threadIdx.x != 0) return;
        for (uint32_t i = 0; i < (1u << 24) && !*prod_done; i++) {}
        if (!*prod_done) return;
        const uint32_t n = *prod_n;
        for (uint32_t k = 1; k <= NUM_STAGES && k <= n; k++) {
            const uint32_t f = n - k;
            for (uint32_t i = 0; i < (1u << 22) && !mbar_try_wait(&full[f % NUM_STAGES], (f / NUM_STAGES) & 1); i++) {}
        }
    };

    // ---- consumers
    uint32_t tile_no = 0, group_no = 0;
    bool ok = true;
    for (int p = 0; p < a.n_phases; p++) {
        const FusedPhase& ph = a.ph[p];
        if (p > 0) {
            // everything this CTA wrote in the previous phase is ordered before thread 0's arrival; after the barrier
            // the other CTAs' writes are visible to plain loads.  A ring wait that gave up in any warp (the error
            // word is set) turns into the CTA-wide abort flag here, so all warps leave together.
            if (!ok) *abort_flag = 1;
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            if (threadIdx.x == 0 && !*abort_flag && !grid_arrive_and_wait(state, a.arrive_inc, a.per_barrier)) *abort_flag = 1;
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            if (*abort_flag) {
                drain();
                return;
            }
        }
        if (ph.kind == FUSED_MERGE) {
            merge_phase(a.merge);
            continue;
        }
        switch (ph.epi) {
            case EPI_RESID_NORM: ok = consume_phase<NT, EPI_RESID_NORM>(ph, a.tokens, ring, inv_rms, red, tile_out0, tile_no, group_no, state, abort_flag); break;
            case EPI_SILU: ok = consume_phase<NT, EPI_SILU>(ph, a.tokens, ring, inv_rms, red, tile_out0, tile_no, group_no, state, abort_flag); break;
            case EPI_ROPE_STORE: ok = consume_phase<NT, EPI_ROPE_STORE>(ph, a.tokens, ring, inv_rms, red, tile_out0, tile_no, group_no, state, abort_flag); break;
            default: ok = consume_phase<NT, EPI_SCALE>(ph, a.tokens, ring, inv_rms, red, tile_out0, tile_no, group_no, state, abort_flag); break;
        }
    }
    if (!ok) *abort_flag = 1;
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
    if (*abort_flag) drain();
}

template <int NT>
constexpr size_t fused_smem_bytes() {
    return 64 + 256 + (size_t)2 * CONSUMER_WARPS * NT * 4 * 32 * sizeof(float) + (size_t)4 * NT * 8 * 16 * sizeof(float) +
           (size_t)NUM_STAGES * STAGE_BYTES + 128;
}

template <int NT>
cudaError_t launch_chain_nt(tsb_ctx* ctx, cudaStream_t st, FusedArgs& args) {
    auto kern = fused_chain_kernel<NT>;
    static SmemOptIn configured;
    static int per_sm[TSB_MAX_DEVICES] = {};
    constexpr size_t smem = fused_smem_bytes<NT>();
    if (cudaError_t e = tsb_opt_in_smem(ctx, kern, smem, configured); e != cudaSuccess) return e;
    const int dev = ctx->device;
    if (dev < 0 || dev >= TSB_MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!per_sm[dev]) {
        int n = 0;
        if (cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, GEMM_THREADS, smem); e != cudaSuccess) return e;
        per_sm[dev] = n > 0 ? n : -1;
    }
    if (per_sm[dev] < 1) return cudaErrorLaunchOutOfResources;
    // one or two CTAs per SM; the arrival increment keeps one barrier = 2 * sm_count counts whatever the grid
    const int want = NT <= 2 ? 2 : 1;
    const int per = per_sm[dev] >= want ? want : 1;
    args.arrive_inc = (unsigned)(2 / per);
    args.per_barrier = (unsigned)(2 * ctx->sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ctx->sm_count * per));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ctx->launches++;
    return cudaLaunchKernelEx(&cfg, kern, args);
}

}  // namespace

bool gemm_chain_supported(int qtype, int64_t rows, int64_t cols, int tokens) {
    return qtype == TSB_Q4_K && rows > 0 && cols > 0 && cols % 256 == 0 && tokens >= 1 && tokens <= 64;
}

cudaError_t launch_gemm_chain(tsb_ctx* ctx, cudaStream_t st, FusedArgs& args) {
    if (args.n_phases < 1 || args.n_phases > FUSED_MAX_PHASES || args.tokens < 1 || args.tokens > 64) return cudaErrorInvalidValue;
    args.state = ctx->dev_error;
    if (args.tokens <= 8) return launch_chain_nt<1>(ctx, st, args);
    if (args.tokens <= 16) return launch_chain_nt<2>(ctx, st, args);
    if (args.tokens <= 32) return launch_chain_nt<4>(ctx, st, args);
    return launch_chain_nt<8>(ctx, st, args);
}
