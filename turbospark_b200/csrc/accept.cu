// Rejection-sampling acceptance on the device.
//
// What it replaces: the host-side accept step of the reference's round loop
// (crates/runtime/src/speculative.rs:694-754,861-879) together with the f64
// sampler it calls (crates/selection/src/choose.rs:111-321, distribution.rs:57-125).
// The reference shapes every row into an explicit distribution in RANK order
// (probability descending, ties by ascending index) and walks cumulative sums
// in that order; everything is f64, summed sequentially.  This kernel keeps the
// arithmetic in f64 and the order semantics, but replaces the sort + sequential
// walk by an order-preserving radix descent over the logit keys with exact
// integer (2^-60 fixed point) bin masses, so the result does not depend on
// thread scheduling.  Decisions (accept / reject, drawn token) equal the
// reference's unless a uniform lies within ~1e-13 of a decision boundary; the
// distances to the nearest boundary are returned so such a case is visible.
//
// Shaping covered here: temperature (including 0 = argmax), whole vocabulary
// (top_k = 0, top_p off, min_p off), no penalties.
//
// Kernel 1 (one CTA per logits row): max, first argmax, sum = sum_i exp(l_i - max)
// and total = sum_i w_i with w_i = ((e_i / sum) / top)^(1/T).
// Kernel 2 (one CTA per stream): the accept chain on thread 0, then the one draw
// the round needs (residual, or bonus from the last row) by the whole CTA.
#include "accept.cuh"

namespace {

constexpr int ACC_THREADS = 1024;
constexpr int NBINS = 2048;

struct RowStats {
    float max;
    int32_t argmax;
    double sum;
    double total;
    int32_t nonfinite;
    int32_t _pad;
};

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
    // fixed shape: lane tree, then warps in index order
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < ACC_THREADS / 32; i++) t += red[i];
    return t;
}

__device__ __forceinline__ uint32_t desc_key(float x) {
    // ascending unsigned order of ~key == descending order of x
    uint32_t u = __float_as_uint(x);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ~u;
}

// w_i of reweight (choose.rs:296-321): ((e/sum)/top)^(1/T), top = max_i e_i/sum = 1/sum.
__device__ __forceinline__ double weight_of(double e, double sum, double top, double inv_t, bool unit_t) {
    const double p = e / sum;
    const double r = top > 0.0 ? p / top : p;
    return unit_t ? r : pow(r, inv_t);
}

__global__ void __launch_bounds__(ACC_THREADS)
    accept_stats_kernel(const __half* __restrict__ target, const __half* __restrict__ draft, int k, int vocab,
                        double temperature, RowStats* __restrict__ stats, int rows_per_stream, int64_t single_stride) {
    __shared__ double red[ACC_THREADS / 32];
    __shared__ float fred[ACC_THREADS / 32];
    __shared__ int ired[ACC_THREADS / 32];
    __shared__ int nf_flag;
    pdl_wait();
    const int b = blockIdx.x / rows_per_stream, r = blockIdx.x % rows_per_stream;
    // rows 0..k are the target's, k+1..2k the drafter's
    // single_stride != 0: one row per stream, `single_stride` elements apart (the draft-side draw)
    const __half* row = single_stride ? target + (size_t)b * single_stride
                        : (r <= k)    ? target + ((size_t)b * (k + 1) + r) * vocab
                                      : draft + ((size_t)b * k + (r - k - 1)) * vocab;
    if (threadIdx.x == 0) nf_flag = 0;
    __syncthreads();
    // pass A: max and first argmax, finiteness
    float mx = -INFINITY;
    int am = 0x7fffffff;
    bool bad = false;
    for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) {
        const float v = __half2float(row[i]);
        bad |= !isfinite(v);
        if (v > mx || (v == mx && i < am)) mx = v, am = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oam = __shfl_xor_sync(0xffffffffu, am, o);
        if (omx > mx || (omx == mx && oam < am)) mx = omx, am = oam;
    }
    if (bad) nf_flag = 1;
    if ((threadIdx.x & 31) == 0) fred[threadIdx.x >> 5] = mx, ired[threadIdx.x >> 5] = am;
    __syncthreads();
    mx = fred[0], am = ired[0];
    for (int i = 1; i < ACC_THREADS / 32; i++)
        if (fred[i] > mx || (fred[i] == mx && ired[i] < am)) mx = fred[i], am = ired[i];
    RowStats st;
    st.max = mx, st.argmax = am, st.sum = 1.0, st.total = 1.0, st.nonfinite = nf_flag, st._pad = 0;
    if (temperature != 0.0 && !nf_flag) {
        const double dmx = (double)mx;
        double s = 0.0;
        for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) s += exp((double)__half2float(row[i]) - dmx);
        const double sum = block_sum_f64(s, red);
        const double top = 1.0 / sum;  // the max entry's exp is exactly 1
        const double inv_t = 1.0 / temperature;
        const bool unit_t = temperature == 1.0;
        double t = 0.0;
        for (int i = threadIdx.x; i < vocab; i += ACC_THREADS)
            t += weight_of(exp((double)__half2float(row[i]) - dmx), sum, top, inv_t, unit_t);
        const double total = block_sum_f64(t, red);
        st.sum = sum, st.total = total;
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0) stats[blockIdx.x] = st;
}

// probability of one token under a row's shaped distribution (distribution.rs:61-66 over the full support)
__device__ __forceinline__ double prob_of(const __half* row, const RowStats& st, int token, double inv_t, bool unit_t) {
    const double e = exp((double)__half2float(row[token]) - (double)st.max);
    const double w = weight_of(e, st.sum, 1.0 / st.sum, inv_t, unit_t);
    return st.total > 0.0 ? w / st.total : 0.0;
}

struct DrawCtx {
    unsigned long long hist[NBINS];
    unsigned long long scan[ACC_THREADS];
    double red[ACC_THREADS / 32];
    unsigned long long last_key;  // fallback: smallest exp (bits) then largest index
    unsigned int last_idx;
    unsigned int sel_bin;
    unsigned long long sel_before;
    int result;
    unsigned long long gap_lo, gap_hi;
};

// Exclusive scan of hist[0..NBINS) in place by the block; finds the first bin whose inclusive prefix
// exceeds `target` (strictly), returns it through ctx.sel_bin with the prefix before it.  If no bin
// does (rounding at the tail) sel_bin = NBINS.
__device__ void find_bin(DrawCtx& c, unsigned long long target, unsigned long long before) {
    constexpr int PER = NBINS / ACC_THREADS;  // 2
    unsigned long long loc[PER], s = 0;
#pragma unroll
    for (int j = 0; j < PER; j++) loc[j] = c.hist[threadIdx.x * PER + j], s += loc[j];
    // block exclusive scan of s
    unsigned long long v = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += n;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 31) c.scan[threadIdx.x >> 5] = v;
    if (threadIdx.x == 0) c.sel_bin = NBINS, c.sel_before = 0;
    __syncthreads();
    unsigned long long wbase = 0;
    for (int i = 0; i < (int)(threadIdx.x >> 5); i++) wbase += c.scan[i];
    unsigned long long run = before + wbase + v - s;  // mass before this thread's first bin
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const unsigned long long after = run + loc[j];
        if (target >= run && target < after) {  // exactly one thread/bin satisfies this
            c.sel_bin = threadIdx.x * PER + j;
            c.sel_before = run;
        }
        run = after;
    }
    __syncthreads();
}

// One draw from a distribution given as fixed-point masses fp[i] (2^-60 units) over keys key(i), in rank
// order (key ascending = logit descending, ties index ascending).  target in 2^-60 units.
__device__ int radix_draw(DrawCtx& c, const __half* __restrict__ krow, const unsigned long long* __restrict__ fp,
                          int vocab, unsigned long long target, unsigned long long* gap_lo, unsigned long long* gap_hi) {
    uint32_t prefix = 0;
    unsigned long long before = 0;
    const int shifts[3] = {21, 10, 0};
    const int widths[3] = {11, 11, 10};
    int done_bits = 0;
    for (int pass = 0; pass < 3; pass++) {
        for (int i = threadIdx.x; i < NBINS; i += ACC_THREADS) c.hist[i] = 0;
        __syncthreads();
        const uint32_t hi_mask = done_bits ? (0xFFFFFFFFu << (32 - done_bits)) : 0u;
        for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) {
            const uint32_t kd = desc_key(__half2float(krow[i]));
            if ((kd & hi_mask) == prefix) {
                const unsigned long long m = fp[i];
                if (m) atomicAdd(&c.hist[(kd >> shifts[pass]) & ((1u << widths[pass]) - 1)], m);
            }
        }
        __syncthreads();
        find_bin(c, target, before);
        if (c.sel_bin == NBINS) return -1;  // past the end: the caller takes the last support entry
        prefix |= c.sel_bin << shifts[pass];
        before = c.sel_before;
        done_bits += widths[pass];
        __syncthreads();
    }
    // all members share the key: walk them in index order (contiguous index ranges per thread)
    const int per = (vocab + ACC_THREADS - 1) / ACC_THREADS;
    const int lo = threadIdx.x * per, hi = min(vocab, lo + per);
    unsigned long long mine = 0;
    for (int i = lo; i < hi; i++)
        if (desc_key(__half2float(krow[i])) == prefix) mine += fp[i];
    unsigned long long v = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += n;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 31) c.scan[threadIdx.x >> 5] = v;
    if (threadIdx.x == 0) c.result = -1;
    __syncthreads();
    unsigned long long wbase = 0;
    for (int i = 0; i < (int)(threadIdx.x >> 5); i++) wbase += c.scan[i];
    unsigned long long run = before + wbase + v - mine;
    for (int i = lo; i < hi; i++) {
        if (desc_key(__half2float(krow[i])) != prefix) continue;
        const unsigned long long after = run + fp[i];
        if (target >= run && target < after) {
            c.result = i;
            c.gap_lo = target - run;
            c.gap_hi = after - target;
        }
        run = after;
    }
    __syncthreads();
    *gap_lo = c.gap_lo;
    *gap_hi = c.gap_hi;
    return c.result;
}

constexpr double FP_ONE = 1152921504606846976.0;  // 2^60

// Fills fp[i] with the fixed-point probability of every token under (a) the shaped row `prow` or
// (b) the normalised residual max(p - q, 0), and finds the last support entry in rank order.
// Returns false when the residual is empty / below the reference's 1e-12 floor.
__device__ bool fill_masses(DrawCtx& c, const __half* prow, const RowStats& ps, const __half* qrow, const RowStats* qs,
                            int vocab, double inv_t, bool unit_t, unsigned long long* fp) {
    const double pmax = (double)ps.max, ptop = 1.0 / ps.sum;
    double norm = ps.total;
    if (qrow) {
        const double qmax = (double)qs->max, qtop = 1.0 / qs->sum;
        double t = 0.0;
        int any = 0;
        for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) {
            const double pp = weight_of(exp((double)__half2float(prow[i]) - pmax), ps.sum, ptop, inv_t, unit_t) / ps.total;
            const double qq = weight_of(exp((double)__half2float(qrow[i]) - qmax), qs->sum, qtop, inv_t, unit_t) / qs->total;
            const double m = fmax(pp - qq, 0.0);
            t += m;
            any |= m > 0.0;
        }
        norm = block_sum_f64(t, c.red);
        const int have = __syncthreads_or(any);
        if (norm < 1e-12 || !have) return false;  // distribution.rs:119-121
    }
    if (threadIdx.x == 0) c.last_key = ~0ull, c.last_idx = 0;
    __syncthreads();
    unsigned long long best = ~0ull;
    for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) {
        const double e = exp((double)__half2float(prow[i]) - pmax);
        double m = weight_of(e, ps.sum, ptop, inv_t, unit_t) / ps.total;
        bool in_support = true;
        if (qrow) {
            const double qq = weight_of(exp((double)__half2float(qrow[i]) - (double)qs->max), qs->sum, 1.0 / qs->sum, inv_t,
                                        unit_t) / qs->total;
            m = fmax(m - qq, 0.0);
            in_support = m > 0.0;
            m = m / norm;
        }
        fp[i] = (unsigned long long)__double2ull_rn(m * FP_ONE);
        if (in_support) best = min(best, (unsigned long long)__double_as_longlong(e));
    }
    atomicMin(&c.last_key, best);
    __syncthreads();
    const unsigned long long lk = c.last_key;
    unsigned int li = 0;
    for (int i = threadIdx.x; i < vocab; i += ACC_THREADS) {
        const double e = exp((double)__half2float(prow[i]) - pmax);
        if ((unsigned long long)__double_as_longlong(e) != lk) continue;
        if (qrow) {
            const double pp = weight_of(e, ps.sum, ptop, inv_t, unit_t) / ps.total;
            const double qq = weight_of(exp((double)__half2float(qrow[i]) - (double)qs->max), qs->sum, 1.0 / qs->sum, inv_t,
                                        unit_t) / qs->total;
            if (!(pp - qq > 0.0)) continue;
        }
        li = max(li, (unsigned int)i);
    }
    atomicMax(&c.last_idx, li);
    __syncthreads();
    return true;
}

__device__ __forceinline__ double unit_interval(uint64_t v) { return (double)(v >> 11) * (1.0 / 9007199254740992.0); }

__global__ void __launch_bounds__(ACC_THREADS)
    accept_decide_kernel(const __half* __restrict__ target, const __half* __restrict__ draft,
                         const int32_t* __restrict__ proposals, int prop_stride, const uint64_t* __restrict__ uniforms,
                         int k, int vocab, double temperature, const RowStats* __restrict__ stats,
                         unsigned long long* __restrict__ scratch, tsb_accept_out* __restrict__ out,
                         int32_t* __restrict__ next_tokens, int next_stride) {
    __shared__ DrawCtx c;
    __shared__ int s_accepted, s_draws, s_rejected, s_status;
    __shared__ double s_margin;
    pdl_wait();
    const int b = blockIdx.x;
    const int rps = 2 * k + 1;
    const RowStats* st = stats + (size_t)b * rps;
    const __half* trows = target + (size_t)b * (k + 1) * vocab;
    const __half* drows = draft + (size_t)b * k * vocab;
    const int32_t* prop = proposals + (size_t)b * prop_stride;
    const uint64_t* un = uniforms + (size_t)b * rps;
    unsigned long long* fp = scratch + (size_t)b * vocab;
    const bool sampled = temperature != 0.0;
    const double inv_t = sampled ? 1.0 / temperature : 1.0;
    const bool unit_t = temperature == 1.0;

    if (threadIdx.x == 0) {
        int accepted = 0, draws = 0, rejected = 0, status = 0;
        double margin = INFINITY;
        for (int i = 0; i < rps; i++) status |= st[i].nonfinite;
        if (!status) {
            for (int i = 0; i < k; i++) {
                const int x = prop[i];
                if (x < 0 || x >= vocab) {
                    status = 2;
                    break;
                }
                if (sampled) {
                    const double px = prob_of(trows + (size_t)i * vocab, st[i], x, inv_t, unit_t);
                    const double qx = prob_of(drows + (size_t)i * vocab, st[k + 1 + i], x, inv_t, unit_t);
                    const double r = unit_interval(un[draws++]);
                    margin = fmin(margin, fabs(r * qx - px));
                    if (r * qx <= px) {
                        out[b].tokens[accepted++] = x;
                    } else {
                        rejected = 1;
                        break;
                    }
                } else {
                    if (st[i].argmax != x) break;
                    out[b].tokens[accepted++] = x;
                }
            }
        }
        s_accepted = accepted, s_draws = draws, s_rejected = rejected, s_status = status, s_margin = margin;
    }
    __syncthreads();
    const int accepted = s_accepted;
    int token = -1;
    unsigned long long gap_lo = ~0ull, gap_hi = ~0ull;
    if (s_status == 0) {
        const __half* prow = trows + (size_t)accepted * vocab;
        if (!sampled) {
            token = st[accepted].argmax;
        } else {
            const uint64_t u = un[s_draws];
            const unsigned long long tgt = (unsigned long long)(u >> 11) << 7;  // k * 2^-53 in 2^-60 units
            bool have = false;
            if (s_rejected)
                have = fill_masses(c, prow, st[accepted], drows + (size_t)accepted * vocab, &st[k + 1 + accepted], vocab, inv_t,
                                   unit_t, fp);
            if (!have) fill_masses(c, prow, st[accepted], nullptr, nullptr, vocab, inv_t, unit_t, fp);
            token = radix_draw(c, prow, fp, vocab, tgt, &gap_lo, &gap_hi);
            if (token < 0) token = (int)c.last_idx, gap_lo = gap_hi = 0;
        }
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tsb_accept_out& o = out[b];
        o.accepted = accepted;
        o.draws = s_draws + ((sampled && s_status == 0) ? 1 : 0);
        o.tokens[accepted] = token;
        for (int i = accepted + 1; i < 16; i++) o.tokens[i] = -1;
        o.status = s_status;
        o._pad = 0;
        o.margin_accept = s_margin;
        o.margin_draw = (double)(gap_lo < gap_hi ? gap_lo : gap_hi) / FP_ONE;
        if (next_tokens) next_tokens[(size_t)b * next_stride] = token;
    }
}

// Draft-side draw: one CTA per stream, one row each.
__global__ void __launch_bounds__(ACC_THREADS)
    sample_kernel(const __half* __restrict__ logits, int64_t logits_stride, const uint64_t* __restrict__ uniforms,
                  int uni_stride, int vocab, double temperature, const RowStats* __restrict__ stats,
                  unsigned long long* __restrict__ scratch, int32_t* __restrict__ tokens, int token_stride,
                  double* __restrict__ margins, uint32_t* __restrict__ err) {
    __shared__ DrawCtx c;
    pdl_wait();
    const int b = blockIdx.x;
    const RowStats st = stats[b];
    const __half* row = logits + (size_t)b * logits_stride;
    int token;
    unsigned long long gap_lo = ~0ull, gap_hi = ~0ull;
    if (st.nonfinite) {
        token = -1;
        if (threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_NONFINITE);
    } else if (temperature == 0.0) {
        token = st.argmax;
    } else {
        unsigned long long* fp = scratch + (size_t)b * vocab;
        fill_masses(c, row, st, nullptr, nullptr, vocab, 1.0 / temperature, temperature == 1.0, fp);
        const unsigned long long tgt = (unsigned long long)(uniforms[(size_t)b * uni_stride] >> 11) << 7;
        token = radix_draw(c, row, fp, vocab, tgt, &gap_lo, &gap_hi);
        if (token < 0) token = (int)c.last_idx, gap_lo = gap_hi = 0;
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tokens[(size_t)b * token_stride] = token;
        if (margins) margins[b] = (double)(gap_lo < gap_hi ? gap_lo : gap_hi) / FP_ONE;
    }
}

int32_t check_shaping(tsb_ctx* ctx, const tsb_shaping* sh) {
    TSB_REQUIRE(ctx, sh, "null shaping");
    // crates/selection/src/shaping.rs:84-123
    TSB_REQUIRE(ctx, isfinite(sh->temperature) && sh->temperature >= 0.0, "temperature must be finite and non-negative");
    TSB_REQUIRE(ctx, sh->top_k <= 256, "top_k must be between 0 and 256");
    TSB_REQUIRE(ctx, !(sh->top_p > 0.0) || sh->top_p <= 1.0, "top_p must be in (0, 1]");
    TSB_REQUIRE(ctx, isfinite(sh->repetition_penalty) && sh->repetition_penalty > 0.0, "repetition_penalty must be > 0");
    if (sh->temperature != 0.0 &&
        (sh->top_k != 0 || sh->top_p > 0.0 || sh->min_p > 0.0 || sh->repetition_penalty != 1.0 ||
         sh->presence_penalty != 0.0 || sh->frequency_penalty != 0.0))
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED,
                        "the device sampler covers temperature with the whole vocabulary only (top_k = 0, top_p, min_p "
                        "and penalties off)");
    return TSB_OK;
}

}  // namespace

size_t accept_scratch_bytes(int batch, int k, int vocab) {
    const size_t stats = ((size_t)batch * (2 * k + 1) * sizeof(RowStats) + 255) & ~(size_t)255;
    return stats + (size_t)batch * vocab * sizeof(unsigned long long);
}

cudaError_t launch_accept(tsb_ctx* ctx, cudaStream_t st, const __half* target, const __half* draft, const int32_t* proposals,
                          int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, double temperature,
                          tsb_accept_out* out_dev, int32_t* next_tokens, int next_stride, void* scratch) {
    RowStats* stats = reinterpret_cast<RowStats*>(scratch);
    const size_t stats_bytes = ((size_t)batch * (2 * k + 1) * sizeof(RowStats) + 255) & ~(size_t)255;
    unsigned long long* fp = reinterpret_cast<unsigned long long*>((char*)scratch + stats_bytes);
    const int rps = 2 * k + 1;
    cudaError_t e = tsb_launch(ctx, accept_stats_kernel, dim3((unsigned)(batch * rps)), dim3(ACC_THREADS), 0, st, true, target,
                               draft, k, vocab, temperature, stats, rps, (int64_t)0);
    if (e != cudaSuccess) return e;
    return tsb_launch(ctx, accept_decide_kernel, dim3((unsigned)batch), dim3(ACC_THREADS), 0, st, true, target, draft,
                      proposals, prop_stride, uniforms, k, vocab, temperature, (const RowStats*)stats, fp, out_dev,
                      next_tokens, next_stride);
}

cudaError_t launch_sample(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int64_t logits_stride,
                          const uint64_t* uniforms, int uni_stride, int batch, int vocab, double temperature,
                          int32_t* tokens_dev, int token_stride, double* margins_dev, void* scratch) {
    RowStats* stats = reinterpret_cast<RowStats*>(scratch);
    const size_t stats_bytes = ((size_t)batch * sizeof(RowStats) + 255) & ~(size_t)255;
    unsigned long long* fp = reinterpret_cast<unsigned long long*>((char*)scratch + stats_bytes);
    cudaError_t e = tsb_launch(ctx, accept_stats_kernel, dim3((unsigned)batch), dim3(ACC_THREADS), 0, st, true, logits,
                               (const __half*)nullptr, 0, vocab, temperature, stats, 1, logits_stride);
    if (e != cudaSuccess) return e;
    return tsb_launch(ctx, sample_kernel, dim3((unsigned)batch), dim3(ACC_THREADS), 0, st, true, logits, logits_stride,
                      uniforms, uni_stride, vocab, temperature, (const RowStats*)stats, fp, tokens_dev, token_stride,
                      margins_dev, ctx->dev_error);
}

int32_t accept_check_shaping(tsb_ctx* ctx, const tsb_shaping* sh) { return check_shaping(ctx, sh); }

extern "C" {

size_t tsb_accept_scratch_bytes(int32_t batch, int32_t k, int32_t vocab) {
    if (batch <= 0 || k < 0 || vocab <= 0) return 0;
    return accept_scratch_bytes(batch, k, vocab);
}

int32_t tsb_accept(tsb_ctx* ctx, tsb_stream s, const void* target_logits_f16, const void* draft_logits_f16,
                   const int32_t* proposals, const uint64_t* uniforms, int32_t batch, int32_t k, int32_t vocab,
                   const tsb_shaping* shaping, tsb_accept_out* out_dev, void* scratch, size_t scratch_bytes) {
    if (!ctx) return TSB_ERR_INVALID;
    int32_t rc = check_shaping(ctx, shaping);
    if (rc) return rc;
    TSB_REQUIRE(ctx, target_logits_f16 && out_dev && scratch, "null buffer");
    TSB_REQUIRE(ctx, batch > 0 && vocab > 0, "batch and vocab must be positive");
    TSB_REQUIRE(ctx, k >= 0 && k <= 15, "k must be 0..15 (the reference allows blocks 1..=15)");
    TSB_REQUIRE(ctx, k == 0 || (draft_logits_f16 && proposals), "draft logits and proposals are required when k > 0");
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_scratch_bytes(batch, k, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_accept(ctx, (cudaStream_t)s, (const __half*)target_logits_f16, (const __half*)draft_logits_f16,
                                proposals, k, uniforms, batch, k, vocab, shaping->temperature, out_dev, nullptr, 0, scratch));
    return TSB_OK;
}

int32_t tsb_sample(tsb_ctx* ctx, tsb_stream s, const void* logits_f16, const uint64_t* uniforms, int32_t batch,
                   int32_t vocab, const tsb_shaping* shaping, int32_t* tokens_dev, double* margins_dev, void* scratch,
                   size_t scratch_bytes) {
    if (!ctx) return TSB_ERR_INVALID;
    int32_t rc = check_shaping(ctx, shaping);
    if (rc) return rc;
    TSB_REQUIRE(ctx, logits_f16 && tokens_dev && scratch, "null buffer");
    TSB_REQUIRE(ctx, batch > 0 && vocab > 0, "batch and vocab must be positive");
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_scratch_bytes(batch, 0, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_sample(ctx, (cudaStream_t)s, (const __half*)logits_f16, vocab, uniforms, 1, batch, vocab,
                                shaping->temperature, tokens_dev, 1, margins_dev, scratch));
    return TSB_OK;
}

}  // extern "C"
