// Rejection-sampling acceptance on the device.
//
// What it replaces: the host-side accept step of the reference's round loop
// (crates/runtime/src/speculative.rs:694-754,861-879) together with the f64
// sampler it calls (crates/selection/src/choose.rs:111-321, distribution.rs:57-125).
// The reference shapes every row into an explicit distribution in RANK order
// (probability descending, ties by ascending index) and walks cumulative sums
// in that order; everything is f64, summed sequentially.  These kernels keep
// the arithmetic in f64 and the order semantics, but replace the sort and the
// sequential walk by an order-preserving radix descent over the logit keys with
// exact integer (2^-60 fixed point) bin masses, so the outcome does not depend
// on thread scheduling.  Decisions (accept / reject, drawn token) equal the
// reference's unless a uniform lies within ~1e-13 of a decision boundary; the
// distance to the nearest boundary is returned so such a case is visible.
//
// Shaping covered: temperature (0 = argmax), top_k / top_p / min_p (the rank-order
// prefix the reference keeps), and - through the entry points that take the token
// history - the repetition, presence and frequency penalties (penalty.rs:15-82):
// a pre-pass writes the penalised rows as f32 and the same kernels run over them
// with 32-bit order keys.
//
// Parallel layout: one thread-block cluster of eight CTAs per logits row
// (statistics) or per stream (decision + draw).  Each CTA owns a contiguous
// eighth of the vocabulary, keeps its f64 exponentials / fixed-point masses in
// its own shared memory, and the eight CTAs reduce and broadcast through
// distributed shared memory in a fixed rank order.  Everything a draw needs
// stays on chip: the logits are read from HBM/L2 once or twice per row.
#include <cooperative_groups.h>

#include "accept.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int ACC_THREADS = 1024;
constexpr int CL = 8;               // CTAs per cluster
constexpr int SLICE_MAX = 20480;    // vocabulary entries one CTA can hold (8 * 20480 = 163840)
constexpr int RADIX_BINS = 256;     // the draw resolves a key eight bits at a time
constexpr int HIST_COPIES = 16;     // histogram copies per CTA: two warps share one
constexpr double FP_ONE = 1152921504606846976.0;  // 2^60

struct RowStats {
    float max;
    int32_t argmax;
    double sum;
    double total;    // sum of the weights of the surviving entries
    int32_t nonfinite;
    int32_t has_cut;  // truncation: the support is the rank-order prefix up to (cut_key, cut_idx) ...
    uint32_t cut_key;
    int32_t cut_idx;
    double min_e;     // ... whose exp is at least this (min-p), 0 = off
};

// Exchange area every CTA of a cluster exposes to its peers.
struct Xchg {
    double d[4];
    unsigned long long u[4];
    float f;
    int i[4];
};

__device__ __forceinline__ uint32_t desc_key(float x) {
    // ascending unsigned order of the key == descending order of x
    uint32_t u = __float_as_uint(x);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ~u;
}
// The same order on the 16 bits of an f16 logit (the rows are f16, so 16 bits carry the whole order; -0 ranks as +0,
// as it does when the values are compared).
__device__ __forceinline__ uint32_t desc_key16(__half h) {
    uint32_t u = __half_as_ushort(h);
    if (u == 0x8000u) u = 0;
    u = (u & 0x8000u) ? (~u & 0xFFFFu) : (u | 0x8000u);
    return ~u & 0xFFFFu;
}

// Row element types: f16 logits as the model writes them (two 8-bit radix passes resolve the order), or f32 rows after
// the history penalties (four passes).  -0 ranks as +0, as it does when the values are compared.
template <typename LT>
struct Logit;
template <>
struct Logit<__half> {
    static constexpr int KEY_PASSES = 2;
    static constexpr uint32_t KEY_MAX = 0xFFFFu;
    static __device__ __forceinline__ float val(__half h) { return __half2float(h); }
    static __device__ __forceinline__ uint32_t key(__half h) { return desc_key16(h); }
};
template <>
struct Logit<float> {
    static constexpr int KEY_PASSES = 4;
    static constexpr uint32_t KEY_MAX = 0xFFFFFFFFu;
    static __device__ __forceinline__ float val(float x) { return x; }
    static __device__ __forceinline__ uint32_t key(float x) { return desc_key(x == 0.f ? 0.f : x); }
};

#ifdef TSB_SAMPLE_TRACE
__device__ unsigned long long* g_sample_trace = nullptr;  // development builds: phase stamps of cluster 0, rank 0, thread 0
#define STRC(i) do { if (g_sample_trace && blockIdx.x == 0 && threadIdx.x == 0) g_sample_trace[i] = global_timer_ns(); } while (0)
#else
#define STRC(i)
#endif

// w_i of reweight (choose.rs:296-321): ((e/sum)/top)^(1/T), top = max_i e_i/sum = 1/sum.
__device__ __forceinline__ double weight_of(double e, double sum, double top, double inv_t, bool unit_t) {
    const double p = e / sum;
    const double r = top > 0.0 ? p / top : p;
    return unit_t ? r : pow(r, inv_t);
}

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

// Sum of one double per CTA over the cluster, ranks in order.  Slot selects which field of the exchange area.
__device__ __forceinline__ double cluster_sum_f64(cg::cluster_group& cluster, Xchg* x, int slot, double mine) {
    // one barrier: a slot is written once per kernel (or again only after other cluster barriers), so nobody can
    // overwrite it while a neighbour still reads
    if (threadIdx.x == 0) x->d[slot] = mine;
    cluster.sync();
    double t = 0.0;
    for (int r = 0; r < CL; r++) t += cluster.map_shared_rank(x, r)->d[slot];
    return t;
}

struct Slice {
    int lo, n;
};
__device__ __forceinline__ Slice my_slice(int vocab, int rank) {
    const int sl = ((vocab + CL - 1) / CL + 1) & ~1;
    Slice s;
    s.lo = min(vocab, rank * sl);
    s.n = min(vocab, s.lo + sl) - s.lo;
    return s;
}

// --------------------------------------------------------------------- draw
struct DrawShared {
    unsigned long long hist[HIST_COPIES][RADIX_BINS];
    unsigned long long scan[ACC_THREADS / 32];
    double red[ACC_THREADS / 32];
    Xchg xch;
    // written by rank 0 for everybody, or by the winning CTA into rank 0
    unsigned int sel_bin;
    unsigned long long sel_before;
    int result;
    unsigned long long gap_lo, gap_hi;
    unsigned long long best_exp;
    unsigned int best_idx;
};

// The draw over this cluster's row: fp[] holds every CTA's slice of fixed-point masses (2^-60 units), keys come
// from krow.  target in 2^-60 units.  Returns the token (same value in every CTA), -1 for "past the end".
template <typename LT, class MassFn>
__device__ int cluster_radix_select(cg::cluster_group& cluster, DrawShared& c, MassFn fp, const LT* __restrict__ krow, Slice sl,
                                    unsigned long long target, unsigned long long* gap) {
    const int rank = (int)cluster.block_rank();
    uint32_t prefix = 0;
    unsigned long long before = 0;
    constexpr int RB = 256;  // bins per pass: the key is resolved eight bits at a time, most significant first
    constexpr int PASSES = Logit<LT>::KEY_PASSES;
    for (int pass = 0; pass < PASSES; pass++) {
        const int shift = 8 * (PASSES - 1 - pass);
        for (int i = threadIdx.x; i < HIST_COPIES * RB; i += ACC_THREADS) (&c.hist[0][0])[i] = 0;
        __syncthreads();
        // Masses go into one of HIST_COPIES histograms (two warps share a copy): the first pass would otherwise
        // serialise every warp of the CTA on the handful of bins that hold most of a row (sign, exponent and two
        // mantissa bits of a logit).  Integer sums: the result does not depend on the order.
        {
            unsigned long long* hist = c.hist[(threadIdx.x >> 5) & (HIST_COPIES - 1)];
            for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
                const uint32_t kd = Logit<LT>::key(krow[sl.lo + j]);
                if (pass == 0 || (kd >> (shift + 8)) == (prefix >> (shift + 8))) {
                    const unsigned long long m = fp(j);
                    if (m) atomicAdd(&hist[(kd >> shift) & (RB - 1)], m);
                }
            }
        }
        __syncthreads();
        if (threadIdx.x < RB) {  // the copies fold into the first one, which is what the cluster's first CTA reads
            unsigned long long t = 0;
#pragma unroll
            for (int cp = 0; cp < HIST_COPIES; cp++) t += c.hist[cp][threadIdx.x];
            c.hist[0][threadIdx.x] = t;
        }
        STRC(6 + 2 * (pass & 1));
        cluster.sync();
        STRC(7 + 2 * (pass & 1));
        if (rank == 0) {
            // sum the members' histograms bin by bin, scan, find the bin the target falls into
            unsigned long long t = 0;
            if (threadIdx.x < RB)
                for (int rr = 0; rr < CL; rr++) t += cluster.map_shared_rank(&c, rr)->hist[0][threadIdx.x];
            unsigned long long v = t;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
                if ((threadIdx.x & 31) >= o) v += n;
            }
            if ((threadIdx.x & 31) == 31) c.scan[threadIdx.x >> 5] = v;
            if (threadIdx.x == 0) c.sel_bin = RB, c.sel_before = 0;
            __syncthreads();
            if (threadIdx.x < RB) {
                unsigned long long wbase = 0;
                for (int i = 0; i < (int)(threadIdx.x >> 5); i++) wbase += c.scan[i];
                const unsigned long long run = before + wbase + v - t, after = run + t;
                if (target >= run && target < after) c.sel_bin = threadIdx.x, c.sel_before = run;
            }
        }
        cluster.sync();
        const DrawShared* root = cluster.map_shared_rank(&c, 0);
        const unsigned int bin = root->sel_bin;
        const unsigned long long bef = root->sel_before;
        // no barrier here: rank 0 rewrites the selection only after the next pass's first cluster barrier, which every
        // member reaches after this read
        if (bin == RB) {
            cluster.sync();  // leave together: the caller may go on to use the exchange area
            return -1;
        }
        prefix |= bin << shift;
        before = bef;
    }
    // every member shares the key: walk them in index order.  Threads own contiguous runs of their CTA's slice;
    // CTAs are ordered by rank.
    const int per = (sl.n + ACC_THREADS - 1) / ACC_THREADS;
    const int lo = min(sl.n, (int)threadIdx.x * per), hi = min(sl.n, lo + per);
    unsigned long long mine = 0;
    for (int j = lo; j < hi; j++)
        if (Logit<LT>::key(krow[sl.lo + j]) == prefix) mine += fp(j);
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
    unsigned long long wbase = 0, cta_total = 0;
    for (int i = 0; i < ACC_THREADS / 32; i++) {
        if (i < (int)(threadIdx.x >> 5)) wbase += c.scan[i];
        cta_total += c.scan[i];
    }
    if (threadIdx.x == 0) c.xch.u[0] = cta_total;
    cluster.sync();
    unsigned long long rank_base = 0;
    for (int rr = 0; rr < rank; rr++) rank_base += cluster.map_shared_rank(&c.xch, rr)->u[0];
    unsigned long long run = before + rank_base + wbase + v - mine;
    DrawShared* root = cluster.map_shared_rank(&c, 0);
    for (int j = lo; j < hi; j++) {
        if (Logit<LT>::key(krow[sl.lo + j]) != prefix) continue;
        const unsigned long long after = run + fp(j);
        if (target >= run && target < after) {  // exactly one thread of one CTA
            root->result = sl.lo + j;
            root->gap_lo = target - run;
            root->gap_hi = after - target;
        }
        run = after;
    }
    cluster.sync();
    const int res = root->result;
    const unsigned long long gl = root->gap_lo, gh = root->gap_hi;
    cluster.sync();
    *gap = gl < gh ? gl : gh;
    return res;
}

// The draw over this cluster's row: fp[] holds every CTA's slice of fixed-point masses.
template <typename LT>
__device__ int cluster_radix_draw(cg::cluster_group& cluster, DrawShared& c, const unsigned long long* fp,
                                  const LT* __restrict__ krow, Slice sl, unsigned long long target,
                                  unsigned long long* gap) {
    return cluster_radix_select<LT>(cluster, c, [fp](int j) { return fp[j]; }, krow, sl, target, gap);
}

// What survives truncation (crates/selection/src/choose.rs:176-222): a prefix of the rank order (exp descending,
// index ascending) - the first top_k entries, cut further where the cumulative e/sum first reaches top_p - and of
// those the entries whose exp is at least min_p times the largest exp (which is exactly 1).
struct TruncShape {
    unsigned int top_k;
    double top_p, min_p;
};
template <typename LT>
__device__ __forceinline__ bool survives(const RowStats& st, LT logit, int idx, double e) {
    if (st.has_cut) {
        const uint32_t k = Logit<LT>::key(logit);
        if (k > st.cut_key || (k == st.cut_key && idx > st.cut_idx)) return false;
    }
    return !(st.min_e > 0.0) || e >= st.min_e;
}
// Finds the cut of a row whose exps sit in ecache[] (this CTA's slice) and whose sum is known.  Same result in
// every CTA of the cluster.
template <typename LT>
__device__ void cluster_find_cut(cg::cluster_group& cluster, DrawShared& c, const double* ecache, double sum,
                                 const LT* __restrict__ krow, Slice sl, int vocab, TruncShape tr, RowStats* st) {
    st->has_cut = 0, st->cut_key = Logit<LT>::KEY_MAX, st->cut_idx = 0x7fffffff;
    st->min_e = tr.min_p > 0.0 ? tr.min_p : 0.0;
    unsigned long long gap;
    if (tr.top_k > 0 && tr.top_k < (unsigned)vocab) {
        const int t = cluster_radix_select<LT>(cluster, c, [](int) { return 1ull; }, krow, sl, (unsigned long long)tr.top_k - 1, &gap);
        if (t >= 0) st->has_cut = 1, st->cut_key = Logit<LT>::key(krow[t]), st->cut_idx = t;
    }
    if (tr.top_p > 0.0) {
        // first entry whose cumulative e/sum reaches the threshold, in 2^-60 fixed point ("push, then test >=")
        const unsigned long long thr = (unsigned long long)__double2ull_ru(tr.top_p * FP_ONE);
        if (thr > 0) {
            const int t = cluster_radix_select<LT>(
                cluster, c, [ecache, sum](int j) { return (unsigned long long)__double2ull_rn(ecache[j] / sum * FP_ONE); }, krow, sl,
                thr - 1, &gap);
            if (t >= 0) {
                const uint32_t k = Logit<LT>::key(krow[t]);
                if (!st->has_cut || k < st->cut_key || (k == st->cut_key && t < st->cut_idx)) st->cut_key = k, st->cut_idx = t;
                st->has_cut = 1;
            }
        }
    }
}

// ---------------------------------------------------------------- statistics
// One cluster per row: max / first argmax / finiteness, sum_i exp(l_i - max), total = sum_i w_i.
template <typename LT>
__global__ void __launch_bounds__(ACC_THREADS)
    accept_stats_kernel(const LT* __restrict__ target, const LT* __restrict__ draft, int k, int vocab,
                        double temperature, TruncShape tr, RowStats* __restrict__ stats, int rows_per_stream, int64_t single_stride) {
    extern __shared__ __align__(16) uint8_t dyn[];
    double* ecache = reinterpret_cast<double*>(dyn);  // exp(l - max) of this CTA's slice
    __shared__ DrawShared c;
    Xchg& xch = c.xch;
    double* red = c.red;
    __shared__ float fred[ACC_THREADS / 32];
    __shared__ int ired[ACC_THREADS / 32];
    __shared__ int bad_flag;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int row_id = blockIdx.x / CL;
    pdl_wait();
    const int b = row_id / rows_per_stream, r = row_id % rows_per_stream;
    // rows 0..k are the target's, k+1..2k the drafter's; single_stride != 0: one row per stream, that many elements apart
    const LT* row = single_stride ? target + (size_t)b * single_stride
                    : (r <= k)    ? target + ((size_t)b * (k + 1) + r) * vocab
                                  : draft + ((size_t)b * k + (r - k - 1)) * vocab;
    const Slice sl = my_slice(vocab, rank);
    if (threadIdx.x == 0) bad_flag = 0;
    __syncthreads();
    float mx = -INFINITY;
    int am = 0x7fffffff;
    bool bad = false;
    for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
        const float v = Logit<LT>::val(row[sl.lo + j]);
        bad |= !isfinite(v);
        if (v > mx) mx = v, am = sl.lo + j;  // indices grow with j, so the first maximum is kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oam = __shfl_xor_sync(0xffffffffu, am, o);
        if (omx > mx || (omx == mx && oam < am)) mx = omx, am = oam;
    }
    if (bad) bad_flag = 1;
    if ((threadIdx.x & 31) == 0) fred[threadIdx.x >> 5] = mx, ired[threadIdx.x >> 5] = am;
    __syncthreads();
    if (threadIdx.x == 0) {
        mx = fred[0], am = ired[0];
        for (int i = 1; i < ACC_THREADS / 32; i++)
            if (fred[i] > mx || (fred[i] == mx && ired[i] < am)) mx = fred[i], am = ired[i];
        xch.f = mx, xch.i[0] = am, xch.i[1] = bad_flag;
    }
    cluster.sync();
    int nonfinite = 0;
    mx = -INFINITY, am = 0x7fffffff;
    for (int rr = 0; rr < CL; rr++) {
        const Xchg* o = cluster.map_shared_rank(&xch, rr);
        const float omx = o->f;
        const int oam = o->i[0];
        nonfinite |= o->i[1];
        if (omx > mx || (omx == mx && oam < am)) mx = omx, am = oam;
    }
    cluster.sync();
    RowStats st;
    st.max = mx, st.argmax = am, st.sum = 1.0, st.total = 1.0, st.nonfinite = nonfinite;
    st.has_cut = 0, st.cut_key = Logit<LT>::KEY_MAX, st.cut_idx = 0x7fffffff, st.min_e = 0.0;
    if (temperature != 0.0 && !nonfinite) {
        const double dmx = (double)mx;
        double s = 0.0;
        for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
            const double e = exp((double)Logit<LT>::val(row[sl.lo + j]) - dmx);
            ecache[j] = e;
            s += e;
        }
        const double sum = cluster_sum_f64(cluster, &xch, 0, block_sum_f64(s, red));
        const double top = 1.0 / sum;  // the max entry's exp is exactly 1
        const double inv_t = 1.0 / temperature;
        const bool unit_t = temperature == 1.0;
        st.sum = sum;
        const bool truncating = (tr.top_k > 0 && tr.top_k < (unsigned)vocab) || tr.top_p > 0.0 || tr.min_p > 0.0;
        if (truncating) cluster_find_cut<LT>(cluster, c, ecache, sum, row, sl, vocab, tr, &st);
        double t = 0.0;
        for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS)
            if (!truncating || survives(st, row[sl.lo + j], sl.lo + j, ecache[j])) t += weight_of(ecache[j], sum, top, inv_t, unit_t);
        st.total = cluster_sum_f64(cluster, &xch, 1, block_sum_f64(t, red));
    }
    pdl_launch_dependents();
    if (rank == 0 && threadIdx.x == 0) stats[row_id] = st;
    cluster.sync();  // nobody leaves while a neighbour may still read its exchange area
}

// probability of one token under a row's shaped distribution (distribution.rs:61-66 over the full support)
template <typename LT>
__device__ __forceinline__ double prob_of(const LT* row, const RowStats& st, int token, double inv_t, bool unit_t) {
    const double e = exp((double)Logit<LT>::val(row[token]) - (double)st.max);
    if (!survives(st, row[token], token, e)) return 0.0;  // distribution.rs:61-66: not in the support
    const double w = weight_of(e, st.sum, 1.0 / st.sum, inv_t, unit_t);
    return st.total > 0.0 ? w / st.total : 0.0;
}

// Fills fp[] (this CTA's slice) with the fixed-point probability of every token under (a) the shaped row prow
// or (b) the normalised residual max(p - q, 0), and finds the last support entry in rank order (smallest exp,
// then largest index).  Returns false when the residual is empty or below the reference's 1e-12 floor.
template <typename LT>
__device__ bool cluster_fill_masses(cg::cluster_group& cluster, DrawShared& c, unsigned long long* fp, const LT* prow,
                                    const RowStats& ps, const LT* qrow, const RowStats* qs, Slice sl, double inv_t,
                                    bool unit_t, unsigned int* last_idx) {
    const double pmax = (double)ps.max, ptop = 1.0 / ps.sum;
    double norm = 1.0;
    double* mass = reinterpret_cast<double*>(fp);  // the same storage holds f64 masses first, fixed point after
    double t = 0.0;
    int any = 0;
    unsigned long long best = ~0ull;
    // temperature 1: the weight is e up to two roundings, so the mass is e / total (see sample_kernel)
    const double p_inv = 1.0 / ps.total, q_inv = qrow ? 1.0 / qs->total : 0.0;
    for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
        const double e = exp((double)Logit<LT>::val(prow[sl.lo + j]) - pmax);
        double m = unit_t ? e * p_inv : weight_of(e, ps.sum, ptop, inv_t, unit_t) / ps.total;
        bool in_support = survives(ps, prow[sl.lo + j], sl.lo + j, e);
        if (!in_support) m = 0.0;
        if (qrow && in_support) {
            const double eq = exp((double)Logit<LT>::val(qrow[sl.lo + j]) - (double)qs->max);
            double qq = unit_t ? eq * q_inv : weight_of(eq, qs->sum, 1.0 / qs->sum, inv_t, unit_t) / qs->total;
            if (!survives(*qs, qrow[sl.lo + j], sl.lo + j, eq)) qq = 0.0;
            m = fmax(m - qq, 0.0);
            in_support = m > 0.0;
            t += m;
            any |= in_support;
        }
        mass[j] = m;
        if (in_support) best = min(best, (unsigned long long)__double_as_longlong(e));
    }
    if (qrow) {
        norm = cluster_sum_f64(cluster, &c.xch, 0, block_sum_f64(t, c.red));
        const int have_local = __syncthreads_or(any);
        if (threadIdx.x == 0) c.xch.i[0] = have_local;
        cluster.sync();
        int have = 0;
        for (int rr = 0; rr < CL; rr++) have |= cluster.map_shared_rank(&c.xch, rr)->i[0];
        cluster.sync();
        if (norm < 1e-12 || !have) return false;  // distribution.rs:119-121
    }
    // last support entry: smallest exp over the support, then the largest index holding it
    if (threadIdx.x == 0) c.best_exp = ~0ull, c.best_idx = 0;
    __syncthreads();
    atomicMin(&c.best_exp, best);
    cluster.sync();
    unsigned long long gbest = ~0ull;
    for (int rr = 0; rr < CL; rr++) gbest = min(gbest, cluster.map_shared_rank(&c, rr)->best_exp);
    unsigned int li = 0;
    for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
        const double e = exp((double)Logit<LT>::val(prow[sl.lo + j]) - pmax);
        if ((unsigned long long)__double_as_longlong(e) == gbest && survives(ps, prow[sl.lo + j], sl.lo + j, e) && (!qrow || mass[j] > 0.0))
            li = max(li, (unsigned int)(sl.lo + j));
    }
    atomicMax(&c.best_idx, li);
    cluster.sync();
    unsigned int gl = 0;
    for (int rr = 0; rr < CL; rr++) gl = max(gl, cluster.map_shared_rank(&c, rr)->best_idx);
    cluster.sync();
    *last_idx = gl;
    // f64 masses -> fixed point, in place
    for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
        const double m = qrow ? mass[j] / norm : mass[j];
        fp[j] = (unsigned long long)__double2ull_rn(m * FP_ONE);
    }
    __syncthreads();
    return true;
}

__device__ __forceinline__ double unit_interval(uint64_t v) { return (double)(v >> 11) * (1.0 / 9007199254740992.0); }

template <typename LT>
__global__ void __launch_bounds__(ACC_THREADS)
    accept_decide_kernel(const LT* __restrict__ target, const LT* __restrict__ draft,
                         const int32_t* __restrict__ proposals, int prop_stride, const uint64_t* __restrict__ uniforms,
                         int k, int vocab, double temperature, const RowStats* __restrict__ stats,
                         tsb_accept_out* __restrict__ out, int32_t* __restrict__ next_tokens, int next_stride) {
    extern __shared__ __align__(16) uint8_t dyn[];
    unsigned long long* fp = reinterpret_cast<unsigned long long*>(dyn);
    __shared__ DrawShared c;
    __shared__ int s_accepted, s_draws, s_rejected, s_status;
    __shared__ double s_margin;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    pdl_wait();
    const int b = blockIdx.x / CL;
    const int rps = 2 * k + 1;
    const RowStats* st = stats + (size_t)b * rps;
    const LT* trows = target + (size_t)b * (k + 1) * vocab;
    const LT* drows = draft + (size_t)b * k * vocab;
    const int32_t* prop = proposals + (size_t)b * prop_stride;
    const uint64_t* un = uniforms + (size_t)b * rps;
    const bool sampled = temperature != 0.0;
    const double inv_t = sampled ? 1.0 / temperature : 1.0;
    const bool unit_t = temperature == 1.0;
    const Slice sl = my_slice(vocab, rank);

    // the accept chain is a few scalar steps: every CTA runs it redundantly (same inputs, same result)
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
                        accepted++;
                    } else {
                        rejected = 1;
                        break;
                    }
                } else {
                    if (st[i].argmax != x) break;
                    accepted++;
                }
            }
        }
        s_accepted = accepted, s_draws = draws, s_rejected = rejected, s_status = status, s_margin = margin;
    }
    __syncthreads();
    const int accepted = s_accepted;
    int token = -1;
    unsigned long long gap = ~0ull;
    if (s_status == 0) {
        const LT* prow = trows + (size_t)accepted * vocab;
        if (!sampled) {
            token = st[accepted].argmax;
        } else {
            const uint64_t u = un[s_draws];
            const unsigned long long tgt = (unsigned long long)(u >> 11) << 7;  // k * 2^-53 in 2^-60 units
            bool have = false;
            unsigned int last = 0;
            if (s_rejected)
                have = cluster_fill_masses<LT>(cluster, c, fp, prow, st[accepted], drows + (size_t)accepted * vocab,
                                               &st[k + 1 + accepted], sl, inv_t, unit_t, &last);
            if (!have) cluster_fill_masses<LT>(cluster, c, fp, prow, st[accepted], (const LT*)nullptr, nullptr, sl, inv_t, unit_t, &last);
            token = cluster_radix_draw<LT>(cluster, c, fp, prow, sl, tgt, &gap);
            if (token < 0) token = (int)last, gap = 0;
        }
    }
    pdl_launch_dependents();
    if (rank == 0 && threadIdx.x == 0) {
        tsb_accept_out& o = out[b];
        o.accepted = accepted;
        o.draws = s_draws + ((sampled && s_status == 0) ? 1 : 0);
        for (int i = 0; i < accepted; i++) o.tokens[i] = prop[i];
        o.tokens[accepted] = token;
        for (int i = accepted + 1; i < 16; i++) o.tokens[i] = -1;
        o.status = s_status;
        o._pad = 0;
        o.margin_accept = s_margin;
        o.margin_draw = (double)gap / FP_ONE;
        if (next_tokens) next_tokens[(size_t)b * next_stride] = token;
    }
}

// Draft-side draw: one cluster per stream, one row each; statistics and draw in one kernel, so exp(l - max) is
// evaluated once per entry and stays in shared memory (first as e, then as the weight, then as the fixed-point mass).
template <typename LT>
__global__ void __launch_bounds__(ACC_THREADS)
    sample_kernel(const LT* __restrict__ logits, int64_t logits_stride, const uint64_t* __restrict__ uniforms,
                  int uni_stride, int vocab, double temperature, TruncShape tr, int32_t* __restrict__ tokens, int token_stride,
                  double* __restrict__ margins, uint32_t* __restrict__ err) {
    extern __shared__ __align__(16) uint8_t dyn[];
    unsigned long long* fp = reinterpret_cast<unsigned long long*>(dyn);
    double* ecache = reinterpret_cast<double*>(dyn);
    __shared__ DrawShared c;
    __shared__ float fred[ACC_THREADS / 32];
    __shared__ int ired[ACC_THREADS / 32];
    __shared__ int bad_flag;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    STRC(0);
    pdl_wait();
    STRC(1);
    const int b = blockIdx.x / CL;
    const LT* row = logits + (size_t)b * logits_stride;
    const Slice sl = my_slice(vocab, rank);
    // ---- max, first argmax, finiteness (as accept_stats_kernel)
    if (threadIdx.x == 0) bad_flag = 0;
    __syncthreads();
    float mx = -INFINITY;
    int am = 0x7fffffff;
    bool bad = false;
    for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
        const float v = Logit<LT>::val(row[sl.lo + j]);
        bad |= !isfinite(v);
        if (v > mx) mx = v, am = sl.lo + j;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oam = __shfl_xor_sync(0xffffffffu, am, o);
        if (omx > mx || (omx == mx && oam < am)) mx = omx, am = oam;
    }
    if (bad) bad_flag = 1;
    if ((threadIdx.x & 31) == 0) fred[threadIdx.x >> 5] = mx, ired[threadIdx.x >> 5] = am;
    __syncthreads();
    if (threadIdx.x == 0) {
        mx = fred[0], am = ired[0];
        for (int i = 1; i < ACC_THREADS / 32; i++)
            if (fred[i] > mx || (fred[i] == mx && ired[i] < am)) mx = fred[i], am = ired[i];
        c.xch.f = mx, c.xch.i[0] = am, c.xch.i[1] = bad_flag;
    }
    cluster.sync();
    int nonfinite = 0;
    mx = -INFINITY, am = 0x7fffffff;
    for (int rr = 0; rr < CL; rr++) {
        const Xchg* o = cluster.map_shared_rank(&c.xch, rr);
        const float omx = o->f;
        const int oam = o->i[0];
        nonfinite |= o->i[1];
        if (omx > mx || (omx == mx && oam < am)) mx = omx, am = oam;
    }
    cluster.sync();

    int token;
    unsigned long long gap = ~0ull;
    STRC(2);
    if (nonfinite) {
        token = -1;
        if (rank == 0 && threadIdx.x == 0) atomicCAS(err, 0u, (uint32_t)TSB_DEV_NONFINITE);
    } else if (temperature == 0.0) {
        token = am;
    } else {
        const double dmx = (double)mx, inv_t = 1.0 / temperature;
        const bool unit_t = temperature == 1.0;
        const bool truncating = (tr.top_k > 0 && tr.top_k < (unsigned)vocab) || tr.top_p > 0.0 || tr.min_p > 0.0;
        // e = exp(l - max) and its sum (and, when every entry survives, the last entry in rank order on the way)
        double acc = 0.0;
        unsigned long long best = ~0ull;
        unsigned int best_i = 0;
        for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
            const double e = exp((double)Logit<LT>::val(row[sl.lo + j]) - dmx);
            ecache[j] = e;
            acc += e;
            const unsigned long long eb = (unsigned long long)__double_as_longlong(e);
            if (eb <= best) best = eb, best_i = (unsigned int)(sl.lo + j);  // indices grow with j
        }
        STRC(3);
        const double sum = cluster_sum_f64(cluster, &c.xch, 0, block_sum_f64(acc, c.red));
        STRC(4);
        const double top = 1.0 / sum;
        RowStats st;
        st.has_cut = 0, st.cut_key = Logit<LT>::KEY_MAX, st.cut_idx = 0x7fffffff, st.min_e = 0.0;
        if (truncating) cluster_find_cut<LT>(cluster, c, ecache, sum, row, sl, vocab, tr, &st);
        // weights of the survivors, their total, and the last survivor in rank order (smallest e, then the largest index);
        // at temperature 1 without truncation the weights are the exps themselves and the total is their sum
        double total = sum;
        if (truncating || !unit_t) {
        acc = 0.0;
        best = ~0ull, best_i = 0;
        for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) {
            const double e = ecache[j];
            if (truncating && !survives(st, row[sl.lo + j], sl.lo + j, e)) {
                ecache[j] = 0.0;
                continue;
            }
            // At temperature 1 the reference's weight ((e/sum)/top with top = 1/sum) is e up to two roundings.  The
            // few-ulp difference can move a draw only when the target lies within ~1e-15 of a boundary, which the
            // reported margin shows.
            const double w = unit_t ? e : weight_of(e, sum, top, inv_t, unit_t);
            ecache[j] = w;
            acc += w;
            const unsigned long long eb = (unsigned long long)__double_as_longlong(e);
            if (eb <= best) best = eb, best_i = (unsigned int)(sl.lo + j);  // indices grow with j
        }
        total = cluster_sum_f64(cluster, &c.xch, 1, block_sum_f64(acc, c.red));
        }
        {
            const double scale = FP_ONE / total;
            for (int j = threadIdx.x; j < sl.n; j += ACC_THREADS) fp[j] = (unsigned long long)__double2ull_rn(ecache[j] * scale);
        }
        __syncthreads();
        STRC(5);
        const unsigned long long tgt = (unsigned long long)(uniforms[(size_t)b * uni_stride] >> 11) << 7;
        token = cluster_radix_draw<LT>(cluster, c, fp, row, sl, tgt, &gap);
        STRC(10);
        if (token < 0) {
            // the target lies past the last cumulative sum (rounding of the masses): the reference's walk then returns
            // the last entry in rank order - the smallest exp, and of those the largest index.  Rare, so the cluster-wide
            // search runs only here (the same answer in every CTA of the cluster, which all take this branch together).
            if (threadIdx.x == 0) c.best_exp = ~0ull, c.best_idx = 0;
            __syncthreads();
            atomicMin(&c.best_exp, best);
            cluster.sync();
            unsigned long long gbest = ~0ull;
            for (int rr = 0; rr < CL; rr++) gbest = min(gbest, cluster.map_shared_rank(&c, rr)->best_exp);
            if (best == gbest && best != ~0ull) atomicMax(&c.best_idx, best_i);
            cluster.sync();
            unsigned int last = 0;
            for (int rr = 0; rr < CL; rr++) last = max(last, cluster.map_shared_rank(&c, rr)->best_idx);
            cluster.sync();
            token = (int)last, gap = 0;
        }
    }
    pdl_launch_dependents();
    if (rank == 0 && threadIdx.x == 0) {
        tokens[(size_t)b * token_stride] = token;
        if (margins) margins[b] = (double)gap / FP_ONE;
    }
}

// The `width` largest logits of each listed row, by value descending and token id ascending on ties (the order
// in which a static draft tree takes the children of a node).  One CTA per row; width <= 8.  Row r of the launch
// reads logits + rows[r] * vocab and writes out[r * 8 .. r * 8 + width).
__global__ void __launch_bounds__(1024)
    topk_rows_kernel(const __half* __restrict__ logits, int vocab, const int32_t* __restrict__ rows, int width,
                     int32_t* __restrict__ out) {
    __shared__ float fred[32];
    __shared__ int ired[32];
    __shared__ int chosen[8];
    pdl_wait();
    const __half* row = logits + (size_t)rows[blockIdx.x] * vocab;
    for (int pick = 0; pick < width; pick++) {
        float mx = -INFINITY;
        int am = 0x7fffffff;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
            bool taken = false;
            for (int c = 0; c < pick; c++) taken |= chosen[c] == j;
            if (taken) continue;
            const float v = __half2float(row[j]);
            if (v > mx || (v == mx && j < am) || am == 0x7fffffff) mx = v, am = j;  // NaN never wins over a number
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
            const int oam = __shfl_xor_sync(0xffffffffu, am, o);
            if (oam != 0x7fffffff && (am == 0x7fffffff || omx > mx || (omx == mx && oam < am))) mx = omx, am = oam;
        }
        if ((threadIdx.x & 31) == 0) fred[threadIdx.x >> 5] = mx, ired[threadIdx.x >> 5] = am;
        __syncthreads();
        if (threadIdx.x == 0) {
            mx = fred[0], am = ired[0];
            for (int i = 1; i < (int)(blockDim.x >> 5); i++)
                if (ired[i] != 0x7fffffff && (am == 0x7fffffff || fred[i] > mx || (fred[i] == mx && ired[i] < am))) mx = fred[i], am = ired[i];
            chosen[pick] = am;
            out[blockIdx.x * 8 + pick] = am == 0x7fffffff ? -1 : am;
        }
        __syncthreads();
    }
    pdl_launch_dependents();
}

int32_t check_shaping(tsb_ctx* ctx, const tsb_shaping* sh, bool have_history = false) {
    TSB_REQUIRE(ctx, sh, "null shaping");
    // crates/selection/src/shaping.rs:84-123
    TSB_REQUIRE(ctx, isfinite(sh->temperature) && sh->temperature >= 0.0, "temperature must be finite and non-negative");
    TSB_REQUIRE(ctx, sh->top_k <= 256, "top_k must be between 0 and 256");
    TSB_REQUIRE(ctx, !(sh->top_p > 0.0) || sh->top_p <= 1.0, "top_p must be in (0, 1]");
    TSB_REQUIRE(ctx, isfinite(sh->repetition_penalty) && sh->repetition_penalty > 0.0, "repetition_penalty must be > 0");
    TSB_REQUIRE(ctx, !(sh->min_p > 0.0) || sh->min_p <= 1.0, "min_p must be in (0, 1]");
    TSB_REQUIRE(ctx, isfinite(sh->presence_penalty) && isfinite(sh->frequency_penalty), "presence and frequency penalties must be finite");
    if (!have_history && sh->temperature != 0.0 && (sh->repetition_penalty != 1.0 || sh->presence_penalty != 0.0 || sh->frequency_penalty != 0.0))
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED,
                        "repetition, presence and frequency penalties need the token history: use the entry points that take it "
                        "(tsb_accept_history, tsb_sample_history)");
    return TSB_OK;
}

size_t slice_smem(int vocab) { return (size_t)(((vocab + CL - 1) / CL + 1) & ~1) * sizeof(unsigned long long); }

// the cluster kernels keep a vocabulary slice in dynamic shared memory (opt-in per device, per instantiation)
template <typename LT>
cudaError_t configure_kernels(const tsb_ctx* ctx) {
    static SmemOptIn stats_done, decide_done, sample_done;
    cudaError_t e = tsb_opt_in_smem(ctx, accept_stats_kernel<LT>, (size_t)SLICE_MAX * 8, stats_done);
    if (e == cudaSuccess) e = tsb_opt_in_smem(ctx, accept_decide_kernel<LT>, (size_t)SLICE_MAX * 8, decide_done);
    if (e == cudaSuccess) e = tsb_opt_in_smem(ctx, sample_kernel<LT>, (size_t)SLICE_MAX * 8, sample_done);
    return e;
}

// ---- history penalties (crates/selection/src/penalty.rs:15-82, applied at choose.rs:139-154) as a pre-pass
// One CTA per shaped row: the row is copied to f32, then every DISTINCT id of the row's history is attenuated once
// (repetition: s > 0 ? s / penalty : s * penalty, saturated to the finite range) and every distinct id of the
// generated suffix loses presence + frequency * count.  Which history a row sees follows the round loop
// (crates/runtime/src/speculative.rs:636-648,701-734): a drafter row was shaped when the drafter ran, with the round's
// starting history; target row i is shaped after proposals 0..i were committed, so they are part of its history and of
// its generated count.  `marks` is a zeroed word per vocabulary entry per row: bit 31 = seen, low bits = occurrences
// in the generated suffix; the thread that exchanges a word back to zero applies the update, so each id is handled
// exactly once and the area is zero again when the kernel ends.
struct PenaltyArgs {
    const int32_t* history;   // [batch][hist_stride]
    int hist_stride;
    const int32_t* hist_len;  // [batch]
    const int32_t* generated; // [batch]: how many of the last history entries were generated in this turn
    const int32_t* proposals; // [batch][prop_stride] (null in sample mode)
    int prop_stride;
    float repetition;         // clamped to the normal f32 range
    double presence, frequency;
};
__global__ void __launch_bounds__(1024)
    penalize_rows_kernel(const __half* __restrict__ target, const __half* __restrict__ draft, int k, int vocab, int rows_per_stream,
                         int64_t single_stride, PenaltyArgs pa, float* __restrict__ out_target, float* __restrict__ out_draft,
                         uint32_t* __restrict__ marks) {
    pdl_wait();
    const int b = blockIdx.x / rows_per_stream, r = blockIdx.x % rows_per_stream;
    const bool is_target = single_stride != 0 || r <= k;
    const __half* row = single_stride ? target + (size_t)b * single_stride
                        : is_target   ? target + ((size_t)b * (k + 1) + r) * vocab
                                      : draft + ((size_t)b * k + (r - k - 1)) * vocab;
    float* out = single_stride ? out_target + (size_t)b * vocab
                 : is_target   ? out_target + ((size_t)b * (k + 1) + r) * vocab
                               : out_draft + ((size_t)b * k + (r - k - 1)) * vocab;
    uint32_t* mark = marks + (size_t)blockIdx.x * vocab;
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) out[v] = __half2float(row[v]);
    const int extra = (single_stride == 0 && is_target) ? r : 0;  // proposals already committed when this row is shaped
    const int nh = pa.hist_len[b];
    const int n_eff = nh + extra;
    int gen = pa.generated[b] + extra;
    gen = gen < 0 ? 0 : (gen > n_eff ? n_eff : gen);
    auto token_at = [&](int j) { return j < nh ? pa.history[(size_t)b * pa.hist_stride + j] : pa.proposals[(size_t)b * pa.prop_stride + (j - nh)]; };
    for (int j = threadIdx.x; j < n_eff; j += blockDim.x) {
        const int t = token_at(j);
        if (t < 0 || t >= vocab) continue;  // ids outside the vocabulary are skipped, as the reference skips them
        atomicOr(&mark[t], 0x80000000u);
        if (j >= n_eff - gen) atomicAdd(&mark[t], 1u);
    }
    __syncthreads();
    const bool rep_on = pa.repetition != 1.0f, pf_on = pa.presence != 0.0 || pa.frequency != 0.0;
    for (int j = threadIdx.x; j < n_eff; j += blockDim.x) {
        const int t = token_at(j);
        if (t < 0 || t >= vocab) continue;
        const uint32_t old = atomicExch(&mark[t], 0u);
        if (!old) continue;
        float sc = out[t];
        if (rep_on) {
            const float att = sc > 0.0f ? __fdiv_rn(sc, pa.repetition) : __fmul_rn(sc, pa.repetition);
            sc = fminf(fmaxf(att, -3.402823466e+38f), 3.402823466e+38f);
            if (att != att) sc = att;  // Rust's clamp keeps a NaN
        }
        const uint32_t cnt = old & 0x7fffffffu;
        if (pf_on && cnt > 0) sc = __fsub_rn(sc, (float)(pa.presence + pa.frequency * (double)cnt));
        out[t] = sc;
    }
    pdl_launch_dependents();
}

}  // namespace

size_t accept_scratch_bytes(int batch, int k, int vocab) {
    (void)vocab;
    return ((size_t)batch * (2 * k + 1) * sizeof(RowStats) + 255) & ~(size_t)255;
}

int accept_max_vocab() { return CL * SLICE_MAX; }

template <typename LT>
static cudaError_t launch_accept_t(tsb_ctx* ctx, cudaStream_t st, const LT* target, const LT* draft, const int32_t* proposals,
                                   int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, AcceptShape shape,
                                   tsb_accept_out* out_dev, int32_t* next_tokens, int next_stride, void* scratch) {
    RowStats* stats = reinterpret_cast<RowStats*>(scratch);
    const int rps = 2 * k + 1;
    const size_t smem = slice_smem(vocab);
    if (cudaError_t e = configure_kernels<LT>(ctx); e != cudaSuccess) return e;
    const TruncShape tr{shape.top_k, shape.top_p, shape.min_p};
    const double temperature = shape.temperature;
    cudaError_t e = tsb_launch_cluster(ctx, accept_stats_kernel<LT>, dim3((unsigned)(batch * rps * CL)), dim3(ACC_THREADS), smem, st,
                                       true, (unsigned)CL, target, draft, k, vocab, temperature, tr, stats, rps, (int64_t)0);
    if (e != cudaSuccess) return e;
    return tsb_launch_cluster(ctx, accept_decide_kernel<LT>, dim3((unsigned)(batch * CL)), dim3(ACC_THREADS), smem, st, true,
                              (unsigned)CL, target, draft, proposals, prop_stride, uniforms, k, vocab, temperature,
                              (const RowStats*)stats, out_dev, next_tokens, next_stride);
}

cudaError_t launch_accept(tsb_ctx* ctx, cudaStream_t st, const __half* target, const __half* draft, const int32_t* proposals,
                          int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, AcceptShape shape,
                          tsb_accept_out* out_dev, int32_t* next_tokens, int next_stride, void* scratch) {
    return launch_accept_t<__half>(ctx, st, target, draft, proposals, prop_stride, uniforms, batch, k, vocab, shape, out_dev, next_tokens,
                                   next_stride, scratch);
}

template <typename LT>
static cudaError_t launch_sample_t(tsb_ctx* ctx, cudaStream_t st, const LT* logits, int64_t logits_stride, const uint64_t* uniforms,
                                   int uni_stride, int batch, int vocab, AcceptShape shape, int32_t* tokens_dev, int token_stride,
                                   double* margins_dev) {
    const TruncShape tr{shape.top_k, shape.top_p, shape.min_p};
    const double temperature = shape.temperature;
    const size_t smem = slice_smem(vocab);
    if (cudaError_t e = configure_kernels<LT>(ctx); e != cudaSuccess) return e;
    return tsb_launch_cluster(ctx, sample_kernel<LT>, dim3((unsigned)(batch * CL)), dim3(ACC_THREADS), smem, st, true, (unsigned)CL,
                              logits, logits_stride, uniforms, uni_stride, vocab, temperature, tr, tokens_dev, token_stride,
                              margins_dev, ctx->dev_error);
}

cudaError_t launch_sample(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int64_t logits_stride,
                          const uint64_t* uniforms, int uni_stride, int batch, int vocab, AcceptShape shape,
                          int32_t* tokens_dev, int token_stride, double* margins_dev, void* scratch) {
    (void)scratch;
    return launch_sample_t<__half>(ctx, st, logits, logits_stride, uniforms, uni_stride, batch, vocab, shape, tokens_dev, token_stride,
                                   margins_dev);
}

// Scratch of the history variants: the statistics records, then the penalised f32 rows, then one mark word per
// vocabulary entry per row.
static size_t penalty_rows_bytes(int batch, int rows_per_stream, int vocab) { return (size_t)batch * rows_per_stream * vocab * sizeof(float); }
size_t accept_history_scratch_bytes(int batch, int k, int vocab) {
    return accept_scratch_bytes(batch, k, vocab) + 2 * penalty_rows_bytes(batch, 2 * k + 1, vocab) + 256;
}

static PenaltyArgs penalty_args(const tsb_shaping& sh, const int32_t* history, int hist_stride, const int32_t* hist_len,
                                const int32_t* generated, const int32_t* proposals, int prop_stride) {
    PenaltyArgs pa;
    pa.history = history, pa.hist_stride = hist_stride, pa.hist_len = hist_len, pa.generated = generated;
    pa.proposals = proposals, pa.prop_stride = prop_stride;
    // penalty.rs:21-27: the f64 setting is cast to f32 and clamped to the normal range
    float rp = (float)sh.repetition_penalty;
    rp = fminf(fmaxf(rp, 1.17549435e-38f), 3.402823466e+38f);
    pa.repetition = rp;
    pa.presence = sh.presence_penalty, pa.frequency = sh.frequency_penalty;
    return pa;
}

cudaError_t launch_accept_history(tsb_ctx* ctx, cudaStream_t st, const __half* target, const __half* draft, const int32_t* proposals,
                                  int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, const tsb_shaping& sh,
                                  const int32_t* history, int hist_stride, const int32_t* hist_len, const int32_t* generated,
                                  tsb_accept_out* out_dev, void* scratch, int32_t* next_tokens, int next_stride) {
    const int rps = 2 * k + 1;
    uint8_t* base = reinterpret_cast<uint8_t*>(scratch) + accept_scratch_bytes(batch, k, vocab);
    float* t32 = reinterpret_cast<float*>(base);
    float* d32 = t32 + (size_t)batch * (k + 1) * vocab;
    uint32_t* marks = reinterpret_cast<uint32_t*>(base + penalty_rows_bytes(batch, rps, vocab));
    cudaError_t e = cudaMemsetAsync(marks, 0, penalty_rows_bytes(batch, rps, vocab), st);
    if (e != cudaSuccess) return e;
    e = tsb_launch(ctx, penalize_rows_kernel, dim3((unsigned)(batch * rps)), dim3(1024), 0, st, false, target, draft, k, vocab, rps, (int64_t)0,
                   penalty_args(sh, history, hist_stride, hist_len, generated, proposals, prop_stride), t32, d32, marks);
    if (e != cudaSuccess) return e;
    return launch_accept_t<float>(ctx, st, t32, d32, proposals, prop_stride, uniforms, batch, k, vocab, AcceptShape(sh), out_dev, next_tokens,
                                  next_stride, scratch);
}

cudaError_t launch_sample_history(tsb_ctx* ctx, cudaStream_t st, const __half* logits, const uint64_t* uniforms, int batch, int vocab,
                                  const tsb_shaping& sh, const int32_t* history, int hist_stride, const int32_t* hist_len,
                                  const int32_t* generated, int32_t* tokens_dev, double* margins_dev, void* scratch, int64_t logits_stride,
                                  int uni_stride, int token_stride) {
    if (logits_stride <= 0) logits_stride = vocab;
    uint8_t* base = reinterpret_cast<uint8_t*>(scratch) + accept_scratch_bytes(batch, 0, vocab);
    float* l32 = reinterpret_cast<float*>(base);
    uint32_t* marks = reinterpret_cast<uint32_t*>(base + penalty_rows_bytes(batch, 1, vocab));
    cudaError_t e = cudaMemsetAsync(marks, 0, penalty_rows_bytes(batch, 1, vocab), st);
    if (e != cudaSuccess) return e;
    e = tsb_launch(ctx, penalize_rows_kernel, dim3((unsigned)batch), dim3(1024), 0, st, false, logits, (const __half*)nullptr, 0, vocab, 1,
                   logits_stride, penalty_args(sh, history, hist_stride, hist_len, generated, nullptr, 0), l32, (float*)nullptr, marks);
    if (e != cudaSuccess) return e;
    return launch_sample_t<float>(ctx, st, l32, vocab, uniforms, uni_stride, batch, vocab, AcceptShape(sh), tokens_dev, token_stride, margins_dev);
}

cudaError_t launch_topk_rows(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int vocab, const int32_t* rows_dev, int n_rows,
                             int width, int32_t* out_dev) {
    return tsb_launch(ctx, topk_rows_kernel, dim3((unsigned)n_rows), dim3(1024), 0, st, true, logits, vocab, rows_dev, width, out_dev);
}

cudaError_t launch_argmax_rows(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int n_rows, int vocab, void* scratch) {
    // the statistics kernel at temperature 0: max, first argmax and finiteness of every row (rows are "target rows")
    RowStats* stats = reinterpret_cast<RowStats*>(scratch);
    const size_t smem = slice_smem(vocab);
    if (cudaError_t e = configure_kernels<__half>(ctx); e != cudaSuccess) return e;
    return tsb_launch_cluster(ctx, accept_stats_kernel<__half>, dim3((unsigned)(n_rows * CL)), dim3(ACC_THREADS), smem, st, true,
                              (unsigned)CL, logits, (const __half*)nullptr, n_rows - 1, vocab, 0.0, TruncShape{0u, 0.0, 0.0}, stats, n_rows,
                              (int64_t)0);
}

int accept_row_stats_bytes() { return (int)sizeof(RowStats); }
void accept_row_stats_read(const void* host_stats, int row, int32_t* argmax, int32_t* nonfinite) {
    const RowStats* st = reinterpret_cast<const RowStats*>(host_stats) + row;
    *argmax = st->argmax;
    *nonfinite = st->nonfinite;
}

int32_t accept_check_shaping(tsb_ctx* ctx, const tsb_shaping* sh, bool have_history) { return check_shaping(ctx, sh, have_history); }
bool accept_has_penalties(const tsb_shaping& sh) {
    return sh.temperature != 0.0 && (sh.repetition_penalty != 1.0 || sh.presence_penalty != 0.0 || sh.frequency_penalty != 0.0);
}

#ifdef TSB_SAMPLE_TRACE
extern "C" __attribute__((visibility("default"))) void tsb_debug_set_sample_trace(void* p) {
    unsigned long long* q = static_cast<unsigned long long*>(p);
    cudaMemcpyToSymbol(g_sample_trace, &q, sizeof(q));
}
#endif

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
    if (vocab > accept_max_vocab())
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "vocabulary %d exceeds the %d entries one cluster holds on chip", vocab, accept_max_vocab());
    TSB_REQUIRE(ctx, k >= 0 && k <= 15, "k must be 0..15 (the reference allows blocks 1..=15)");
    TSB_REQUIRE(ctx, k == 0 || (draft_logits_f16 && proposals), "draft logits and proposals are required when k > 0");
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_scratch_bytes(batch, k, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_accept(ctx, (cudaStream_t)s, (const __half*)target_logits_f16, (const __half*)draft_logits_f16,
                                proposals, k, uniforms, batch, k, vocab, AcceptShape(*shaping), out_dev, nullptr, 0, scratch));
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
    if (vocab > accept_max_vocab())
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "vocabulary %d exceeds the %d entries one cluster holds on chip", vocab, accept_max_vocab());
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_scratch_bytes(batch, 0, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_sample(ctx, (cudaStream_t)s, (const __half*)logits_f16, vocab, uniforms, 1, batch, vocab,
                                AcceptShape(*shaping), tokens_dev, 1, margins_dev, scratch));
    return TSB_OK;
}

size_t tsb_accept_history_scratch_bytes(int32_t batch, int32_t k, int32_t vocab) {
    if (batch <= 0 || k < 0 || vocab <= 0) return 0;
    return accept_history_scratch_bytes(batch, k, vocab);
}

int32_t tsb_accept_history(tsb_ctx* ctx, tsb_stream s, const void* target_logits_f16, const void* draft_logits_f16,
                           const int32_t* proposals, const uint64_t* uniforms, int32_t batch, int32_t k, int32_t vocab,
                           const tsb_shaping* shaping, const int32_t* history_dev, int32_t hist_stride, const int32_t* hist_len_dev,
                           const int32_t* generated_dev, tsb_accept_out* out_dev, void* scratch, size_t scratch_bytes) {
    if (!ctx) return TSB_ERR_INVALID;
    int32_t rc = check_shaping(ctx, shaping, true);
    if (rc) return rc;
    TSB_REQUIRE(ctx, target_logits_f16 && out_dev && scratch, "null buffer");
    TSB_REQUIRE(ctx, history_dev && hist_len_dev && generated_dev && hist_stride > 0, "the history, its lengths and the generated counts are required");
    TSB_REQUIRE(ctx, batch > 0 && vocab > 0, "batch and vocab must be positive");
    if (vocab > accept_max_vocab())
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "vocabulary %d exceeds the %d entries one cluster holds on chip", vocab, accept_max_vocab());
    TSB_REQUIRE(ctx, k >= 0 && k <= 15, "k must be 0..15 (the reference allows blocks 1..=15)");
    TSB_REQUIRE(ctx, k == 0 || (draft_logits_f16 && proposals), "draft logits and proposals are required when k > 0");
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_history_scratch_bytes(batch, k, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_accept_history(ctx, (cudaStream_t)s, (const __half*)target_logits_f16, (const __half*)draft_logits_f16, proposals, k,
                                        uniforms, batch, k, vocab, *shaping, history_dev, hist_stride, hist_len_dev, generated_dev, out_dev,
                                        scratch));
    return TSB_OK;
}

int32_t tsb_sample_history(tsb_ctx* ctx, tsb_stream s, const void* logits_f16, const uint64_t* uniforms, int32_t batch, int32_t vocab,
                           const tsb_shaping* shaping, const int32_t* history_dev, int32_t hist_stride, const int32_t* hist_len_dev,
                           const int32_t* generated_dev, int32_t* tokens_dev, double* margins_dev, void* scratch, size_t scratch_bytes) {
    if (!ctx) return TSB_ERR_INVALID;
    int32_t rc = check_shaping(ctx, shaping, true);
    if (rc) return rc;
    TSB_REQUIRE(ctx, logits_f16 && tokens_dev && scratch, "null buffer");
    TSB_REQUIRE(ctx, history_dev && hist_len_dev && generated_dev && hist_stride > 0, "the history, its lengths and the generated counts are required");
    TSB_REQUIRE(ctx, batch > 0 && vocab > 0, "batch and vocab must be positive");
    if (vocab > accept_max_vocab())
        return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "vocabulary %d exceeds the %d entries one cluster holds on chip", vocab, accept_max_vocab());
    TSB_REQUIRE(ctx, shaping->temperature == 0.0 || uniforms, "uniforms are required at a positive temperature");
    TSB_REQUIRE(ctx, scratch_bytes >= tsb_accept_history_scratch_bytes(batch, 0, vocab), "scratch too small");
    DeviceGuard g(ctx);
    TSB_CUDA(ctx, launch_sample_history(ctx, (cudaStream_t)s, (const __half*)logits_f16, uniforms, batch, vocab, *shaping, history_dev,
                                        hist_stride, hist_len_dev, generated_dev, tokens_dev, margins_dev, scratch));
    return TSB_OK;
}

}  // extern "C"
