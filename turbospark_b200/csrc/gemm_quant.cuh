// Internal interface of the quantized-matmul kernels (shared with the model runner).
#pragma once
#include "common.cuh"
#include "kv.cuh"

// The activation operand the matmul kernels consume ("fragment-major" f16).
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
// xs holds, per tile, block and lane, a uint4 with the sums of the f16 values
// of every 16-column run of the block (sixteen sums s[0..16) per token), each
// split into an f16 high part and an f16 remainder, laid out as the B operand
// of one m16n8k16 mma over those sums:
//   .x = hi(s[2tig]) | hi(s[2tig+1]) << 16     .y = hi(s[2tig+8]) | hi(s[2tig+9]) << 16
//   .z, .w the same for the remainders
// (the Q4_K min term multiplies these sums by the sub-block mins).
struct ActOperand {
    const uint4* xp;  // [tiles][cols/256][8][32]
    const uint4* xs;  // [tiles][cols/256][32]
};
struct ActOut {  // where a producer writes an operand (both null = do not)
    uint4* xp;
    uint4* xs;
};

inline int act_tiles(int tokens) { return (tokens + 7) / 8; }
inline size_t act_xp_bytes(int tokens, int64_t cols) { return (size_t)act_tiles(tokens) * 8 * cols * sizeof(__half); }
inline size_t act_xs_bytes(int tokens, int64_t cols) { return (size_t)act_tiles(tokens) * (cols / 256) * 32 * sizeof(uint4); }

// What the kernel does with a finished 16-row tile (or pair of tiles).
enum GemmEpi {
    EPI_PLAIN = 0,       // y[t, row] = acc                               (public operator)
    EPI_SCALE = 1,       // y[t, row] = inv_rms[t] * acc                  (head over a pre-normed operand)
    EPI_RESID_NORM = 2,  // h += f16(acc); next operand = f16(h * g); partial sum of h^2   (o_proj, down)
    EPI_SILU = 3,        // pair (gate tile, up tile): operand = f16(silu(f16(inv*g)) * f16(inv*u))
    EPI_ROPE_STORE = 4,  // pair (low half, high half) of a q or k head: scale, rotate, q -> buffer, k -> cache; v -> cache
    EPI_MOE_ACT = 5,     // pair (gate tile, up tile) of one expert: operand = f16(act(g) * u), no norm, no f16 rounding of g, u
};

// RMSNorm split around a matmul.  The reference computes xn = f16(x * w * inv_rms) and feeds it to the matmul
// (crates/gpu/src/shaders/rmsnorm.metal:70-95).  Here the producer of x (an epilogue) writes f16(x * w) as the
// operand plus per-tile partial sums of x^2, and the consuming matmul multiplies its fp32 result by
// inv_rms = 1/sqrt(mean(x^2) + eps): the matmul is linear, so only the position of one f16 rounding moves.
struct EpiArgs {
    // input-side norm (EPI_SCALE, EPI_SILU, EPI_ROPE_STORE): partial sums of x^2, [tokens][ss_parts]
    const float* ss_in = nullptr;
    int ss_parts = 0;
    int d_in = 0;
    float eps = 0.f;
    // EPI_PLAIN / EPI_SCALE
    void* y = nullptr;
    int64_t y_stride = 0;
    int y_f32 = 0;
    const int32_t* y_rows = nullptr;  // EPI_PLAIN: output row of token t is y_rows[t] (negative: not stored) instead of t
    int y_every = 0;  // > 1: only the last token of every run of y_every tokens is stored, as output row token / y_every
    // EPI_RESID_NORM: residual stream h [tokens, rows], next norm weight g (bf16, [rows]), outputs
    __half* h = nullptr;
    const uint16_t* g = nullptr;
    float* ss_out = nullptr;  // [tokens][rows/16]
    // operand written by EPI_RESID_NORM (width rows) and EPI_SILU (width rows/2)
    ActOut out{nullptr, nullptr};
    // EPI_ROPE_STORE
    KvView kv{};
    int layer = 0;
    const tsb_row_desc* row_desc = nullptr;
    const float* cs = nullptr;  // [tokens][head_dim]: cos[0..hd/2) then sin[0..hd/2) of the row's position
    __half* q_out = nullptr;    // [tokens, n_q_heads * head_dim]
    int n_q_heads = 0, n_kv_heads = 0, head_dim = 0;
    int n_v_heads = -1;  // v heads among the rows; negative: as many as k heads.  q|k only: 0.  v only: n_q = n_kv = 0.
};

// x [tokens, cols] f16 natural order -> ActOperand buffers.
cudaError_t launch_act_prepare(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, int tokens, int cols,
                               uint4* xp, uint4* xs);
// the same with a row gather: operand token t comes from x row src_rows[t] (device array)
cudaError_t launch_act_prepare_gather(tsb_ctx* ctx, cudaStream_t st, const __half* x, int64_t x_stride, const int32_t* src_rows,
                                      int tokens, int cols, uint4* xp, uint4* xs);

// The matmul over verbatim block rows with the chosen epilogue.  rows = weight rows (for EPI_SILU the gate and
// up halves back to back; for EPI_ROPE_STORE q heads, k heads, v heads back to back).
cudaError_t launch_gemm_fused(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, int tokens, int epi, const EpiArgs& args);
// One launch (per 64 token rows) over n_mats matrices of one shape, w_stride bytes apart: matrix m multiplies
// count[m] token rows (device array) whose operand tiles start at tile tile_start[m] (device array) of `act`;
// outputs are indexed from token tile_start[m] * 8.  max_tokens bounds every count.  Epilogues: EPI_MOE_ACT, EPI_PLAIN.
cudaError_t launch_gemm_grouped(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t w_stride, int n_mats,
                                int64_t rows, int64_t cols, ActOperand act, const int32_t* count, const int32_t* tile_start,
                                int max_tokens, int epi, const EpiArgs& args);
// y[t, r] = W[r,:] . x[t,:]; y f16 or f32, [tokens, rows] with row stride y_stride (elements).
cudaError_t launch_gemm_quant(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t rows, int64_t cols,
                              ActOperand act, void* y, int64_t y_stride, int tokens, bool y_f32);

// The routed feed-forward (csrc/moe.cu): y = half(residual + sum over slots of w * down_e(act(gate_e x) * up_e x)).
// x rows have stride x_stride; ids / weights are [tokens, k]; workspace holds moe_ffn_workspace_bytes(...) bytes.
size_t moe_ffn_workspace_bytes(int tokens, int k, int n_experts, int d_model, int ffn);
// With y == nullptr launch_moe_ffn stops before the combine step and leaves the per-(row, slot) expert outputs,
// f32 [tokens * k, d_model], at this address inside the workspace.
const float* moe_ffn_values(const void* workspace, int tokens, int k, int n_experts, int d_model, int ffn);
cudaError_t launch_router_logits(tsb_ctx* ctx, cudaStream_t st, const uint8_t* q, const uint16_t* scale, const uint16_t* bias,
                                 const __half* x, int64_t x_stride, int tokens, int n_experts, int d, float* out);
cudaError_t launch_moe_route(tsb_ctx* ctx, cudaStream_t st, const float* logits, int tokens, int n_experts, int k, int32_t* ids,
                             __half* weights);
// expert_lo / n_local: the expert matrices passed hold experts [expert_lo, expert_lo + n_local) only (n_local == 0: all
// of them); (row, slot) pairs routed elsewhere are skipped and their values are zero.
cudaError_t launch_moe_ffn(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* gate_up, const uint8_t* down, int n_experts,
                           int d_model, int ffn, const __half* x, int64_t x_stride, const __half* residual, const int32_t* ids,
                           const __half* weights, int tokens, int k, __half* y, void* workspace, int expert_lo = 0, int n_local = 0);
// f16(x) for n f32 values (the summed o_proj shares of a tensor-parallel pass)
cudaError_t launch_f32_to_f16(tsb_ctx* ctx, cudaStream_t st, const float* x, __half* y, int64_t n);

// The tensor-memory (tcgen05) path for many token rows: Q4_K, rows a multiple of 128.  x is natural f16.
bool gemm_wide_supported(int qtype, int64_t rows, int64_t cols, int tokens);
// workspace: gemm_wide_workspace_bytes(cols, tokens) bytes the call may use for its operand copy (null: stream-ordered allocation)
// partials: gemm_wide_partial_bytes(...) bytes for the sums of tiles cut into runs (0: none needed).  Its first 4096
// bytes are ticket words: zero before the first call; every call leaves them zero again
size_t gemm_wide_workspace_bytes(int64_t cols, int tokens);
size_t gemm_wide_partial_bytes_for(int sm_count, int64_t rows, int64_t cols);  // the same for a device with that many SMs
size_t gemm_wide_partial_bytes(const tsb_ctx* ctx, int64_t rows, int64_t cols);
cudaError_t launch_gemm_wide_q4k(tsb_ctx* ctx, cudaStream_t st, const uint8_t* w, int64_t rows, int64_t cols, const __half* x,
                                 int64_t x_stride, int tokens, void* y, int64_t y_stride, bool y_f32, void* workspace = nullptr,
                                 void* partials = nullptr);

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
// Store the sum of one 16-column run (columns col16..col16+15 of token t) as hi + lo halves.
__device__ __forceinline__ void act_store_sum16(uint4* xs, int t, int col16, int nblk, float s) {
    const int blk = col16 >> 8, i = (col16 >> 4) & 15;
    const int tig = (i & 7) >> 1, comp = i >> 3, pos = i & 1;
    __half* q = reinterpret_cast<__half*>(xs + ((((size_t)(t >> 3) * nblk + blk) << 5) + ((t & 7) << 2) + tig));
    const __half hi = __float2half_rn(s);
    q[comp * 2 + pos] = hi;
    q[4 + comp * 2 + pos] = __float2half_rn(s - __half2float(hi));
}
// Pack eight f16 values (natural order) into the operand's stored order.
__device__ __forceinline__ uint4 act_pack8(const __half (&h)[8]) {
    uint4 o;
    __half2 a = __halves2half2(h[0], h[2]), b = __halves2half2(h[1], h[3]);
    __half2 c = __halves2half2(h[4], h[6]), d = __halves2half2(h[5], h[7]);
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    o.z = *reinterpret_cast<uint32_t*>(&c);
    o.w = *reinterpret_cast<uint32_t*>(&d);
    return o;
}

// Device helper for producers of matmul inputs: a thread that holds eight consecutive f32 outputs v[0..8) of
// column e0 (a multiple of 8) of token t stores them, rounded to f16, into the operand; the thread holding the
// even run of each 16-column pair also stores the pair's sum.  Threads of a warp must hold consecutive runs
// (lane i and lane i^1 form a pair) and all 32 lanes must call it together.
__device__ __forceinline__ void act_store8(const float (&v)[8], uint4* xp, uint4* xs, int t, int e0, int nblk,
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
    if (active) {
        xp[act_xp_index(t, e0, nblk)] = act_pack8(h);
        if ((e0 & 8) == 0) act_store_sum16(xs, t, e0, nblk, s);
    }
}
#endif
