/*
 * tsb.h — C ABI of libtsb, a CUDA (sm_100a) backend for TurboSpark's
 * speculative-decoding verify path.
 *
 * Each entry point replaces one operator of the reference's Metal backend
 * (crates/gpu, "encode_*" functions) or one method of its SpeculativeProducer
 * trait (crates/runtime/src/producer.rs); the comment above each declaration
 * cites the reference interface it stands in for (path within the reference
 * project : lines).
 *
 * Conventions, kept from the reference's operator API (crates/gpu/src/lib.rs:181-503):
 *   - the caller owns every buffer; pointers are plain device pointers unless
 *     a parameter is named host_*;
 *   - quantized weights are the verbatim GGUF block bytes, one contiguous run
 *     of blocks per output row, addressed as (region, byte offset);
 *   - work is enqueued on the given CUDA stream (cudaStream_t passed as void*,
 *     NULL = the legacy default stream) and the caller synchronises;
 *   - precondition violations are refused before anything is enqueued;
 *   - every function returns a tsb_status (0 = OK), never throws, never aborts;
 *     tsb_last_error(ctx) returns the message of the last failure on that ctx;
 *   - a ctx belongs to one host thread and one GPU.
 *
 * Activations are IEEE binary16, accumulation is fp32, norm weights are
 * bfloat16 — the reference's storage contract
 * (crates/gpu/src/shaders/dequant_q4_k.metal:98-130, rmsnorm.metal:70-95).
 */
#ifndef TSB_H
#define TSB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TSB_API __attribute__((visibility("default")))
#else
#define TSB_API
#endif

typedef struct tsb_ctx tsb_ctx;
typedef struct tsb_kv tsb_kv;
typedef struct tsb_model tsb_model;
typedef struct tsb_session tsb_session;
typedef struct tsb_comm tsb_comm;
typedef void* tsb_stream; /* cudaStream_t */

typedef enum tsb_status {
    TSB_OK = 0,
    TSB_ERR_INVALID = 1,     /* bad argument; nothing was enqueued              */
    TSB_ERR_CUDA = 2,        /* a CUDA runtime call failed                       */
    TSB_ERR_UNSUPPORTED = 3, /* shape or format outside what the kernels cover   */
    TSB_ERR_STATE = 4,       /* cursor / ordering contract violated              */
    TSB_ERR_OOM = 5,         /* out of pages or device memory                    */
    TSB_ERR_DEVICE = 6       /* a kernel reported an error word (bounded wait, bad index) */
} tsb_status;

/* Block formats.  The values in parentheses are the dtype tag bytes of the
 * reference's resident weight index (crates/repack/src/resident_writer.rs:105,107,162). */
typedef enum tsb_qtype {
    TSB_Q4_K = 0, /* (7)  256 elements / 144 bytes: crates/compute/src/quant_gguf/q4_k.rs */
    TSB_Q6_K = 1, /* (8)  256 elements / 210 bytes: crates/compute/src/quant_gguf/q6_k.rs */
    TSB_MXFP4 = 2, /* (14) 32 elements / 17 bytes:  crates/compute/src/quant_gguf_mxfp4.rs */
    TSB_Q5_K = 3, /* 256 elements / 176 bytes: crates/compute/src/quant_gguf/q5_k.rs (cols a multiple of 256) */
    TSB_Q8_0 = 4  /* 32 elements / 34 bytes:   crates/compute/src/quant_gguf/q8_0.rs (cols a multiple of 256 here) */
} tsb_qtype;
#define TSB_QTYPE_LAST TSB_Q8_0

/* ------------------------------------------------------------------ context */

/* Replaces MetalContext::new (crates/gpu/src/context/mod.rs): one context per GPU per host thread. */
TSB_API int32_t tsb_ctx_create(int32_t device_ordinal, tsb_ctx** out);
TSB_API void tsb_ctx_destroy(tsb_ctx* ctx);
/* Replaces GpuError's Display (crates/gpu/src/context/error.rs:5-22). */
TSB_API const char* tsb_last_error(const tsb_ctx* ctx);
TSB_API int32_t tsb_device_ordinal(const tsb_ctx* ctx);
/* Device memory owned by the caller (replaces MetalContext buffer allocation). */
TSB_API int32_t tsb_alloc(tsb_ctx* ctx, size_t bytes, void** out_dev);
TSB_API int32_t tsb_free(tsb_ctx* ctx, void* dev);
/* Replaces the resident weight buffer (crates/model-io/src/resident_buffer.rs): raw block bytes, verbatim. */
TSB_API int32_t tsb_weights_upload(tsb_ctx* ctx, const void* host_bytes, size_t bytes, void** out_dev_region);
TSB_API int32_t tsb_memcpy_h2d(tsb_ctx* ctx, tsb_stream s, void* dev, const void* host, size_t bytes);
TSB_API int32_t tsb_memcpy_d2h(tsb_ctx* ctx, tsb_stream s, void* host, const void* dev, size_t bytes);
/* Replaces PassEncoder commit_and_wait_checked (crates/gpu/src/context/pass.rs:180): waits, then
 * surfaces both CUDA errors and the kernels' own error word. */
TSB_API int32_t tsb_stream_sync(tsb_ctx* ctx, tsb_stream s);
/* Every wait inside a kernel (on a copy's arrival barrier) is bounded by
 * time: when the limit runs out the kernel records TSB_ERR_DEVICE's "bounded barrier wait gave up" word, drains and
 * returns, and the context stays usable.  Default 1 s.  Synchronises the device.  (The reference's Metal passes have
 * no device-side waits; its host-side equivalent is the command-buffer status check of
 * crates/gpu/src/context/pass.rs:180.) */
TSB_API int32_t tsb_ctx_set_wait_limit_us(tsb_ctx* ctx, uint32_t microseconds);
/* Test hook: one CTA waits on a barrier nobody arrives on, so the bounded wait runs out.  out_u32_dev receives
 * 1 if the wait reported success (it must not), 0 otherwise; the following tsb_stream_sync returns TSB_ERR_DEVICE. */
TSB_API int32_t tsb_debug_wait_nobody(tsb_ctx* ctx, tsb_stream s, void* out_u32_dev);
/* Bytes one row of `cols` elements occupies in the given format. */
TSB_API int64_t tsb_row_bytes(int32_t qtype, int64_t cols);
/* Number of kernel launches this ctx has enqueued since creation. */
TSB_API uint64_t tsb_launch_count(const tsb_ctx* ctx);

/* ---------------------------------------------------- quantized matmul (hot) */

/* y[t, r] = sum_c W[r, c] * x[t, c],  W = `rows` rows of verbatim blocks at region + w_off,
 * x [tokens, cols] f16, y [tokens, rows] f16 (y_f32 = 0) or f32 (y_f32 = 1), fp32 accumulate.
 * A token's result never depends on the other tokens of the call (row invariance), so a
 * decode step (tokens = 1) and a verify batch produce identical bits per token.
 * Replaces encode_dequant_q4_k_gemv / encode_dequant_q6_k_gemv / encode_dequant_mxfp4_gemv
 * (crates/gpu/src/dequant_q4_k_gemv.rs:110-140, dequant_q6_k_gemv.rs, dequant_ext_gemv.rs:176-201)
 * for tokens = 1 and encode_dequant_kquant_gemm_batch (crates/gpu/src/dequant_kquant_gemm_batch.rs:96-126)
 * for tokens > 1.  cols must be a whole number of blocks (256 for K-quants, 32 for MXFP4). */
TSB_API int32_t tsb_gemm_quant(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off,
                               int64_t rows, int64_t cols, const void* x_f16, void* y, int32_t tokens,
                               int32_t y_f32);
/* tsb_gemm_quant without allocations: the caller owns the operand workspace (tsb_gemm_workspace_bytes, 256-byte
 * aligned).  tsb_gemm_prepare converts token rows x into the layout the matmul kernel reads (the step
 * tsb_gemm_quant does on every call); tsb_gemm_quant_prepared is then the matmul alone and may be repeated over many
 * matrices with the same operand - how the reference reuses one activation buffer across the q, k, v projections
 * (crates/gpu/src/real_forward_dispatch.rs:900-1054).  With 24 token rows and more of a Q4_K matrix whose rows are a
 * multiple of 128 the tensor-memory kernel runs instead; it converts inside its own launch sequence, into the same
 * workspace. */
TSB_API size_t tsb_gemm_workspace_bytes(int32_t qtype, int64_t rows, int64_t cols, int32_t tokens);
TSB_API int32_t tsb_gemm_prepare(tsb_ctx* ctx, tsb_stream s, int32_t qtype, int64_t rows, int64_t cols, const void* x_f16, int32_t tokens,
                                 void* workspace, size_t workspace_bytes);
TSB_API int32_t tsb_gemm_quant_prepared(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off, int64_t rows,
                                        int64_t cols, const void* x_f16, void* workspace, void* y, int32_t tokens, int32_t y_f32);
/* The reference's per-format names, kept so a binding reads like the original call sites. */
TSB_API int32_t tsb_gemv_q4k(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                             int64_t cols, const void* x_f16, void* y_f16);
TSB_API int32_t tsb_gemv_q6k(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                             int64_t cols, const void* x_f16, void* y_f16);
TSB_API int32_t tsb_gemv_mxfp4(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                               int64_t cols, const void* x_f16, void* y_f16);
TSB_API int32_t tsb_gemm_q4k(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                             int64_t cols, const void* x_f16, void* y_f16, int32_t tokens);
TSB_API int32_t tsb_gemm_q6k(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                             int64_t cols, const void* x_f16, void* y_f16, int32_t tokens);
TSB_API int32_t tsb_gemm_mxfp4(tsb_ctx* ctx, tsb_stream s, const void* region, uint64_t w_off, int64_t rows,
                               int64_t cols, const void* x_f16, void* y_f16, int32_t tokens);

/* out[i, :] = dequantized row row_ids[i] (row_ids NULL = rows 0..n-1), fp32, bit-exact with
 * dequantize_q4_k / dequantize_q6_k / dequantize_mxfp4 (crates/compute/src/quant_gguf/q4_k.rs:67-108,
 * q6_k.rs:52-95, quant_gguf_mxfp4.rs:114-141). */
TSB_API int32_t tsb_dequant_rows(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off,
                                 int64_t cols, const int32_t* row_ids, int32_t n_rows, float* out_f32);
/* out[i, :] = f16(dequantized row token_ids[i] * out_scale).  Replaces encode_embed_lookup_q4_k /
 * _mxfp4 (crates/gpu/src/shaders/dequant_q4_k.metal:142-169, dequant_ext.metal:176-189). */
TSB_API int32_t tsb_embed_rows(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* region, uint64_t w_off,
                               int64_t vocab_rows, int64_t cols, const int32_t* token_ids, int32_t n, void* out_f16,
                               float out_scale);

/* ------------------------------------------------------------ row operators */

/* out[r,:] = f16( x[r,:] * rsqrt(mean(x^2) + eps) * w ), w bf16.  If residual != NULL, x[r,:] is first
 * replaced by f16(x + residual) (the reference's residual_add_fp16 followed by rmsnorm_bf16w).
 * Replaces encode_rms_norm rows variant (crates/gpu/src/shaders/rmsnorm.metal:70-95) and
 * residual_add_fp16 (utility.metal:199-208). */
TSB_API int32_t tsb_rmsnorm_rows(tsb_ctx* ctx, tsb_stream s, void* x_f16, const void* residual_f16,
                                 const void* w_bf16, void* out_f16, int32_t rows, int32_t d, float eps);
/* NeoX RoPE in place with one position per row: pairs (i, head_dim/2 + i), i < rotated_pairs, angle
 * pos * theta^(-2i/head_dim).  x is [rows, row_stride] f16 with `heads` heads of head_dim at the start of
 * each row.  Replaces encode_rope_neox_subdim_rows_positions (crates/gpu/src/shaders/rope.metal:80-180). */
TSB_API int32_t tsb_rope_neox_rows_positions(tsb_ctx* ctx, tsb_stream s, void* x_f16, int32_t rows, int32_t heads,
                                             int32_t head_dim, int32_t rotated_pairs, int64_t row_stride,
                                             const int32_t* positions, float theta);
/* out = f16( silu(gate) * up ).  gate/up/out are [rows, n] with the given row strides (elements).
 * Replaces silu_mul_fp16 (utility.metal:41-52). */
TSB_API int32_t tsb_silu_mul(tsb_ctx* ctx, tsb_stream s, const void* gate_f16, const void* up_f16, void* out_f16,
                             int32_t rows, int32_t n, int64_t in_stride, int64_t out_stride);
/* x = f16(x + y).  Replaces residual_add_fp16 (utility.metal:199-208). */
TSB_API int32_t tsb_residual_add(tsb_ctx* ctx, tsb_stream s, void* x_f16, const void* y_f16, int64_t n);

/* ------------------------------------------------------------ paged KV cache */

/* An fp16 K/V cache for `layers` layers shared by up to max_seqs independent streams.  Storage is a
 * pool of pages of page_tokens positions (a power of two >= 16); a stream's logical position p lives in
 * page table[seq][p / page_tokens].  Replaces KvCacheManager (crates/gpu/src/kv_cache.rs:47-69,292-378),
 * which is one linear buffer per layer; paging is this backend's addition for many streams. */
TSB_API int32_t tsb_kv_create(tsb_ctx* ctx, int32_t layers, int32_t kv_heads, int32_t head_dim,
                              int32_t page_tokens, int32_t num_pages, int32_t max_seqs, int32_t max_pages_per_seq,
                              tsb_kv** out);
TSB_API void tsb_kv_destroy(tsb_kv* kv);
/* Make positions [0, tokens) of stream `seq` addressable (allocates pages; host side). */
TSB_API int32_t tsb_kv_reserve(tsb_kv* kv, int32_t seq, int64_t tokens);
/* Release every page of a stream and zero its cursor. */
TSB_API int32_t tsb_kv_reset(tsb_kv* kv, int32_t seq);
/* Cursor = number of committed positions.  Replaces KvCacheManager::position / advance. */
TSB_API int64_t tsb_kv_cursor(const tsb_kv* kv, int32_t seq);
TSB_API int32_t tsb_kv_set_cursor(tsb_kv* kv, int32_t seq, int64_t position);
/* Replaces rewind_by (crates/gpu/src/kv_cache_rewind.rs:46-55): a cursor move; rows are overwritten later. */
TSB_API int32_t tsb_kv_rewind_by(tsb_kv* kv, int32_t seq, int64_t count);
/* Copy rows [pos0, pos0+n) of one layer to/from host, [n, kv_heads*head_dim] f16 (tests, prefix import). */
TSB_API int32_t tsb_kv_write_rows(tsb_kv* kv, tsb_stream s, int32_t seq, int32_t layer, int64_t pos0, int32_t n,
                                  const void* host_k_f16, const void* host_v_f16);
TSB_API int32_t tsb_kv_read_rows(tsb_kv* kv, tsb_stream s, int32_t seq, int32_t layer, int64_t pos0, int32_t n,
                                 void* host_k_f16, void* host_v_f16);
/* Fill positions [0, tokens) of every layer of a stream with seeded pseudo-random f16 values in
 * roughly N(0,1) (benchmark set-up: a pre-filled context without a prefill pass). */
TSB_API int32_t tsb_kv_fill_random(tsb_kv* kv, tsb_stream s, int32_t seq, int64_t tokens, uint64_t seed);

/* One row of a verify (or decode) batch, as the attention and KV-store kernels see it. */
typedef struct tsb_row_desc {
    int32_t seq;      /* stream the row belongs to                                      */
    int32_t base;     /* committed prefix length: positions [0, base) are all attended   */
    int32_t slot;     /* the row's own in-flight slot j: its K/V go to position base + j */
    int32_t position; /* RoPE position (base + depth)                                    */
    uint64_t mask[2]; /* bit j set = in-flight slot j is an ancestor-or-self of this row */
} tsb_row_desc;

/* Rotate q and k (NeoX, per-row position) and store k, v into the cache at each row's slot.
 * qkv is [rows, (nq + 2*nkv) * head_dim] f16 (q heads, then k heads, then v heads); q is rotated in
 * place.  Replaces the K/V projection's direct cache write plus encode_rope on Q and on the cached K
 * (crates/runtime/src/families/llama/attn.rs:175-210,280-367). */
TSB_API int32_t tsb_rope_store_kv(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, void* qkv_f16,
                                  const tsb_row_desc* rows_dev, int32_t rows, int32_t n_q_heads, float theta);

/* Split-KV decode attention for a batch of rows.  Rows are grouped per stream: rows_per_seq
 * consecutive rows belong to one stream, share `seq` and `base`, and are ordered by slot (row j of a
 * group has slot j).  Row r attends to its stream's committed prefix [0, base) and to the in-flight
 * slots its mask names (a chain row m has bits 0..m; a tree row has its root path).  q is
 * [rows, q_stride] f16 with nq*head_dim values at the start of each row, out [rows, nq*head_dim] f16.
 * max_len bounds base + rows_per_seq over the batch (it sizes the split; the kernels read the true
 * lengths from the descriptors).  scratch must hold tsb_attn_scratch_bytes(...) bytes.  Replaces
 * encode_attention_decode, encode_attention_decode_tree and the combine pass
 * (crates/gpu/src/attention_decode.rs:920-1046,1153-1230; shaders/attention.metal:285-446,983-1031). */
TSB_API int32_t tsb_attn_decode_rows(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, const void* q_f16,
                                     int64_t q_stride, void* out_f16, const tsb_row_desc* rows_dev, int32_t rows,
                                     int32_t rows_per_seq, int32_t n_q_heads, float scale, int32_t max_len,
                                     void* scratch, size_t scratch_bytes);
TSB_API size_t tsb_attn_scratch_bytes(int32_t rows, int32_t n_q_heads, int32_t head_dim);

/* The same attention for callers that cannot supply scratch memory: a binding that owns no device
 * allocator (it only forwards buffers it was handed), or a caller that must not allocate where the
 * call sits.  It has no counterpart in the reference, whose encoders always take caller buffers.
 * The chunk partials go to a fixed area of TSB_ATTN_STATIC_SCRATCH_BYTES that is part of the loaded
 * library, one copy per device; the call allocates nothing, on the host's heap or on the device.
 *  - A shape needing more than that (tsb_attn_scratch_bytes(rows, n_q_heads, head_dim) bytes) is
 *    refused with TSB_ERR_INVALID and a message naming both sizes; nothing is launched.
 *  - The first call on each device looks the area's address up once; make that call before any
 *    stream capture is begun on that device.
 *  - All calls on a device share the one area and it keeps what the previous call left.  The
 *    call clears the words that must start at zero itself, in stream order.  Two calls that may
 *    overlap in time (different streams, different threads) race on the area: keep such calls on
 *    one stream, or use tsb_attn_decode_rows with separate buffers.
 * Results equal tsb_attn_decode_rows on the same inputs. */
#define TSB_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
TSB_API int32_t tsb_attn_decode_rows_static(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t layer, const void* q_f16,
                                            int64_t q_stride, void* out_f16, const tsb_row_desc* rows_dev,
                                            int32_t rows, int32_t rows_per_seq, int32_t n_q_heads, float scale,
                                            int32_t max_len);

/* In-place compaction of an accepted tree path: for every layer and for K and V, row base+r <- row
 * base+path[r], r < keep.  path[0] must be 0 and path strictly increasing (so path[r] >= r): the only
 * shape for which an in-place gather is race-free.  Replaces encode_gather_rows_fp16 driven by
 * dflash_tree_compact (crates/gpu/src/dflash_conv.rs:199-259, crates/runtime/src/families/qwen/dflash_tree.rs:106-207). */
TSB_API int32_t tsb_kv_commit_path(tsb_ctx* ctx, tsb_stream s, tsb_kv* kv, int32_t seq, int64_t base,
                                   const uint32_t* host_path, int32_t keep);

/* --------------------------------------------------------------- acceptance */

/* crates/selection/src/shaping.rs:40-50.  top_p <= 0 and min_p <= 0 mean "off". */
typedef struct tsb_shaping {
    double temperature;
    uint32_t top_k;
    uint32_t _pad;
    double top_p;
    double repetition_penalty;
    double presence_penalty;
    double frequency_penalty;
    double min_p;
    uint64_t seed;
} tsb_shaping;

typedef struct tsb_accept_out {
    int32_t accepted;     /* accepted prefix length                                      */
    int32_t draws;        /* uniforms consumed                                           */
    int32_t tokens[16];   /* accepted proposals, then the corrected / bonus token        */
    int32_t status;       /* 0 ok, 1 non-finite logit                                     */
    int32_t _pad;
    double margin_accept; /* min |r*q(x) - p(x)| over tested proposals                    */
    double margin_draw;   /* distance from the uniform to the nearest cumulative boundary */
} tsb_accept_out;

/* One round's acceptance for `batch` independent streams, on the device.  Per stream b:
 * target_logits [(k+1), V] f16, draft_logits [k, V] f16, proposals [k], uniforms [2k+1] u64 (the
 * values derive_step_value would give for consecutive draw steps; mapped through the top-53-bit rule).
 * For each proposal: accept iff r*q(x) <= p(x) over the shaped distributions; on rejection draw the
 * corrected token from the normalised max(p-q, 0) in p's rank order (from p when the residual mass is
 * below 1e-12); on full acceptance draw the bonus from the last row.  temperature 0 = argmax equality.
 * Replaces the host-side accept step of the round loop (crates/runtime/src/speculative.rs:694-754,
 * 861-879) and select / shaped_distribution / residual (crates/selection/src/choose.rs:62-232,
 * distribution.rs:57-125).  Temperature, top_k (<= 256), top_p and min_p are applied on the device (the support is
 * the reference's rank-order prefix); repetition, presence and frequency penalties need the token history: this entry
 * point refuses them with TSB_ERR_UNSUPPORTED, tsb_accept_history applies them. */
TSB_API int32_t tsb_accept(tsb_ctx* ctx, tsb_stream s, const void* target_logits_f16, const void* draft_logits_f16,
                           const int32_t* proposals, const uint64_t* uniforms, int32_t batch, int32_t k,
                           int32_t vocab, const tsb_shaping* shaping, tsb_accept_out* out_dev, void* scratch,
                           size_t scratch_bytes);
TSB_API size_t tsb_accept_scratch_bytes(int32_t batch, int32_t k, int32_t vocab);

/* token[b] = draw from the shaped distribution of logits[b, :] with uniforms[b] (argmax at temperature 0).
 * Replaces select / ShapedDistribution::draw on the draft side (crates/runtime/src/speculative.rs:636-659). */
TSB_API int32_t tsb_sample(tsb_ctx* ctx, tsb_stream s, const void* logits_f16, const uint64_t* uniforms,
                           int32_t batch, int32_t vocab, const tsb_shaping* shaping, int32_t* tokens_dev,
                           double* margins_dev, void* scratch, size_t scratch_bytes);

/* tsb_accept / tsb_sample with the history penalties of the shaping record (crates/selection/src/penalty.rs:15-82,
 * applied at choose.rs:139-154 before the softmax): repetition_penalty attenuates every distinct id of the history
 * once (s > 0 ? s / penalty : s * penalty, in f32), presence_penalty + frequency_penalty * count is subtracted for
 * every distinct id of the GENERATED suffix of the history.  Per stream b: history_dev[b * hist_stride + j] for
 * j < hist_len_dev[b] is the committed stream (prompt, then what this turn generated, the confirmed token that
 * entered the round included), generated_dev[b] how many of its last entries this turn generated.  Which history a
 * row sees follows the round loop (crates/runtime/src/speculative.rs:636-648,701-734): a drafter row was shaped with
 * the history of the round's start, target row i after proposals 0..i were committed (they count as history and as
 * generated).  With the identity penalties the results equal tsb_accept / tsb_sample.  All arrays are device memory;
 * scratch: tsb_accept_history_scratch_bytes(batch, k, vocab) (k = 0 for tsb_sample_history). */
TSB_API int32_t tsb_accept_history(tsb_ctx* ctx, tsb_stream s, const void* target_logits_f16, const void* draft_logits_f16,
                                   const int32_t* proposals, const uint64_t* uniforms, int32_t batch, int32_t k, int32_t vocab,
                                   const tsb_shaping* shaping, const int32_t* history_dev, int32_t hist_stride,
                                   const int32_t* hist_len_dev, const int32_t* generated_dev, tsb_accept_out* out_dev,
                                   void* scratch, size_t scratch_bytes);
TSB_API int32_t tsb_sample_history(tsb_ctx* ctx, tsb_stream s, const void* logits_f16, const uint64_t* uniforms, int32_t batch,
                                   int32_t vocab, const tsb_shaping* shaping, const int32_t* history_dev, int32_t hist_stride,
                                   const int32_t* hist_len_dev, const int32_t* generated_dev, int32_t* tokens_dev,
                                   double* margins_dev, void* scratch, size_t scratch_bytes);
TSB_API size_t tsb_accept_history_scratch_bytes(int32_t batch, int32_t k, int32_t vocab);

/* Uniform sources: mode 0 = derive_step_value(seed, step) (crates/selection/src/derive.rs:20-48),
 * mode 1 = Philox4x32-10 keyed by seed with counter = step (this backend's addition). */
TSB_API uint64_t tsb_uniform_u64(int32_t mode, uint64_t seed, uint64_t step);

/* ------------------------------------------------------ mixture of experts */

/* Routing of `tokens` rows over n_experts router logits (f32, [tokens, n_experts]): the k (<= 8) largest logits,
 * ties to the lower expert index, softmax over the selected logits only, times per_expert_scale (null = ones);
 * ids_out [tokens, k] in rank order, weights [tokens, k] as f16.  Replaces router_topk_gemma4
 * (crates/runtime/src/real_forward_dispatch.rs:1135-1158) and the f16 routing-weight upload
 * (crates/runtime/src/families/llama/moe.rs:118-127). */
TSB_API int32_t tsb_moe_route(tsb_ctx* ctx, tsb_stream s, const float* router_logits_f32, int32_t tokens, int32_t n_experts,
                              int32_t k, const float* per_expert_scale, int32_t* ids_out, void* weights_f16_out);
/* The routed feed-forward: for every row, y = half(residual + sum over its k slots, in slot order, of
 * float(weight) * down_e(half(act(gate_e x) * (up_e x)))).  Expert e's gate rows then up rows sit at
 * gate_up_region + gate_up_off + e * (2*ffn rows of d_model columns), its down rows at down_region + down_off +
 * e * (d_model rows of ffn columns), all verbatim blocks of `qtype`.  x, residual and y are [tokens, d_model] f16;
 * ids / weights come from tsb_moe_route.  Nothing comes back to the host: a device kernel sorts the (row, slot) pairs
 * into per-expert tiles, one grouped launch of the matmul kernel per phase covers every active expert, and an expert
 * id outside the table sets the context's device error word (reported by tsb_stream_sync).  Replaces
 * moe_phase1_gate_up_act_* and moe_phase2_down_reduce_k8_* (crates/gpu/src/shaders/moe_gguf.metal:561-678). */
TSB_API int32_t tsb_moe_ffn(tsb_ctx* ctx, tsb_stream s, int32_t qtype, const void* gate_up_region, uint64_t gate_up_off,
                            const void* down_region, uint64_t down_off, int32_t n_experts, int32_t d_model, int32_t ffn,
                            const void* x_f16, const void* residual_f16, const int32_t* ids_dev, const void* weights_f16_dev,
                            int32_t tokens, int32_t k, void* y_f16);

/* ------------------------------------------------------ model and producer */

/* A dense Llama-style decoder (RMSNorm -> q/k/v -> RoPE -> attention -> o_proj -> residual -> RMSNorm ->
 * gate/up -> SiLU*up -> down -> residual; final RMSNorm + lm_head): the op order of
 * crates/runtime/src/families/llama/mod.rs:205-291 and dense.rs:48-120. */
typedef struct tsb_model_config {
    int32_t n_layers, d_model, n_q_heads, n_kv_heads, head_dim, ffn, vocab, max_context;
    float rms_eps, rope_theta;
} tsb_model_config;

enum { TSB_W_Q = 0, TSB_W_K, TSB_W_V, TSB_W_O, TSB_W_GATE, TSB_W_UP, TSB_W_DOWN, TSB_W_EMBED, TSB_W_LM_HEAD };
enum { TSB_N_ATTN = 0, TSB_N_FFN, TSB_N_OUT };

TSB_API int32_t tsb_model_create(tsb_ctx* ctx, const tsb_model_config* cfg, tsb_model** out);
TSB_API void tsb_model_destroy(tsb_model* m);
/* Upload one matrix as verbatim block rows (rows x cols, row-major rows of blocks).  q and k of a layer
 * must share a format, as must gate and up: they are laid out back to back and run as one matmul.  v joins
 * q and k when its format is theirs; otherwise (mixed recipes keep v in Q6_K) it runs as a launch of its own.
 * layer is ignored for TSB_W_EMBED / TSB_W_LM_HEAD.  A model may point its embedding and head at another
 * model's tensors with tsb_model_share (a drafter sharing the trunk's tables). */
TSB_API int32_t tsb_model_set_matrix(tsb_model* m, int32_t layer, int32_t which, int32_t qtype,
                                     const void* host_blocks, int64_t rows, int64_t cols);
TSB_API int32_t tsb_model_set_norm(tsb_model* m, int32_t layer, int32_t which, const void* host_bf16, int32_t n);
/* dst layer `dst_layer` uses src layer `src_layer`'s tensors (no copy); layer < 0 shares embedding, final
 * norm and head.  src must outlive dst. */
TSB_API int32_t tsb_model_share(tsb_model* dst, int32_t dst_layer, const tsb_model* src, int32_t src_layer);
/* Fill every tensor with seeded synthetic blocks directly on the device (benchmark set-up: weights of the
 * right shapes and formats without a host copy; values are valid blocks with small scales). */
TSB_API int32_t tsb_model_fill_synthetic(tsb_model* m, int32_t qtype, int32_t lm_head_qtype, uint64_t seed);
TSB_API int64_t tsb_model_weight_bytes(const tsb_model* m);
/* Routed feed-forward (the llama family's MoE layers: crates/runtime/src/families/llama/moe.rs:36-221, router
 * families/llama/router.rs:12-66).  tsb_model_set_moe, called before any tensor is uploaded, makes every layer's
 * feed-forward routed: n_experts experts of width moe_ffn, top_k per token (the config's dense `ffn` is then
 * unused and gate / up / down are not uploaded).  The router is the reference's 8-bit affine matrix: u8
 * [n_experts, d_model] with bf16 scale and bias per 64 columns (dtype tag 5); experts are verbatim block rows,
 * per expert gate rows then up rows [2 moe_ffn, d_model], and down rows [d_model, moe_ffn]. */
TSB_API int32_t tsb_model_set_moe(tsb_model* m, int32_t n_experts, int32_t top_k, int32_t moe_ffn);
TSB_API int32_t tsb_model_set_router(tsb_model* m, int32_t layer, const void* q_u8, const void* scale_bf16, const void* bias_bf16);
TSB_API int32_t tsb_model_set_experts(tsb_model* m, int32_t layer, int32_t qtype, const void* gate_up_blocks,
                                      const void* down_blocks);
/* router_gemv_gemma4 (crates/gpu/src/moe_decode.rs:491-530, shaders/moe.metal:107-145) with the all-ones
 * effective scale: logits[t, e] = sum over 64-column groups of fma(s, q.x, .) and fma(b, sum x, .), f32. */
TSB_API int32_t tsb_router_logits(tsb_ctx* ctx, tsb_stream s, const void* q_u8, const void* scale_bf16, const void* bias_bf16,
                                  const void* x_f16, int32_t tokens, int32_t n_experts, int32_t d_model, float* logits_out);

/* ------------------------------------------------------------------ resident weight file
 * The leading index region of the reference's resident weight file: 24-byte header, 72-byte entries, string
 * table, optional "GTURBIDX" format trailer (crates/model-io/src/resident_index.rs:19-67, load at :131-283,
 * trailer check at :289-317; written by crates/repack/src/resident_writer.rs:375-470).  Host code only: these
 * calls need no device.  Errors go to tsb_resident_last_error() (per thread): a malformed index answers
 * TSB_ERR_INVALID with "index corrupt: ..." (ModelError::IndexCorrupt), a trailer naming another format version
 * answers TSB_ERR_UNSUPPORTED (ModelError::UnsupportedIndexFormat). */
typedef struct tsb_resident tsb_resident;
typedef struct tsb_resident_entry { /* ResidentIndexEntry, resident_index.rs:47-66 */
    uint8_t dtype;                  /* dtype tag byte (crates/repack/src/resident_writer.rs:80-162) */
    uint8_t _pad[3];
    uint32_t shape[4];              /* rank padded to 4 */
    uint64_t file_offset;           /* absolute file offset of the payload (>= index size) */
    uint64_t size_bytes;
    uint64_t scale_offset, scale_size, bias_offset, bias_size; /* zero for the block formats */
} tsb_resident_entry;
TSB_API int32_t tsb_resident_open(const char* path, tsb_resident** out);
TSB_API void tsb_resident_close(tsb_resident* idx);
TSB_API const char* tsb_resident_last_error(void);
TSB_API int64_t tsb_resident_count(const tsb_resident* idx);
TSB_API uint64_t tsb_resident_index_size(const tsb_resident* idx); /* tensor bytes start here */
TSB_API uint64_t tsb_resident_data_size(const tsb_resident* idx);
TSB_API int32_t tsb_resident_entry_at(const tsb_resident* idx, int64_t i, tsb_resident_entry* out, char* name_buf, int32_t name_cap);
TSB_API int32_t tsb_resident_find(const tsb_resident* idx, const char* name, tsb_resident_entry* out);
/* dtype tag -> tsb_qtype (7 Q4_K, 8 Q6_K, 14 MXFP4, 13 Q5_K, 6 Q8_0), -1 for anything else */
TSB_API int32_t tsb_resident_qtype_of(int32_t dtype_tag);
/* Upload the Llama-family tensor set the reference's runner looks up by name (embed_tokens, per layer
 * input_layernorm / self_attn.{q,k,v,o}_proj / post_attention_layernorm / mlp.{gate,up,down}_proj, model.norm,
 * lm_head or the embedding again when tied: crates/runtime/src/families/llama/mod.rs:49-51,99,371-386) from the
 * file into `m`, blocks verbatim.  A tensor whose byte count does not match its format and the model's shape
 * is refused (real_forward_dispatch.rs:1008-1016), as is a dtype outside the block formats. */
TSB_API int32_t tsb_model_load_resident(tsb_model* m, const tsb_resident* idx, int32_t tie_word_embeddings);

/* ------------------------------------------------- sharding one routed model over the GPUs of a box
 * The reference runs on one Apple GPU and has no counterpart; the shapes follow its routed layer
 * (crates/runtime/src/families/llama/moe.rs:36-221).  One process per GPU.  Attention is tensor-parallel over heads:
 * a rank's model is built with ITS heads only (n_q_heads / world query heads and the K/V heads they read, a K/V head
 * being replicated where world exceeds the K/V head count), its o_proj matrix holds the matching head columns, and the
 * partial projections are summed over the ranks (f32 all-reduce).  Experts are sharded: a rank holds experts
 * [expert_lo, expert_lo + n_local) of every layer, computes the (row, slot) outputs routed to them and leaves zeros
 * for the rest; the f32 all-reduce of those per-slot outputs adds only zeros to each value, so every rank then holds
 * exactly what one GPU computes and the slot-ordered weighted sum is bit-identical on all ranks.  Router, norms,
 * embedding and head are replicated.  The collectives are NCCL calls on the session's stream; NCCL is loaded at run
 * time (TSB_NCCL_LIB overrides the library name). */
/* Rank 0 makes the id, the host program hands the 128 bytes to every rank (any channel), every rank creates. */
TSB_API int32_t tsb_comm_unique_id(tsb_ctx* ctx, void* out_128_bytes);
TSB_API int32_t tsb_comm_create(tsb_ctx* ctx, const void* unique_id_128_bytes, int32_t rank, int32_t world, tsb_comm** out);
TSB_API void tsb_comm_destroy(tsb_comm* c);
/* In-place sum over the ranks of `count` f32 values (the exchange step itself, as an operator). */
TSB_API int32_t tsb_comm_all_reduce_f32(tsb_comm* c, tsb_stream s, void* buf_f32_dev, size_t count);
/* This rank's experts: set after tsb_model_set_moe and before the expert tensors, which then hold n_local experts. */
TSB_API int32_t tsb_model_set_expert_shard(tsb_model* m, int32_t expert_lo, int32_t n_local);
/* The session's passes exchange through `c` (NULL: single GPU).  Every rank must run the same passes in the same
 * order with the same rows. */
TSB_API int32_t tsb_session_set_comm(tsb_session* s, tsb_comm* c);

/* A session = the producer: a target model, an optional stand-alone draft model, paged K/V caches for
 * `n_streams` independent request streams, and every activation / logits / scratch buffer a round
 * needs for up to `max_rows` rows per stream.  Mirrors what RealForwardRunner owns
 * (crates/runtime/src/real_forward_traits.rs:6-60). */
TSB_API int32_t tsb_session_create(tsb_ctx* ctx, const tsb_model* target, const tsb_model* draft, int32_t n_streams,
                                   int32_t max_rows, int32_t page_tokens, tsb_session** out);
TSB_API void tsb_session_destroy(tsb_session* s);
TSB_API tsb_kv* tsb_session_kv(tsb_session* s, int32_t which_model /* 0 target, 1 draft */);
/* Number of kernel launches / CUDA-graph launches issued so far by this session's ctx is tsb_launch_count. */

/* LogitProducer / SpeculativeProducer, one stream at a time (crates/runtime/src/producer.rs:17-104,164-387).
 * logits_out_host: vocab f16 values per row, or NULL to leave them on the device.  Errors keep the
 * reference's contract: a call that violates the cursor is refused and changes nothing. */
TSB_API int32_t tsb_producer_reset(tsb_session* s, int32_t stream);
TSB_API int32_t tsb_producer_produce(tsb_session* s, int32_t stream, int32_t token, int64_t position, void* logits_out_host);
TSB_API int32_t tsb_producer_produce_prefill(tsb_session* s, int32_t stream, int32_t token, int64_t position);
TSB_API int32_t tsb_producer_prime_drafter(tsb_session* s, int32_t stream, int32_t next, int64_t position);
TSB_API int32_t tsb_producer_draft_step(tsb_session* s, int32_t stream, int32_t next, int64_t position, void* logits_out_host);
TSB_API int32_t tsb_producer_verify(tsb_session* s, int32_t stream, const int32_t* feed, int32_t n, int64_t base,
                                    void* logits_out_host);
/* verify_tree: feed[0] is the anchor, slot_parent[0] = -1 and parents precede children
 * (crates/runtime/src/families/qwen/batched_scratch.rs:97-124). */
TSB_API int32_t tsb_producer_verify_tree(tsb_session* s, int32_t stream, const int32_t* feed, const int32_t* slot_parent,
                                         int32_t n, int64_t base, void* logits_out_host);
/* compact_tree (producer.rs:287-291): moves the accepted path's slots (path[0] == 0, increasing) to rows 0..keep of
 * the verify, in the target's cache and - for the slots the drafter ran over - in the drafter's; the record of fed
 * tokens takes the path's tokens from the last verify_tree. */
TSB_API int32_t tsb_producer_compact_tree(tsb_session* s, int32_t stream, int64_t base, const uint32_t* path, int32_t keep);
/* One node of a drafted tree (crates/runtime/src/dflash_tree.rs:10-16): candidate `cand` at `depth` below the anchor,
 * under node `parent` (-1 for a child of the anchor).  Node i sits in slot i + 1 of the verify. */
typedef struct tsb_tree_node {
    int32_t depth, cand, parent;
} tsb_tree_node;
/* The trees this session's producer drafts: `nodes` drafted nodes per round in at most `levels` levels.  best_first
 * == 0: the static shape in which every node of level l gets its branching[l] most likely next tokens, cut
 * breadth-first at `nodes`.  best_first == 1: grown by path probability (dflash_best_first_tree,
 * crates/runtime/src/dflash_tree.rs:30-82) with `cand` (1..8) candidates scored under every expanded node - a
 * parent's children share a softmax over the drafter's logits of those candidates.  nodes == 0 turns trees off. */
TSB_API int32_t tsb_session_set_tree(tsb_session* s, int32_t nodes, int32_t levels, const int32_t* branching /* [levels], may be NULL when best_first */,
                                     int32_t best_first, int32_t cand);
/* tree_nodes (producer.rs:256-262): nodes per tree round, 0 when the producer verifies chains only. */
TSB_API int32_t tsb_producer_tree_nodes(const tsb_session* s);
/* draft_tree (producer.rs:264-275): a tree of up to `nodes` nodes anchored at `anchor` (the token at `base`), parents
 * before children; tokens_out[i] is node i's token.  Greedy drafter picks (the reference runs tree rounds at
 * temperature 0 only).  The drafter's cursor stays at `base`. */
TSB_API int32_t tsb_producer_draft_tree(tsb_session* s, int32_t stream, int32_t anchor, int64_t base, int32_t nodes,
                                        tsb_tree_node* tree_out, int32_t* tokens_out, int32_t* n_out);
/* dflash_tree_slot_parents (dflash_tree.rs:117-124): slot 0 is the anchor (-1), node i sits at slot i + 1 under its
 * parent's slot.  out has n + 1 entries. */
TSB_API int32_t tsb_tree_slot_parents(const tsb_tree_node* tree, int32_t n, int32_t* out);
/* dflash_best_first_tree over a fixed score table scores[depth * branch + cand] (the shape the reference's own tests
 * use, dflash_tree.rs:130-190): returns the number of nodes written. */
TSB_API int32_t tsb_best_first_tree(const float* scores, int32_t depth_max, int32_t branch, int32_t nodes, tsb_tree_node* out);
/* dflash_tree_accept (dflash_tree.rs:92-115): from the anchor, step into the child whose token is the target's pick
 * at the current node's row while there is one.  target_pick has n + 1 entries (slot order).  Returns the number of
 * accepted node ids written to accepted_out. */
TSB_API int32_t tsb_tree_accept(const tsb_tree_node* tree, const int32_t* tokens, int32_t n, const int32_t* target_pick, int32_t* accepted_out);
/* draft_block (producer.rs:236-254): `block` proposals for positions base + 1 ..= base + block in one call, the
 * drafter's greedy picks, each fed back as the next step's input (the last step is taken for its cache row alone, as
 * the step-wise loop does).  drafts_block_passes answers 0: the round loop of this library drives draft_step. */
TSB_API int32_t tsb_producer_draft_block(tsb_session* s, int32_t stream, int32_t anchor, int64_t base, int32_t block,
                                         int32_t* proposals_out);
TSB_API int32_t tsb_producer_drafts_block_passes(const tsb_session* s);
/* commit_pending / discard_pending (producer.rs:332-350).  A verify leaves its rows pending until the round's outcome
 * is known.  commit_pending(keep_rows) closes a round that kept `keep_rows` rows (nothing is deferred here - K/V rows
 * are final when written - so it only checks the count and clears the mark; a no-op when nothing is pending).
 * discard_pending rewinds the target's cursor and the record of fed tokens to where the verify started and the
 * drafter to at most one row past it; the loops call it when a round fails between verify and commit. */
TSB_API int32_t tsb_producer_commit_pending(tsb_session* s, int32_t stream, int32_t keep_rows);
TSB_API int32_t tsb_producer_discard_pending(tsb_session* s, int32_t stream);
/* supports_retaining_rollback (producer.rs:352-358): 1 - a pure-attention cache keeps rows in place.
 * supports_headless_prefill (producer.rs:306-322): 1 - the drafter is a stand-alone decoder that reads nothing of
 * the trunk's final norm. */
TSB_API int32_t tsb_producer_supports_retaining_rollback(const tsb_session* s);
TSB_API int32_t tsb_producer_supports_headless_prefill(const tsb_session* s);
TSB_API int64_t tsb_producer_checkpoint(tsb_session* s, int32_t stream);
TSB_API int32_t tsb_producer_rollback(tsb_session* s, int32_t stream, int64_t point);
TSB_API int32_t tsb_producer_rollback_retaining(tsb_session* s, int32_t stream, int64_t point, int32_t keep_rows);
TSB_API int32_t tsb_producer_rewind_drafter(tsb_session* s, int32_t stream, int64_t position);
/* try_reuse_prefix (crates/runtime/src/producer.rs:21-47): commit to continuing from the stream's current state for
 * the leading N tokens of the prompt and return N (at most n - 1, so the last prompt token is always fed for its
 * logits).  Keyed on the token ids that were actually fed; cursors past the agreed prefix are moved back to it. */
TSB_API int64_t tsb_producer_try_reuse_prefix(tsb_session* s, int32_t stream, const int32_t* prompt_ids, int32_t n);
/* record_committed (crates/runtime/src/producer.rs:324-330): the tokens a round committed, at pos0, for later
 * prefix reuse.  The loops of this library keep that record themselves; the call is for callers that drive the
 * producer functions directly. */
TSB_API int32_t tsb_producer_record_committed(tsb_session* s, int32_t stream, const int32_t* tokens, int32_t n, int64_t pos0);

/* Generation settings of the round loop (crates/runtime/src/config.rs GenerationConfig, reduced to what
 * the loop reads without a tokenizer). */
typedef struct tsb_run_config {
    tsb_shaping shaping;
    int32_t max_new_tokens;
    int32_t block;        /* proposals per round, 1..=15 (crates/core/src/runtime_config.rs:43) */
    int32_t uniform_mode; /* 0 derive_step_value, 1 Philox4x32-10 */
    int32_t n_stop;
    int32_t stop_tokens[8];
    int32_t adaptive;     /* 0 = fixed depth, else the adaptive controller's floor */
    /* Tree rounds (crates/runtime/src/speculative.rs:461-560).  tree_nodes > 0 turns them on for rounds that are
     * neither truncated nor adaptive: a static tree is drafted level by level - every node of level l gets the
     * tree_branching[l] most likely next tokens of the drafter at that node - and cut breadth-first at tree_nodes
     * nodes; `block` must equal tree_levels (the longest path a round can accept).  The target verifies anchor +
     * nodes in one pass with the ancestor mask, the walk accepts a child that carries the target's pick, and the
     * accepted path is compacted in place.  Temperature must be 0 (the reference refuses sampled tree rounds). */
    int32_t tree_nodes, tree_levels;
    int32_t tree_branching[8];
    /* 1: keep what the stream's caches already hold for the longest prefix of the prompt whose token ids equal the
     * ids that were fed (try_reuse_prefix, crates/runtime/src/producer.rs:21-47) instead of resetting the stream */
    int32_t reuse_prefix;
    /* 1: tree rounds grow their tree best-first (dflash_best_first_tree) with tree_cand candidates per expanded node
     * and at most tree_levels levels, instead of the static branching shape */
    int32_t tree_best_first, tree_cand;
} tsb_run_config;

typedef struct tsb_run_result {
    int32_t new_tokens, reason /* 0 max tokens, 1 stop token */, rounds, accepted_total, rollbacks, history_len;
    int32_t reused_prefix; /* prompt tokens whose cache rows were kept from the previous run */
    int32_t _pad;
    int64_t kv_position;
    uint64_t draws;
    double prefill_seconds, decode_seconds;
} tsb_run_result;

/* run_raw_completion_speculative (crates/runtime/src/speculative.rs:54-940) for one stream: prefill,
 * then rounds of draft / verify / accept / rollback / commit with the acceptance on the device.
 * out_tokens receives prompt + committed history (kv_backed_token_ids), out_emitted every generated
 * token (the stopping one included).  Refuses an empty prompt, a zero budget, prompt + budget beyond the
 * context window and block == 0, as the reference does (crates/runtime/src/raw_completion.rs:126-146,
 * speculative.rs:208-212). */
TSB_API int32_t tsb_spec_run(tsb_session* s, int32_t stream, const int32_t* prompt, int32_t n_prompt,
                             const tsb_run_config* cfg, int32_t* out_tokens, int32_t* out_emitted, tsb_run_result* res);
/* run_raw_completion (crates/runtime/src/raw_completion.rs:300-420): the sequential loop the speculative
 * one must reproduce token for token at temperature 0. */
TSB_API int32_t tsb_sequential_run(tsb_session* s, int32_t stream, const int32_t* prompt, int32_t n_prompt,
                                   const tsb_run_config* cfg, int32_t* out_tokens, int32_t* out_emitted, tsb_run_result* res);

/* One speculative round for every stream of the session in lockstep (the benchmark's step and the
 * serving inner loop): k draft steps + the row-only step, one batched verify of k+1 rows per stream, the
 * acceptance kernel, cursor commit.  next_tokens_host[stream] is the confirmed token entering the
 * round and receives the token entering the next one; accepted_host[stream] receives the accepted count.
 * Streams must have equal cursors in the target and draft caches (lockstep). */
TSB_API int32_t tsb_session_round(tsb_session* s, const tsb_run_config* cfg, int32_t* next_tokens_host,
                                  int32_t* accepted_host, uint64_t* draw_step_inout);
/* The same round, also returning what each stream committed: tokens_out[stream * 16 + i] for i < accepted is the
 * i-th accepted proposal, tokens_out[stream * 16 + accepted] the corrected / bonus token (the same value that lands
 * in next_tokens_host).  A serving loop appends the confirmed token that entered the round, then the accepted ones
 * (crates/runtime/src/speculative.rs:861-905). */
TSB_API int32_t tsb_session_round_tokens(tsb_session* s, const tsb_run_config* cfg, int32_t* next_tokens_host,
                                         int32_t* accepted_host, int32_t* tokens_out, uint64_t* draw_step_inout);
/* Rounds run as one CUDA graph after the first (copies, kernels); 0 switches to plain launches, which is what
 * makes the per-phase timings below available.  Env TSB_GRAPH=0 does the same at session creation. */
TSB_API int32_t tsb_session_set_graph(tsb_session* s, int32_t enabled);
/* Device time of the last tsb_session_round in milliseconds (CUDA events): [0] draft, [1] verify, [2] accept
 * (-1 when the round ran as a graph), [3] the whole round. */
TSB_API int32_t tsb_session_round_times(tsb_session* s, float* out4_ms);
/* Benchmark set-up: pretend `tokens` positions are committed in both caches of every stream, filling
 * them with seeded pseudo-random K/V. */
TSB_API int32_t tsb_session_fill_context(tsb_session* s, int64_t tokens, uint64_t seed);

/* The history penalties of a shaping record (repetition over the whole history, presence / frequency over the tokens
 * generated in this turn; crates/selection/src/penalty.rs:15-39,59-82) are applied inside tsb_session_round,
 * tsb_spec_run and tsb_sequential_run: a stream's history is the record of tokens fed to its cache plus the confirmed
 * token entering the round.  `generated` says how many tokens at the end of that history count as generated; the
 * generation loops keep it themselves, tsb_session_round adds what each round commits, tsb_producer_reset zeroes it
 * and this call sets it (a serving loop calls it after the prompt: generated = 1 once the first token is chosen).
 * Penalised rounds stage the history from the host every round and run as plain launches, not as a graph. */
TSB_API int32_t tsb_session_set_generated(tsb_session* s, int32_t stream, int32_t generated);
/* verify_tree for every stream of the session in ONE target pass: stream b's slots are feed[b * n .. b * n + n), all
 * streams share the tree shape slot_parent[0..n) (crates/runtime/src/families/qwen/batched_scratch.rs:97-124) and
 * each starts at its own cursor.  Row b * n + j of the logits belongs to stream b's slot j; logits_out_host may be
 * NULL to leave them on the device.  Afterwards each stream is in the state tsb_producer_verify_tree leaves it in:
 * tsb_producer_compact_tree and tsb_producer_rollback_retaining finish the round stream by stream. */
TSB_API int32_t tsb_session_verify_tree(tsb_session* s, const int32_t* feed, const int32_t* slot_parent, int32_t n, void* logits_out_host);
/* The CUDA stream (cudaStream_t) the session enqueues on, so a caller can record its own events on it. */
TSB_API void* tsb_session_stream(tsb_session* s);
/* Measurement aid: enqueue the target's layer matmuls exactly as a pass of `rows` rows launches them (q|k|v with the
 * RoPE / K-V-store epilogue, o_proj and down with the residual + norm epilogue, gate|up with the SiLU epilogue, for
 * every layer; no attention, embedding or head) `iters` times, over whatever the activation buffers hold and rows
 * past the streams' cursors, and return the elapsed device time and the bytes one sequence streams. */
TSB_API int32_t tsb_session_time_matmuls(tsb_session* s, int32_t rows, int32_t iters, float* out_ms, int64_t* out_bytes_per_iter,
                                         int32_t* out_launches_per_iter);
/* Measurement aid, the complement of tsb_session_time_matmuls: enqueue every launch of a `rows`-row pass EXCEPT the
 * layer matmuls (embedding + norm, attention partials and merge of every layer, the head matmul) `iters` times and
 * return the elapsed device time.  A pass's time minus this is what the layer matmuls take inside the pass. */
TSB_API int32_t tsb_session_time_pass_rest(tsb_session* s, int32_t rows, int32_t iters, float* out_ms);

#ifdef __cplusplus
}
#endif
#endif /* TSB_H */
