// Internal interface of the decode-attention kernels (shared with the model runner).
#pragma once
#include "kv.cuh"
#include "rowops.cuh"

struct AttnPlan {
    int chunk;         // KV positions per CTA (multiple of 64)
    int n_splits;      // grid.x = clusters * cluster_size
    int cluster_size;  // CTAs whose shares are merged through distributed shared memory (1, 2, 4, 8 or 16)
    int mt;            // 16-query tiles per CTA (1 or 2)
    int n_qtiles;      // query tiles per (stream, kv head)
    int groups;        // streams in the batch
};
AttnPlan attn_plan(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads, int max_len);
size_t attn_scratch_bytes(int rows, int n_q_heads, int head_dim);
// out (natural f16 rows, may be null) and/or act (matmul operand) receive the attention output.  scratch was sized
// by attn_scratch_bytes(rows_cap, ...) and its trailing ticket words are zero (they reset themselves).
cudaError_t launch_attn_decode_rows(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                    __half* out, ActOut act, const tsb_row_desc* rows_dev, int rows, int rows_per_seq,
                                    int n_q_heads, float scale, int max_len, void* scratch, int rows_cap);
// Partials only: every (stream, kv head, query tile, KV chunk) CTA leaves its share (O, and (m, l)) in `scratch`,
// laid out [rows * n_q_heads][n_splits]; nobody merges (attn_merge_kernel, launched next, does).  Returns where
// the shares sit and how many splits were cut.  When the plan cuts the context into ONE split there is nothing to
// merge: the launch then writes out_single / act_single itself and the caller skips the merge.
cudaError_t launch_attn_partials(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                 const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int n_q_heads, float scale, int max_len,
                                 void* scratch, const float** part_o_out, const float2** part_ml_out, int* n_splits_out,
                                 __half* out_single = nullptr, ActOut act_single = ActOut{nullptr, nullptr});
// The tensor-memory (tcgen05) kernel at head_dim 128: for passes with more than 64 queries per (stream, kv head), and for
// passes whose streams x kv heads alone give every SM a CTA.  The same partials in the same layout; the merge launch always
// follows (also after a single split).
bool attn_tc_applicable(const tsb_ctx* ctx, const tsb_kv* kv, int rows, int rows_per_seq, int n_q_heads);
cudaError_t launch_attn_tc_partials(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, const __half* q, int64_t q_stride,
                                    const tsb_row_desc* rows_dev, int rows, int rows_per_seq, int n_q_heads, float scale, int max_len,
                                    void* scratch, const float** part_o_out, const float2** part_ml_out, int* n_splits_out);
cudaError_t launch_rope_store_kv(tsb_ctx* ctx, cudaStream_t st, tsb_kv* kv, int layer, __half* qkv,
                                 const tsb_row_desc* rows_dev, int rows, int n_q_heads, float theta);
