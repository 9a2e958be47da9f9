// Internal launchers of the acceptance / sampling kernels (shared with the model runner).
#pragma once
#include "common.cuh"

// What the device sampler reads of a shaping record (crates/selection/src/shaping.rs:40-50).
struct AcceptShape {
    double temperature;
    double top_p;  // <= 0: off
    double min_p;  // <= 0: off
    unsigned int top_k;  // 0: off
    AcceptShape(double t = 1.0, unsigned int k = 0, double p = 0.0, double mp = 0.0) : temperature(t), top_p(p), min_p(mp), top_k(k) {}
    explicit AcceptShape(const tsb_shaping& sh) : temperature(sh.temperature), top_p(sh.top_p), min_p(sh.min_p), top_k(sh.top_k) {}
};
size_t accept_scratch_bytes(int batch, int k, int vocab);
int accept_max_vocab();  // largest vocabulary the on-chip draw holds
// have_history: the caller can supply the token history, so the history penalties are accepted
int32_t accept_check_shaping(tsb_ctx* ctx, const tsb_shaping* sh, bool have_history = false);
bool accept_has_penalties(const tsb_shaping& sh);  // the record carries a penalty that changes a sampled distribution
// proposals[b * prop_stride + i]; when next_tokens != null the corrected / bonus token of stream b is also
// written to next_tokens[b * next_stride].
cudaError_t launch_accept(tsb_ctx* ctx, cudaStream_t st, const __half* target, const __half* draft, const int32_t* proposals,
                          int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, AcceptShape shape,
                          tsb_accept_out* out_dev, int32_t* next_tokens, int next_stride, void* scratch);
// row b at logits + b * logits_stride, uniform at uniforms[b * uni_stride], token to tokens_dev[b * token_stride].
cudaError_t launch_sample(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int64_t logits_stride,
                          const uint64_t* uniforms, int uni_stride, int batch, int vocab, AcceptShape shape,
                          int32_t* tokens_dev, int token_stride, double* margins_dev, void* scratch);
// The same two operators with the history penalties of the shaping record applied first (repetition over the whole
// history, presence / frequency over its generated suffix): history[b * hist_stride + j] for j < hist_len[b],
// generated[b] of its last entries produced in this turn.  scratch: accept_history_scratch_bytes(batch, k, vocab).
size_t accept_history_scratch_bytes(int batch, int k, int vocab);
cudaError_t launch_accept_history(tsb_ctx* ctx, cudaStream_t st, const __half* target, const __half* draft, const int32_t* proposals,
                                  int prop_stride, const uint64_t* uniforms, int batch, int k, int vocab, const tsb_shaping& sh,
                                  const int32_t* history, int hist_stride, const int32_t* hist_len, const int32_t* generated,
                                  tsb_accept_out* out_dev, void* scratch, int32_t* next_tokens = nullptr, int next_stride = 0);
cudaError_t launch_sample_history(tsb_ctx* ctx, cudaStream_t st, const __half* logits, const uint64_t* uniforms, int batch, int vocab,
                                  const tsb_shaping& sh, const int32_t* history, int hist_stride, const int32_t* hist_len,
                                  const int32_t* generated, int32_t* tokens_dev, double* margins_dev, void* scratch,
                                  int64_t logits_stride = 0, int uni_stride = 1, int token_stride = 1);
// The `width` (<= 8) largest logits of rows rows_dev[0..n_rows) of a [*, vocab] matrix, value descending, token id
// ascending on ties; row r's picks land in out_dev[r * 8 ..].
cudaError_t launch_topk_rows(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int vocab, const int32_t* rows_dev, int n_rows,
                             int width, int32_t* out_dev);
// max / first argmax / finiteness of n_rows consecutive rows into scratch (one record per row).
cudaError_t launch_argmax_rows(tsb_ctx* ctx, cudaStream_t st, const __half* logits, int n_rows, int vocab, void* scratch);
int accept_row_stats_bytes();
void accept_row_stats_read(const void* host_stats, int row, int32_t* argmax, int32_t* nonfinite);
