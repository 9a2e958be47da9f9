// Internal launchers of the row operators (shared with the model runner).
#pragma once
#include "gemm_quant.cuh"

cudaError_t launch_embed_rows(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t vocab_rows, int cols,
                              const int32_t* ids, int id_stride, int n, __half* out, float out_scale);
// x <- f16(x + residual) when residual != null; out (natural f16, may be null) and/or act get the normed rows.
cudaError_t launch_rmsnorm_rows(tsb_ctx* ctx, cudaStream_t st, __half* x, const __half* residual, const void* w_bf16,
                                __half* out, ActOut act, int rows, int d, float eps);
// x += half(sum over slots of w[r, s] * values[r * k + s][.]) (slot order), then the norm of the updated rows.
cudaError_t launch_combine_norm_rows(tsb_ctx* ctx, cudaStream_t st, __half* x, const float* values, const __half* weights, int k,
                                     const void* w_bf16, __half* out, ActOut act, int rows, int d, float eps);
cudaError_t launch_silu_mul(tsb_ctx* ctx, cudaStream_t st, const __half* gate, const __half* up, __half* out, ActOut act,
                            int rows, int n, int64_t in_stride, int64_t out_stride);
// Fused embedding for the model forward: residual stream, first operand f16(h * g), sum of h^2, RoPE table.
cudaError_t launch_embed_norm(tsb_ctx* ctx, cudaStream_t st, int qtype, const uint8_t* w, int64_t vocab_rows, int d,
                              const int32_t* ids, int id_stride, int n, __half* h, const void* g_bf16, ActOut act, float* ss_out,
                              float* cs, const tsb_row_desc* rows, int head_dim, float theta);
