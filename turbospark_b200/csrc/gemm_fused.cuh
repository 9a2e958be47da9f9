// A chain of dependent quantized matmuls (optionally led by the merge of attention partials) run as one
// cooperative launch of persistent CTAs with grid-wide barriers between the phases (gemm_fused.cu).
#pragma once
#include "gemm_quant.cuh"

constexpr int FUSED_MAX_PHASES = 5;
enum FusedKind { FUSED_NONE = 0, FUSED_GEMM = 1, FUSED_MERGE = 2 };

// Split-KV partials of the attention kernel, [rows * n_q_heads][n_splits]: O (head_dim floats) and (m, l).
struct MergeArgs {
    const float* part_o = nullptr;
    const float2* part_ml = nullptr;
    int n_splits = 0, rows = 0, n_q_heads = 0, head_dim = 0;
    ActOut out{nullptr, nullptr};  // the o_proj operand
};

struct FusedPhase {
    int kind = FUSED_NONE;
    int epi = EPI_PLAIN;  // EPI_RESID_NORM, EPI_SILU, EPI_ROPE_STORE or EPI_SCALE
    const uint8_t* w = nullptr;  // Q4_K block rows
    int64_t rows = 0;
    int units = 0;               // 256-column units per row
    ActOperand act{nullptr, nullptr};
    EpiArgs e;
};

struct FusedArgs {
    FusedPhase ph[FUSED_MAX_PHASES];
    int n_phases = 0;
    int tokens = 0;  // 1..64 token rows, the same for every phase
    MergeArgs merge;
    uint32_t* state = nullptr;            // the context's device area (error word, wait bound, barrier counter)
    unsigned arrive_inc = 1, per_barrier = 0;  // filled by the launcher
};

// Every matmul of a chain must satisfy this (Q4_K, whole 256-column units, at most 64 token rows).
bool gemm_chain_supported(int qtype, int64_t rows, int64_t cols, int tokens);
cudaError_t launch_gemm_chain(tsb_ctx* ctx, cudaStream_t st, FusedArgs& args);
