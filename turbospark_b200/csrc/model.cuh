// Model, per-model runtime state and session objects behind the opaque C handles.
#pragma once
#include <vector>

#include "gemm_quant.cuh"
#include "kv.cuh"

struct Mat {
    uint8_t* data = nullptr;
    int qtype = 0;
    int64_t rows = 0, cols = 0;
    bool owned = false;
};

struct LayerW {
    Mat wqkv, wo, wgu, wdown;  // q|k|v rows back to back; gate|up rows back to back
    Mat wv;                    // v rows on their own when their block format differs from q and k (wqkv is then q|k)
    uint8_t qkv_set = 0;       // which of q (1), k (2), v (4) have been uploaded
    uint16_t* attn_norm = nullptr;
    uint16_t* ffn_norm = nullptr;
    bool norms_owned = false;
    // routed feed-forward (when the model has experts): 8-bit affine router [E, d] with bf16 scale / bias per
    // 64 columns, expert matrices as verbatim block rows [E][2F, d] (gate then up) and [E][d, F]
    uint8_t* router_q = nullptr;
    uint16_t *router_scale = nullptr, *router_bias = nullptr;
    uint8_t *experts_gate_up = nullptr, *experts_down = nullptr;
    int experts_qtype = 0;
    bool moe_owned = false;
};

struct tsb_model {
    tsb_ctx* ctx = nullptr;
    tsb_model_config cfg{};
    std::vector<LayerW> layers;
    Mat embed, lm_head;
    uint16_t* out_norm = nullptr;
    bool out_norm_owned = false;
    int n_experts = 0, top_k = 0, moe_ffn = 0;  // n_experts > 0: every layer's feed-forward is routed
};

struct ActBuf {
    uint4* xp = nullptr;
    uint4* xs = nullptr;
};

// What one model needs to run inside a session.
struct ModelRt {
    const tsb_model* model = nullptr;
    tsb_kv* kv = nullptr;
    __half *h = nullptr, *q = nullptr;  // residual stream [R, d]; rotated queries [R, n_q_heads*head_dim]
    float* cs = nullptr;                // RoPE table [R, head_dim]: cos | sin of each row's position
    float* ss = nullptr;                // partial sums of h^2: [2*layers + 1][R][d/16]
    ActBuf act_d, act_o, act_f;  // matmul operands of width d_model, n_q_heads*head_dim, ffn
    void* attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    // many-row passes (24 rows and more, all matrices Q4_K): natural-layout f16 buffers around the tensor-memory matmul
    bool wide_ok = false;
    __half *w_xn = nullptr, *w_qkv = nullptr, *w_ao = nullptr, *w_o = nullptr, *w_gu = nullptr, *w_a = nullptr, *w_logits = nullptr;
    void* w_ws = nullptr;
    void* w_part = nullptr;  // split sums of the matmuls with few row tiles
    // routed feed-forward: router logits [R, E] f32, picks [R, k], weights [R, k] f16, a zero residual, workspace
    float* moe_logits = nullptr;
    int32_t* moe_ids = nullptr;
    __half *moe_w = nullptr, *moe_zero = nullptr;
    float* moe_unit_ss = nullptr;  // [R] sums of squares that make the q|k|v epilogue's 1/rms exactly one (the operand is already normed)
    void* moe_ws = nullptr;
    std::vector<std::vector<int32_t>> fed;  // per stream: tokens absorbed, by position (target only)
};

struct tsb_session {
    tsb_ctx* ctx = nullptr;
    int n_streams = 0, max_rows = 0;
    bool has_draft = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    ModelRt target, draft;
    __half* logits_target = nullptr;  // [n_streams * max_rows, vocab]
    __half* logits_draft = nullptr;   // [n_streams, k, vocab]
    int32_t* feed_dev = nullptr;      // [n_streams, k + 1]: confirmed token, then the proposals
    int32_t* tok1_dev = nullptr;
    int32_t* tree_dev = nullptr;      // tree drafting scratch: 128 row ids, then 8 picks per row
    uint64_t* uniforms_dev = nullptr;
    tsb_accept_out* accept_out_dev = nullptr;
    void* accept_scratch = nullptr;
    size_t accept_scratch_bytes = 0;
    // pinned staging
    tsb_row_desc* stage_rows_host = nullptr;
    int32_t* stage_tok_host = nullptr;
    tsb_row_desc* stage_rows_dev = nullptr;
    int32_t* stage_tok_dev = nullptr;
    int stage_cap = 0, stage_used = 0;
    tsb_accept_out* accept_out_host = nullptr;
    uint64_t* uniforms_host = nullptr;
    int32_t* feed_host = nullptr;
    int32_t* pair_host = nullptr;     // [n_streams, 2]: token before the cursor, confirmed token (drafter's first step)
    int32_t* pair_dev = nullptr;
    void* logits_host = nullptr;
    std::vector<void*> owned;
    // CUDA graph of one round's device work (copies, kernels, event records); rebuilt when the shape key changes
    bool use_graph = true, replay = false, capturing = false, last_round_graphed = false;
    cudaGraphExec_t graph = nullptr;
    uint64_t graph_key = 0, graph_launches = 0;
    int rounds_done = 0;
};

// One speculative round for the listed streams with k proposals each (model.cu).
int32_t session_round_streams(tsb_session* s, const int32_t* streams, int n_active, int k, const tsb_run_config* cfg,
                              int32_t* next_tokens_host, int32_t* accepted_host, int32_t* tokens_out /* [n_active][16] */,
                              int32_t* draws_out, uint64_t* draw_step_inout);
// One tree round for one stream at temperature 0 (model.cu): drafts the static tree of cfg level by level, verifies
// anchor + nodes in one target pass and returns, per slot (0 = anchor, node i = slot i + 1), the fed token, the
// slot's parent and the target's pick at that row.  Both caches' cursors are left at `base`; rows base + slot hold
// the tree (the drafter's only for the first *drafter_rows slots).
int32_t session_tree_round(tsb_session* s, int stream, const tsb_run_config* cfg, int32_t next, int64_t base,
                           std::vector<int32_t>& feed, std::vector<int32_t>& slot_parent, std::vector<int32_t>& picks,
                           int* drafter_rows);
// Keep path[0..keep) of the tree rows of both caches as a chain at base (compaction + cursors + fed-token record).
int32_t session_tree_commit(tsb_session* s, int stream, int64_t base, const std::vector<int32_t>& feed,
                            const std::vector<uint32_t>& path, int keep, int drafter_rows);
// produce_prefill for tokens[0..n) starting at the stream's cursor, several rows per pass (model.cu).
int32_t session_prefill_rows(tsb_session* s, int stream, const int32_t* tokens, int n);
// token = select(logits row of the last single-row target forward) for one stream (model.cu).
int32_t session_select_target(tsb_session* s, const tsb_run_config* cfg, uint64_t uniform, int32_t* token_host);
