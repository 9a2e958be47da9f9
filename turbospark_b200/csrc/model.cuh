// Model, per-model runtime state and session objects behind the opaque C handles.
#pragma once
#include <cmath>
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
    int expert_lo = 0, n_local_experts = 0;     // the experts this model holds (all of them unless sharded)
};

// Shape of the trees a session drafts (tsb_session_set_tree, or a run configuration's tree fields).
struct TreeShape {
    int nodes = 0;      // drafted nodes per round (the anchor row comes on top); 0: chains only
    int levels = 0;     // longest path below the anchor
    int branching[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // static shape: children per node of level l
    int best_first = 0; // 1: grown best-first by path probability (crates/runtime/src/dflash_tree.rs:30-82)
    int cand = 0;       // best-first: candidates scored per expanded node (1..8)
};

// The last verify of a stream until the round's outcome is known (commit_pending / discard_pending).
struct PendingVerify {
    bool active = false, tree = false;
    int64_t base = 0;
    int rows = 0;
    std::vector<int32_t> feed;  // tree verifies: the token fed at every slot
    int drafter_rows = 0;       // tree drafts: slots the drafter's cache holds rows for
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
    // wide_ok: every pass of this model in this session runs the tensor-memory matmul (all matrices Q4_K and the model's
    // largest pass has 24 rows or more) with natural-layout f16 buffers around it; otherwise every pass runs the
    // register path.  Never a mix: the two sum in different orders.
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
    float* tp_partial = nullptr;  // [R, d_model] f32: this rank's share of the o_proj sums, summed over the ranks in place
    std::vector<std::vector<int32_t>> fed;  // per stream: tokens absorbed, by position (target only)
    std::vector<PendingVerify> pending;     // per stream (target only)
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
    // History penalties (repetition / presence / frequency): the sampler and the acceptance then read every stream's
    // token history from the device.  The buffers are made on first use; a round that needs them runs as plain
    // launches (the history is staged from the host record every round).
    std::vector<int32_t> generated;   // per stream: how many tokens at the end of its history were generated in this turn
    int32_t* hist_dev = nullptr;      // [n_streams, max_context]
    int32_t* hist_len_dev = nullptr;  // [n_streams]
    int32_t* gen_dev = nullptr;       // [n_streams]
    void* pen_scratch = nullptr;      // f32 rows + mark words of the penalised distributions
    std::vector<int32_t> hist_host;
    TreeShape tree;  // what tsb_producer_tree_nodes / tsb_producer_draft_tree use
    tsb_comm* comm = nullptr;  // exchange steps of a sharded routed model (null: single GPU)
};

// comm.cu: in-place f32 sum over the ranks on `st` (a no-op for a null or single-rank comm).
cudaError_t comm_all_reduce_f32(tsb_comm* c, cudaStream_t st, float* buf, size_t count);
int comm_world(const tsb_comm* c);

// One speculative round for the listed streams with k proposals each (model.cu).
int32_t session_round_streams(tsb_session* s, const int32_t* streams, int n_active, int k, const tsb_run_config* cfg,
                              int32_t* next_tokens_host, int32_t* accepted_host, int32_t* tokens_out /* [n_active][16] */,
                              int32_t* draws_out, uint64_t* draw_step_inout);
// One tree round for one stream at temperature 0 (model.cu): drafts the static tree of cfg level by level, verifies
// anchor + nodes in one target pass and returns, per slot (0 = anchor, node i = slot i + 1), the fed token, the
// slot's parent and the target's pick at that row.  Both caches' cursors are left at `base`; rows base + slot hold
// the tree (the drafter's only for the first *drafter_rows slots).
// Stage the token history of `n_active` streams for the penalised sampler: stream q's history is the record of
// tokens fed to its target cache up to the cursor, followed by next_tokens[a] when given (the confirmed token that
// enters a round); its generated count is s->generated[q].  Rows land at hist_dev[a * max_context ..].
int32_t session_stage_history(tsb_session* s, const int32_t* streams, int n_active, const int32_t* next_tokens);
int32_t session_tree_round(tsb_session* s, int stream, const tsb_run_config* cfg, int32_t next, int64_t base,
                           std::vector<int32_t>& feed, std::vector<int32_t>& slot_parent, std::vector<int32_t>& picks,
                           int* drafter_rows);
// The drafting half of a tree round at temperature 0: fills feed (slot 0 = the anchor token) and slot_parent, and for
// every drafted node its depth below the anchor, its candidate rank among its parent's children and its parent
// node (-1 under the anchor).  The drafter's cursor is left at `base`.
int32_t session_draft_tree(tsb_session* s, int stream, const TreeShape& shape, int32_t next, int64_t base, std::vector<int32_t>& feed,
                           std::vector<int32_t>& slot_parent, std::vector<tsb_tree_node>& nodes, int* drafter_rows);
// The best-first builder of crates/runtime/src/dflash_tree.rs:30-82 over a callback that scores one parent's children.
// child_scores(depth, parent_node_or_-1, scores_out[branch]) returns a status (0 = fine).  Repeatedly the frontier
// node with the highest path probability is taken and all its children are added; a parent's children share an f64
// softmax over its scores; ties prefer the shallower, then the lower candidate; parents precede children.
template <typename F>
inline int32_t best_first_tree(int depth_max, int nodes, int branch, F&& child_scores, std::vector<tsb_tree_node>& out) {
    out.clear();
    if (depth_max <= 0 || nodes <= 0 || branch <= 0) return 0;
    struct Front {
        double p;
        tsb_tree_node n;
    };
    std::vector<Front> frontier;
    std::vector<float> sc((size_t)branch);
    auto push_children = [&](int depth, int parent, double path_p) -> int32_t {
        int32_t rc = child_scores(depth, parent, sc.data());
        if (rc) return rc;
        float mf = -INFINITY;
        for (int i = 0; i < branch; i++) mf = fmaxf(mf, sc[i]);
        const double m = (double)mf;
        std::vector<double> e((size_t)branch);
        double z = 0.0;
        for (int i = 0; i < branch; i++) e[i] = exp((double)sc[i] - m);
        for (int i = 0; i < branch; i++) z += e[i];
        for (int c = 0; c < branch; c++) frontier.push_back({path_p * (e[c] / z), tsb_tree_node{depth, c, parent}});
        return 0;
    };
    if (int32_t rc = push_children(0, -1, 1.0)) return rc;
    while ((int)out.size() < nodes && !frontier.empty()) {
        size_t best = 0;
        for (size_t i = 1; i < frontier.size(); i++) {
            const Front &f = frontier[i], &b = frontier[best];
            if (f.p > b.p || (f.p == b.p && (f.n.depth < b.n.depth || (f.n.depth == b.n.depth && f.n.cand < b.n.cand)))) best = i;
        }
        const Front picked = frontier[best];
        frontier[best] = frontier.back();
        frontier.pop_back();
        const int id = (int)out.size();
        out.push_back(picked.n);
        if ((int)out.size() < nodes && picked.n.depth + 1 < depth_max)
            if (int32_t rc = push_children(picked.n.depth + 1, id, picked.p)) return rc;
    }
    return 0;
}
// Keep path[0..keep) of the tree rows of both caches as a chain at base (compaction + cursors + fed-token record).
int32_t session_tree_commit(tsb_session* s, int stream, int64_t base, const std::vector<int32_t>& feed,
                            const std::vector<uint32_t>& path, int keep, int drafter_rows);
// produce_prefill for tokens[0..n) starting at the stream's cursor, several rows per pass (model.cu).
int32_t session_prefill_rows(tsb_session* s, int stream, const int32_t* tokens, int n);
// token = select(logits row of the last single-row target forward) for one stream (model.cu).
int32_t session_select_target(tsb_session* s, int stream, const tsb_run_config* cfg, uint64_t uniform, int32_t* token_host);
