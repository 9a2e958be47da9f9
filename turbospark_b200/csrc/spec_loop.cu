// The generation loops: the speculative round loop and the sequential loop it must reproduce.
//
// Restated from crates/runtime/src/speculative.rs:194-940 and raw_completion.rs:300-420 for the
// parts that need no tokenizer: admission, the budget / window clamp of every round, the stop-token
// ladder of the commit sink (token_sink.rs:64-124), the adaptive depth controller
// (speculative_adaptive.rs:104-225), the draw counter, and the cursor discipline
// (checkpoint -> verify -> rollback_retaining -> rewind_drafter).  Selection and acceptance run on
// the device; the host reads back one small record per round.
#include <algorithm>
#include <chrono>
#include <vector>

#include "model.cuh"

namespace {

struct Sink {  // token_sink.rs:64-124 without detokenisation: a stopping token is counted, not pushed
    const tsb_run_config* cfg;
    std::vector<int32_t> history, emitted;
    int64_t generated = 0;
    int commit(int32_t t) {
        generated++;
        emitted.push_back(t);
        for (int i = 0; i < cfg->n_stop && i < 8; i++)
            if (cfg->stop_tokens[i] == t) return 1;
        if (generated >= cfg->max_new_tokens) return 0;
        history.push_back(t);
        return -1;
    }
};

struct Adaptive {  // speculative_adaptive.rs:104-225, default parameters
    int64_t floor, cap, cur, climb = 0, pressure = 0;
    Adaptive(int64_t f, int64_t c) {
        cap = std::max<int64_t>(c, 1);
        floor = std::min(std::max<int64_t>(f, 1), cap);
        cur = floor;
    }
    static int64_t threshold(int64_t d) { return d <= 1 ? 2 : (d <= 3 ? 8 : (d == 4 ? 6 : 4)); }
    void observe(int64_t offered, int64_t accepted) {
        if (offered == 0) return;
        accepted = std::min(accepted, offered);
        if (accepted == offered) {
            pressure = 0;
            if (cur < cap && ++climb >= threshold(cur)) cur++, climb = 0;
        } else {
            climb = 0;
            if (cur > floor) {
                pressure += offered - accepted;
                if (pressure >= 2) cur--, pressure = 0;
            }
        }
    }
};

int32_t admission(tsb_ctx* ctx, int n_prompt, const tsb_run_config* cfg, int max_context) {
    // raw_completion.rs:126-146
    TSB_REQUIRE(ctx, n_prompt > 0, "the prompt is empty");
    TSB_REQUIRE(ctx, cfg->max_new_tokens > 0, "the generation budget is zero");
    if ((int64_t)n_prompt + cfg->max_new_tokens > max_context)
        return tsb_fail(ctx, TSB_ERR_INVALID, "prompt %d + budget %d exceeds the context window %d", n_prompt, cfg->max_new_tokens,
                        max_context);
    return TSB_OK;
}

// Prefill through the target (head on the last token only) and, when present, the drafter.
int32_t prefill(tsb_session* s, int stream, const int32_t* prompt, int n_prompt, bool with_drafter, bool reuse, int32_t* reused) {
    int32_t rc;
    int64_t kept = 0;
    if (reuse) {
        kept = tsb_producer_try_reuse_prefix(s, stream, prompt, n_prompt);
    } else if ((rc = tsb_producer_reset(s, stream))) {
        return rc;
    }
    *reused = (int32_t)kept;
    // all but the last prompt token go through in chunks of rows (one chain pass each, no head); the last one alone,
    // with the head.  Both generation loops prefill this way, so they start from the same cache contents.
    if (n_prompt - 1 > kept && (rc = session_prefill_rows(s, stream, prompt + kept, n_prompt - 1 - (int)kept))) return rc;
    if ((rc = tsb_producer_produce(s, stream, prompt[n_prompt - 1], n_prompt - 1, nullptr))) return rc;
    if (with_drafter && n_prompt >= 2) {
        // prime_drafter(prompt[i+1], i) for every i: after it the drafter holds rows 0..n_prompt-1
        if ((rc = tsb_producer_prime_drafter(s, stream, prompt[n_prompt - 1], n_prompt - 2))) return rc;
    }
    return TSB_OK;
}

double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

uint64_t first_uniform(const tsb_run_config* cfg) {
    // the first pick is `select` at position = generated = 0 (choose.rs:323-338); with an external
    // generator it takes an index no loop draw uses
    return cfg->uniform_mode == 0 ? tsb_uniform_u64(0, cfg->shaping.seed, 0) : tsb_uniform_u64(cfg->uniform_mode, cfg->shaping.seed, 1ull << 63);
}

void finish(tsb_run_result* res, const Sink& sink, int reason, int rounds, int accepted, int rollbacks, int64_t position,
            uint64_t draws, int32_t* out_tokens, int32_t* out_emitted) {
    res->new_tokens = (int32_t)sink.generated;
    res->reason = reason;
    res->rounds = rounds;
    res->accepted_total = accepted;
    res->rollbacks = rollbacks;
    res->history_len = (int32_t)sink.history.size();
    res->kv_position = position;
    res->draws = draws;
    std::copy(sink.history.begin(), sink.history.end(), out_tokens);
    std::copy(sink.emitted.begin(), sink.emitted.end(), out_emitted);
}

}  // namespace

extern "C" {

int32_t tsb_spec_run(tsb_session* s, int32_t stream, const int32_t* prompt, int32_t n_prompt, const tsb_run_config* cfg,
                     int32_t* out_tokens, int32_t* out_emitted, tsb_run_result* res) {
    if (!s || !cfg || !res || !out_tokens || !out_emitted || (!prompt && n_prompt)) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    DeviceGuard g(ctx);
    const int max_context = s->target.model->cfg.max_context;
    int32_t rc = admission(ctx, n_prompt, cfg, max_context);
    if (rc) return rc;
    if (cfg->block == 0)  // speculative.rs:208-212
        return tsb_fail(ctx, TSB_ERR_INVALID, "block size 0 proposes nothing; call tsb_sequential_run instead");
    TSB_REQUIRE(ctx, cfg->block >= 1 && cfg->block <= 15, "block must be 1..=15");
    if (cfg->tree_nodes > 0) {
        TSB_REQUIRE(ctx, cfg->tree_levels == cfg->block, "tree rounds need block (%d) == tree_levels (%d)", cfg->block, cfg->tree_levels);
        TSB_REQUIRE(ctx, cfg->shaping.temperature == 0.0, "tree rounds need temperature 0");
    }
    TSB_REQUIRE(ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    if (!s->has_draft) return tsb_fail(ctx, TSB_ERR_STATE, "speculation needs a drafter");
    const int block = cfg->block;
    const bool sampled = cfg->shaping.temperature != 0.0;

    const double t0 = now_s();
    if ((rc = prefill(s, stream, prompt, n_prompt, true, cfg->reuse_prefix != 0, &res->reused_prefix))) return rc;
    const double t1 = now_s();

    Sink sink;
    sink.cfg = cfg;
    sink.history.assign(prompt, prompt + n_prompt);
    Adaptive adaptive(cfg->adaptive ? cfg->adaptive : 1, block);
    uint64_t draw_step = 0;
    int rounds = 0, accepted_total = 0, rollbacks = 0, reason = 0;
    int64_t position = n_prompt;

    int32_t next;
    s->generated[stream] = 0;
    if ((rc = session_select_target(s, stream, cfg, first_uniform(cfg), &next))) return rc;
    // the confirmed token's stream seed offset is zero for a single-stream run
    tsb_run_config round_cfg = *cfg;
    round_cfg.shaping.seed = cfg->shaping.seed - (uint64_t)stream;

    for (;;) {
        const int stop = sink.commit(next);
        if (stop >= 0) {
            reason = stop;
            break;
        }
        const int64_t base = (int64_t)sink.history.size() - 1;
        position = (int64_t)sink.history.size();
        const int64_t budget_room = std::max<int64_t>(0, cfg->max_new_tokens - sink.generated);
        const int64_t context_room = std::max<int64_t>(0, max_context - position);
        const int64_t wanted = cfg->adaptive ? std::min<int64_t>(adaptive.cur, block) : block;
        const int64_t round_block = std::min(wanted, std::min(budget_room, context_room));
        const bool truncated = round_block < wanted;
        if (round_block == 0) return tsb_fail(ctx, TSB_ERR_STATE, "round_block is 0: no room after admission");
        if (tsb_kv_cursor(s->target.kv, stream) != base)
            return tsb_fail(ctx, TSB_ERR_STATE, "target cursor %lld does not sit at the confirmed token %lld",
                            (long long)tsb_kv_cursor(s->target.kv, stream), (long long)base);

        if (cfg->tree_nodes > 0 && round_block == block && !cfg->adaptive) {
            // ---- a tree round: the walk is the chain's acceptance generalised - at the current node's row the target's
            // pick is accepted when a child of that node carries it (speculative.rs:494-529)
            std::vector<int32_t> feed, parent, picks;
            int drafter_rows = 0;
            if ((rc = session_tree_round(s, stream, cfg, next, base, feed, parent, picks, &drafter_rows))) {
                // speculative.rs:551-557: a round that fails after its verify began is discarded, not half-kept
                tsb_kv_set_cursor(s->target.kv, stream, std::min<int64_t>(tsb_kv_cursor(s->target.kv, stream), base));
                tsb_producer_rewind_drafter(s, stream, base);
                return rc;
            }
            rounds++;
            std::vector<uint32_t> path{0};
            int at = 0, stopped = -1;
            int32_t bonus = -1;
            for (;;) {
                const int32_t target = picks[at];
                int hit = -1;
                for (int c = at + 1; c < (int)feed.size(); c++)
                    if (parent[c] == at && feed[c] == target) {
                        hit = c;
                        break;
                    }
                if (hit < 0) {
                    bonus = target;
                    break;
                }
                path.push_back((uint32_t)hit);
                at = hit;
                const int st = sink.commit(target);
                if (st >= 0) {
                    stopped = st;
                    break;
                }
            }
            accepted_total += (int)path.size() - 1;
            const int64_t committed = (int64_t)sink.history.size() - (base + 1);
            if (committed + 1 < (int64_t)feed.size()) rollbacks++;
            if ((rc = session_tree_commit(s, stream, base, feed, path, (int)committed + 1, drafter_rows))) {
                tsb_kv_set_cursor(s->target.kv, stream, std::min<int64_t>(tsb_kv_cursor(s->target.kv, stream), base));
                tsb_producer_rewind_drafter(s, stream, base);
                return rc;
            }
            position = (int64_t)sink.history.size();
            if (stopped >= 0) {
                reason = stopped;
                break;
            }
            next = bonus;
            continue;
        }

        int32_t accepted = 0, draws = 0, toks[16];
        int32_t confirmed = next;
        s->generated[stream] = sink.generated;  // the history penalties count the tokens of this turn, the confirmed one included
        if ((rc = session_round_streams(s, &stream, 1, (int)round_block, &round_cfg, &confirmed, &accepted, toks, &draws, &draw_step)))
            return rc;
        rounds++;
        // commit the accepted proposals one by one; a stop inside the block ends the run there
        int stopped = -1, counted = 0;
        for (int i = 0; i < accepted; i++) {
            counted++;
            const int st = sink.commit(toks[i]);
            if (st >= 0) {
                stopped = st;
                break;
            }
        }
        accepted_total += counted;
        if (cfg->adaptive && !truncated && stopped < 0) adaptive.observe(round_block, accepted);
        const int64_t committed = (int64_t)sink.history.size() - (base + 1);
        if (committed < round_block) rollbacks++;
        // rollback_retaining(point, committed + 1) and rewind_drafter(base + committed)
        tsb_kv_set_cursor(s->target.kv, stream, base + committed + 1);
        tsb_kv_set_cursor(s->draft.kv, stream, base + committed + 1);
        s->target.fed[stream].resize((size_t)(base + committed + 1));
        position = (int64_t)sink.history.size();
        if (stopped >= 0) {
            reason = stopped;
            break;
        }
        next = confirmed;
    }
    res->prefill_seconds = t1 - t0;
    res->decode_seconds = now_s() - t1;
    finish(res, sink, reason, rounds, accepted_total, rollbacks, position, draw_step, out_tokens, out_emitted);
    return TSB_OK;
}

int32_t tsb_sequential_run(tsb_session* s, int32_t stream, const int32_t* prompt, int32_t n_prompt, const tsb_run_config* cfg,
                           int32_t* out_tokens, int32_t* out_emitted, tsb_run_result* res) {
    if (!s || !cfg || !res || !out_tokens || !out_emitted || (!prompt && n_prompt)) return TSB_ERR_INVALID;
    tsb_ctx* ctx = s->ctx;
    DeviceGuard g(ctx);
    int32_t rc = admission(ctx, n_prompt, cfg, s->target.model->cfg.max_context);
    if (rc) return rc;
    TSB_REQUIRE(ctx, stream >= 0 && stream < s->n_streams, "stream %d outside the session", stream);
    const double t0 = now_s();
    if ((rc = prefill(s, stream, prompt, n_prompt, false, cfg->reuse_prefix != 0, &res->reused_prefix))) return rc;
    const double t1 = now_s();
    Sink sink;
    sink.cfg = cfg;
    sink.history.assign(prompt, prompt + n_prompt);
    int64_t position = n_prompt;
    int reason = 0;
    for (;;) {
        // select(logits, shaping, history, position = generated): the draw index is the generated count
        const uint64_t u = cfg->uniform_mode == 0 ? tsb_uniform_u64(0, cfg->shaping.seed, (uint64_t)sink.generated)
                                                  : tsb_uniform_u64(cfg->uniform_mode, cfg->shaping.seed, (1ull << 63) + (uint64_t)sink.generated);
        int32_t next;
        s->generated[stream] = sink.generated;
        if ((rc = session_select_target(s, stream, cfg, u, &next))) return rc;
        const int stop = sink.commit(next);
        if (stop >= 0) {
            reason = stop;
            break;
        }
        if ((rc = tsb_producer_produce(s, stream, next, position, nullptr))) return rc;
        position++;
    }
    res->prefill_seconds = t1 - t0;
    res->decode_seconds = now_s() - t1;
    finish(res, sink, reason, 0, 0, 0, position, 0, out_tokens, out_emitted);
    return TSB_OK;
}

}  // extern "C"
