"""Tree verification at the tree configuration's shape: one target pass over a 64-node static draft tree (plus the
anchor: 65 rows) per stream, long fp16 contexts, 1..32 streams in lockstep.

    python -m turbospark_b200.treebench --context 8192 --streams 1
    python -m turbospark_b200.treebench --context 32768 --streams 8 --iters 5

Target: 32 layers, d 4096, 32 query / 8 KV heads x 128, FFN 14336, vocabulary 128 256, seeded synthetic Q4_K blocks;
drafter (for the round leg): one decoder layer of the same shape sharing the target's head.  Tree: branching
4,4,2,1,1,1 cut to 64 nodes.  The context is pre-filled with seeded random K/V.  Two legs, one JSON line:

  verify  the pass alone (CUDA events on the session's stream around `--iters` passes, cursors put back between them):
          milliseconds, and the bytes the pass has to read - every weight block once, every stream's K/V once - over that
          time.
  round   at one stream, whole greedy tree rounds through tsb_spec_run (draft the tree level by level, verify, accept
          walk, compaction of both caches): committed tokens per second.  Sampled tree rounds are refused by the
          library as by the reference, so this leg runs at temperature 0 whatever the configuration's 0.7.
"""
import argparse
import json

import numpy as np

from . import capi
from .model import Model, ModelConfig, Session, config_8b_target, run_config
from .capi import shaping


def static_tree(branching, nodes):
    """Slot parents of a level-by-level tree (slot 0 = the anchor) cut at `nodes` drafted nodes."""
    parent, level = [-1], [0]
    for b in branching:
        nxt = []
        for p in level:
            for _ in range(b):
                if len(parent) - 1 == nodes:
                    return parent
                parent.append(p)
                nxt.append(len(parent) - 1)
        level = nxt
    return parent


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warm", type=int, default=3)
    ap.add_argument("--round-tokens", type=int, default=96, help="new tokens of the whole-round leg (0: skip)")
    ap.add_argument("--layers", type=int, default=32)
    a = ap.parse_args()
    import torch
    torch.cuda.set_device(0)
    ctx = capi.Ctx(0)
    branching, nodes = (4, 4, 2, 1, 1, 1), 64
    parent = static_tree(branching, nodes)
    n = len(parent)
    S = a.streams
    max_ctx = a.context + a.round_tokens + 4 * n + 64
    cfg = config_8b_target(max_ctx)
    cfg = ModelConfig(a.layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, max_ctx, cfg.rms_eps, cfg.rope_theta)
    target = Model(ctx, cfg)
    target.fill_synthetic(capi.Q4_K, seed=1)
    draft = Model(ctx, ModelConfig(1, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, max_ctx, cfg.rms_eps, cfg.rope_theta))
    draft.fill_synthetic(capi.Q4_K, seed=2)
    draft.share(-1, target, -1)
    sess = Session(ctx, target, draft, S, n, page_tokens=64)
    sess.fill_context(a.context, seed=7)
    rng = np.random.default_rng(5)
    feed = rng.integers(0, cfg.vocab, size=(S, n)).astype(np.int32)
    stream = torch.cuda.ExternalStream(sess.stream_ptr)
    times = []
    for it in range(a.warm + a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        sess.verify_tree_streams(feed, parent, want_logits=False)
        e1.record(stream)
        ctx.sync()
        for b in range(S):
            sess.discard_pending(stream=b)
        if it >= a.warm:
            times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    w_bytes = target.weight_bytes
    kv_bytes = S * a.layers * (a.context + n) * cfg.n_kv_heads * cfg.head_dim * 2 * 2
    logits_bytes = S * n * cfg.vocab * 2
    algo = w_bytes + kv_bytes + logits_bytes
    out = {"workload": "tree verify: %d-layer 8B-shape Q4_K target, %d rows per stream (64-node tree 4,4,2,1,1,1 + anchor), context %d, %d stream(s)"
                       % (a.layers, n, a.context, S),
           "verify_ms": ms, "verify_ms_min": float(min(times)), "rows": S * n,
           "algorithmic_bytes": {"weights": w_bytes, "kv": kv_bytes, "logits": logits_bytes, "total": algo},
           "gbs": algo / ms / 1e6, "rows_per_s": S * n / (ms * 1e-3)}
    if S == 1 and a.round_tokens > 0:
        # the pre-filled rows are recorded as fed token 0, so a prompt of zeros continues them without a prefill
        rc = run_config(shaping(temperature=0.0), a.round_tokens, len(branching), tree_nodes=nodes, tree_branching=branching, reuse_prefix=True)
        prompt = np.concatenate([np.zeros(a.context, dtype=np.int32), rng.integers(0, cfg.vocab, size=4).astype(np.int32)])
        _, _, res = sess.spec_run(prompt, rc)
        out["round"] = {"new_tokens": int(res.new_tokens), "rounds": int(res.rounds), "reused_prefix": int(res.reused_prefix),
                        "committed_per_round": res.new_tokens / max(1, res.rounds),
                        "tokens_per_s": res.new_tokens / res.decode_seconds, "ms_per_round": res.decode_seconds * 1e3 / max(1, res.rounds),
                        "note": "greedy tree rounds of the library loop (host clock around the decode phase); random unrelated "
                                "weights accept almost nothing, so tokens_per_s is a floor and ms_per_round the figure that carries over"}
    print(json.dumps(out), flush=True)
    sess.close(), draft.close(), target.close(), ctx.close()


if __name__ == "__main__":
    main()
