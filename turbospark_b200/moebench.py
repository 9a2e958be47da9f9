"""Speculative rounds over a routed (mixture-of-experts) model at the MoE configuration's shape.

    python -m turbospark_b200.moebench --streams 1 --rounds 20
    python -m turbospark_b200.moebench --streams 16 --rounds 10 --layers 48

48 layers, d 2048, 32 query / 4 KV heads x 128, 128 experts of width 768 with top-8 routing, vocabulary 151 936,
MXFP4 blocks, context 4096 of pre-filled random K/V; the drafter is the target's first `--draft-layers` layers with
the shared head; chain depth K = 4, temperature 1.  Weights are seeded synthetic blocks, so routing is close to
uniform.  One JSON line: committed tokens/s, the device time of the phases, and the verify pass's achieved bytes/s
against the bytes it has to read: attention, router and head weights once, the distinct routed experts (their
expected number under uniform routing), and the K/V of every stream.
"""
import argparse
import json

import numpy as np

from . import capi
from .model import Model, ModelConfig, Session, run_config
from .capi import shaping


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--rounds", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--draft-layers", type=int, default=4)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--block", type=int, default=4)
    a = ap.parse_args()
    E, TOPK, F, D, V = 128, 8, 768, 2048, 151936
    S, K = a.streams, a.block
    max_ctx = a.context + (a.rounds + a.warmup + 8) * (K + 1) + 64
    ctx = capi.Ctx(0)
    target = Model(ctx, ModelConfig(a.layers, D, 32, 4, 128, 256, V, max_ctx, 1e-6, 1e6))
    target.set_moe(E, TOPK, F)
    target.fill_synthetic(capi.MXFP4, seed=1)
    draft = Model(ctx, ModelConfig(a.draft_layers, D, 32, 4, 128, 256, V, max_ctx, 1e-6, 1e6))
    draft.set_moe(E, TOPK, F)
    for l in range(a.draft_layers):
        draft.share(l, target, l)
    draft.share(-1, target, -1)
    sess = Session(ctx, target, draft, S, K + 1, page_tokens=64)
    sess.fill_context(a.context, seed=7)
    rc = run_config(shaping(temperature=1.0, seed=2), 1 << 30, K, uniform_mode=1)
    nxt = np.random.default_rng(1).integers(0, V, size=S).astype(np.int32)
    steps = np.zeros(S, dtype=np.uint64)
    for _ in range(a.warmup):
        sess.round(rc, nxt, steps)
    committed, dev_ms = 0, 0.0
    for _ in range(a.rounds):
        acc = sess.round(rc, nxt, steps)
        committed += int(acc.sum()) + S
        dev_ms += sess.round_times()[3]
    sess.set_graph(False)
    phase = np.zeros(3)
    for _ in range(3):
        sess.round(rc, nxt, steps)
        phase += np.array(sess.round_times()[:3])
    phase /= 3
    rows = S * (K + 1)
    rb = lambda cols: cols // 32 * 17
    per_expert = 2 * F * rb(D) + D * rb(F)
    attn = (32 * 128 + 2 * 4 * 128) * rb(D) + D * rb(32 * 128)
    distinct = E * (1.0 - (1.0 - TOPK / E) ** rows)
    verify_bytes = a.layers * (attn + E * D + distinct * per_expert + S * a.context * 4 * 128 * 4) + V * rb(D)
    print(json.dumps({
        "workload": "routed model %d layers, d %d, %d experts top-%d width %d, MXFP4, K=%d, context %d, %d stream(s)" %
                    (a.layers, D, E, TOPK, F, K, a.context, S),
        "tokens_per_s": committed / (dev_ms * 1e-3), "ms_per_round": dev_ms / a.rounds, "committed_per_round": committed / a.rounds / S,
        "phases_ms": {"draft": phase[0], "verify": phase[1], "accept": phase[2]},
        "verify_pass": {"rows": rows, "expected_distinct_experts_per_layer": distinct, "algorithmic_bytes": verify_bytes,
                        "gbs": verify_bytes / (phase[1] * 1e-3) / 1e9},
        "weights_bytes": target.weight_bytes, "launches_total": ctx.launches}), flush=True)
    sess.close(), draft.close(), target.close(), ctx.close()


if __name__ == "__main__":
    main()
