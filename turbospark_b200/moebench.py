"""Speculative rounds over a routed (mixture-of-experts) model at the MoE configuration's shape.

    python -m turbospark_b200.moebench --streams 1 --rounds 20
    python -m turbospark_b200.moebench --streams 16 --rounds 10 --layers 48
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m turbospark_b200.moebench --streams 16

Under torch.distributed.run the ONE model is spread over the ranks: attention tensor-parallel over heads (an f32
all-reduce after o_proj), experts sharded 128 / world per rank (an f32 all-reduce of the per-slot outputs, exact), every
rank runs the same streams.  Without it the whole model sits on one GPU.

48 layers, d 2048, 32 query / 4 KV heads x 128, 128 experts of width 768 with top-8 routing, vocabulary 151 936,
MXFP4 blocks, context 4096 of pre-filled random K/V; the drafter is the target's first `--draft-layers` layers with
the shared head; chain depth K = 4, temperature 1.  Weights are seeded synthetic blocks, so routing is close to
uniform.  One JSON line: committed tokens/s, the device time of the phases, and the verify pass's achieved bytes/s
against the bytes it has to read: attention, router and head weights once, the distinct routed experts (their
expected number under uniform routing), and the K/V of every stream.
"""
import argparse
import json
import os

import numpy as np

from . import capi
from .model import Model, ModelConfig, Session, run_config
from .capi import shaping
from .sharding import HeadShard, expert_range


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
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    comm = None
    NQ, NKV = 32, 4
    if world > 1:
        import torch
        import torch.distributed as dist
        from .comm import Comm
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = capi.Ctx(local_rank)
    hs = HeadShard(NQ, NKV, 128, rank, world)
    e_lo, e_n = expert_range(E, rank, world)
    if world > 1:
        comm = Comm.from_torch_distributed(ctx)
    target = Model(ctx, ModelConfig(a.layers, D, hs.q_local, hs.kv_local, 128, 256, V, max_ctx, 1e-6, 1e6))
    target.set_moe(E, TOPK, F)
    if world > 1:
        target.set_expert_shard(e_lo, e_n)
    # replicated tensors (router, norms, embedding, head) must be the same bytes on every rank: the synthetic fill is
    # seeded per tensor, and routing only has to be the same everywhere, which the shared router seed gives
    target.fill_synthetic(capi.MXFP4, seed=1)
    draft = Model(ctx, ModelConfig(a.draft_layers, D, hs.q_local, hs.kv_local, 128, 256, V, max_ctx, 1e-6, 1e6))
    draft.set_moe(E, TOPK, F)
    if world > 1:
        draft.set_expert_shard(e_lo, e_n)
    for l in range(a.draft_layers):
        draft.share(l, target, l)
    draft.share(-1, target, -1)
    sess = Session(ctx, target, draft, S, K + 1, page_tokens=64)
    if comm is not None:
        sess.set_comm(comm)
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
    if world > 1:
        # the slowest rank's times (they run in lockstep through the collectives, so these are close)
        import torch
        import torch.distributed as dist
        t = torch.tensor([dev_ms, phase[0], phase[1], phase[2]], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, phase = float(t[0]), np.array([float(t[1]), float(t[2]), float(t[3])])
    rows = S * (K + 1)
    rb = lambda cols: cols // 32 * 17
    per_expert = 2 * F * rb(D) + D * rb(F)
    attn = (32 * 128 + 2 * 4 * 128) * rb(D) + D * rb(32 * 128)
    distinct = E * (1.0 - (1.0 - TOPK / E) ** rows)
    verify_bytes = a.layers * (attn + E * D + distinct * per_expert + S * a.context * 4 * 128 * 4) + V * rb(D)
    if rank == 0:
      print(json.dumps({
        "workload": "routed model %d layers, d %d, %d experts top-%d width %d, MXFP4, K=%d, context %d, %d stream(s)" %
                    (a.layers, D, E, TOPK, F, K, a.context, S),
        "n_gpus": world, "parallelism": "one replica" if world == 1 else "tp%d attention (f32 all-reduce) + ep%d experts (exact f32 all-reduce)" % (world, world),
        "tokens_per_s": committed / (dev_ms * 1e-3), "ms_per_round": dev_ms / a.rounds, "committed_per_round": committed / a.rounds / S,
        "phases_ms": {"draft": phase[0], "verify": phase[1], "accept": phase[2]},
        "verify_pass": {"rows": rows, "expected_distinct_experts_per_layer": distinct, "algorithmic_bytes": verify_bytes,
                        "gbs": verify_bytes / (phase[1] * 1e-3) / 1e9},
        "weights_bytes_per_gpu": target.weight_bytes, "launches_total": ctx.launches}), flush=True)
    sess.close(), draft.close(), target.close()
    if comm is not None:
        comm.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
