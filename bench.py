#!/usr/bin/env python
"""Benchmark of the speculative-decoding verify path (8B-shape Q4_K target, K = 5).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--streams S]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

A step is one speculative round for every stream of the rank: K draft steps of the 16-layer drafter plus
its row-only step, one batched verify pass of K+1 rows per stream through the 32-layer target, the
device acceptance kernel, cursor commit.  Weights are synthetic valid Q4_K blocks generated on the
device, the 4096-token context is pre-filled with seeded pseudo-random K/V, token ids are random.
Streams are independent and replicated per GPU with no collective ("scaling": "weak").

`--impl reference` times the CPU restatement of the reference's own CPU operators (the oracle) on
the host cores for a bounded sample of the same round, scales the sample to a whole round and prints the
same line (marked "extrapolated", with the scale factors).  Both arms also print rounds_per_s, which needs
no assumption about how many tokens a round commits.

A second, short leg (`streams64`) runs the same round with 64 streams in total, 64 / N per GPU: the
strong-scaling case of the benchmark definition beside the one-stream-per-GPU line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "accepted tokens/s/GPU (8B-shape Q4_K, K=5 spec-decode); verify-pass HBM GB/s"
BLOCK = 5
CONTEXT = 4096


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, the figure used when no measured peak file is present)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.time()])

    def window(self, t0, t1):
        """Keep the samples taken between t0 and t1 (host clock); all of them when none fell inside."""
        inside = [r for r in self.rows if t0 <= r[-1] <= t1]
        if inside:
            self.rows = inside

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        time.sleep(0.05)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 3 + i and str(r[2 + i]).lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# DRAM bytes (read + write) of a captured launch of the matmul kernel over its algorithmic bytes: every weight byte
# is read once, the rest is activations and the profiler's own traffic.  Traffic grows with the weight bytes, so the
# ratio of the captured 132 MB launch is applied to the timed launches (labelled as scaled in the line).
NCU_TRAFFIC_RATIO = 1.034
# What a round of the synthetic (random, unrelated) model pair commits on average: the bonus / corrected token plus
# ~0.6 accepted proposals.  The reference arm cannot measure it (it times operators, not a generation), so its
# tokens/s uses this figure unless TSB_COMMITTED_PER_ROUND gives the GPU arm's measured one; rounds_per_s needs neither.
COMMITTED_PER_ROUND_SYNTHETIC = 1.6


def cpu_round_estimate(threads):
    """Bounded CPU sample of one round on the oracle: one target layer's matmuls at K+1 rows, one layer of
    attention at the benchmark context, one drafter layer at 1 row, 1/16 of the head; scaled to the full
    round.  Returns (seconds per round, description)."""
    import numpy as np
    from oracle import pyoracle as o
    rng = np.random.default_rng(0)
    M = BLOCK + 1

    def t_gemm(rows, cols, tokens, scale=1.0):
        sub = max(256, int(rows * scale) // 256 * 256)
        base = o.quantize(o.Q4K, (rng.standard_normal((256, cols)) * 0.02).astype(np.float32))
        q = np.tile(base, (sub // 256, 1))
        x = rng.standard_normal((tokens, cols)).astype(np.float32)
        t0 = time.perf_counter()
        o.gemm_quant(o.Q4K, q, sub, cols, x, threads=threads)
        return (time.perf_counter() - t0) * rows / sub

    tl = t_gemm(6144, 4096, M) + t_gemm(4096, 4096, M) + t_gemm(28672, 4096, M, 0.25) + t_gemm(4096, 14336, M, 0.5)
    th = t_gemm(128256, 4096, M, 1.0 / 16)
    dl = t_gemm(4096, 2048, 1) + t_gemm(2048, 2048, 1) + t_gemm(16384, 2048, 1, 0.5) + t_gemm(2048, 8192, 1)
    dh = t_gemm(128256, 2048, 1, 1.0 / 16)
    # attention: one row of one layer at the benchmark context (the oracle is single-threaded per row)
    hd, nq, nkv = 128, 32, 8
    k = rng.standard_normal((CONTEXT, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((CONTEXT, nkv * hd)).astype(np.float32)
    qv = rng.standard_normal(nq * hd).astype(np.float32)
    t0 = time.perf_counter()
    o.causal_attention(qv, k, v, hd, nq, nkv, CONTEXT, 1.0 / np.sqrt(hd))
    ta = (time.perf_counter() - t0) * M / max(1, min(threads, M))
    verify = 32 * (tl + ta) + th
    draft = BLOCK * (16 * (dl + ta / M / 2) + dh) + 16 * (dl + ta / M / 2)
    return verify + draft, ("oracle (C++ restatement of crates/compute operators), %d threads: 1 of 32 target layers "
                            "(1/4 of gate|up rows, 1/2 of down rows), 1/16 of the head, 1 of 16 drafter layers, one attention "
                            "row at context %d; scaled to a full K=%d round" % (threads, CONTEXT, BLOCK))


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    secs = []
    desc = ""
    for i in range(args.warmup + args.steps):
        s, desc = cpu_round_estimate(threads)
        if i >= args.warmup:
            secs.append(s)
        if sum(secs) > 0 and time.perf_counter() - run_reference.t0 > 150:
            break
    per_round = statistics.mean(secs)
    # committed tokens per round are a property of the logits, not of who computes them
    cpr = float(os.environ.get("TSB_COMMITTED_PER_ROUND", str(COMMITTED_PER_ROUND_SYNTHETIC)))
    value = cpr / per_round
    line = {"metric": METRIC, "impl": "reference", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(secs),
            "warmup": args.warmup, "ms_per_step": per_round * 1e3, "rounds_per_s": 1.0 / per_round, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 accumulate over Q4_K blocks, f16 activations", "data": "synthetic",
            "extrapolated": True,
            "sample_scale": {"target_layers": "1 of 32", "gate_up_rows": "1/4", "down_rows": "1/2", "head_rows": "1/16",
                             "drafter_layers": "1 of 16", "attention_rows": "1 timed, scaled to K+1"},
            "config": {"workload": "configs[2] dense 8B-shape Q4_K target + 16-layer drafter, K=5, context 4096, 1 stream",
                       "committed_per_round_assumed": cpr,
                       "value_definition": "committed_per_round_assumed / seconds per round (a bounded operator sample scaled to a round)"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


run_reference.t0 = time.perf_counter()


def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch
    import turbospark_b200 as tsb

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = tsb.Ctx(local_rank)
    S, K = args.streams, BLOCK
    max_ctx = CONTEXT + (args.steps + args.warmup + 8) * (K + 1) + 64
    # the sampler starts before the set-up (nvidia-smi takes a while to come up on a box with eight GPUs); only the
    # samples that fall inside the timed region are reported
    sampler = ClockSampler(local_rank)
    sampler.start()
    target = tsb.Model(ctx, tsb.config_8b_target(max_ctx))
    target.fill_synthetic(tsb.Q4_K, seed=1)
    draft = tsb.Model(ctx, tsb.config_8b_draft(max_ctx))
    draft.fill_synthetic(tsb.Q4_K, seed=2)
    sess = tsb.Session(ctx, target, draft, S, K + 1, page_tokens=64)
    sess.fill_context(CONTEXT, seed=7 + rank)
    rc = tsb.run_config(tsb.shaping(temperature=1.0, seed=2 + 1000 * rank), 1 << 30, K, uniform_mode=1)
    rng = np.random.default_rng(1 + rank)
    nxt = rng.integers(0, target.cfg.vocab, size=S).astype(np.int32)
    steps_ctr = np.zeros(S, dtype=np.uint64)
    stream = torch.cuda.ExternalStream(sess.stream_ptr)

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        sess.round(rc, nxt, steps_ctr)
    barrier()
    t_begin = time.time()
    launches0 = ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    committed = accepted = 0
    dev_ms = 0.0
    e0.record(stream)
    for _ in range(args.steps):
        acc = sess.round(rc, nxt, steps_ctr)
        accepted += int(acc.sum())
        committed += int(acc.sum()) + S
        dev_ms += sess.round_times()[3]   # device time of the round: inputs resident, no host gaps
    e1.record(stream)
    barrier()
    sampler.window(t_begin, time.time())
    clocks = sampler.stop()
    launches = ctx.launches - launches0
    e2e_ms = e0.elapsed_time(e1)          # whole loop: host staging, H2D, kernels, D2H, host commit
    # per-phase device times need event records between the phases, which a graphed round does not have:
    # a few plain-launch rounds after the timed region give the split (reported, not part of `value`)
    sess.set_graph(False)
    phase = np.zeros(3)
    n_phase = 3
    for _ in range(n_phase):
        sess.round(rc, nxt, steps_ctr)
        phase += np.array(sess.round_times()[:3])
    phase *= args.steps / n_phase
    sess.set_graph(True)
    times = torch.tensor([e2e_ms, dev_ms, float(committed), float(phase[1])], dtype=torch.float64, device="cuda")
    if dist:
        mx = times.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = times.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        e2e_ms, dev_ms, verify_ms = float(mx[0]), float(mx[1]), float(mx[3])
        committed_all = float(sm[2])
    else:
        verify_ms, committed_all = float(phase[1]), float(committed)

    # roofline of the dominant kernel: the quantized matmul exactly as the verify pass launches it (fused epilogues),
    # timed over the target's own layer weights without the attention, embedding and head launches between
    peak, peak_src = peaks()
    if S * (K + 1) < 24:
        mm_ms, mm_bytes, mm_launches = sess.time_matmuls(S * (K + 1), 3)
        rest_ms = sess.time_pass_rest(S * (K + 1), 3)   # embedding, attention and head of the pass, back to back
    else:
        # with 24 verify rows and more the session's target runs the tensor-memory matmul: the few-row kernel this
        # block describes is not what the pass launches, so no roofline block is printed for such a run
        mm_ms, mm_bytes, mm_launches = 1.0, 0, 1
        rest_ms = 0.0
    achieved = mm_bytes / (mm_ms * 1e-3) / 1e9
    tb, db = target.weight_bytes, draft.weight_bytes
    kv_bytes = 32 * CONTEXT * 8 * 128 * 2 * 2 * S
    verify_bytes = tb + kv_bytes
    verify_gbs = verify_bytes / (verify_ms / args.steps * 1e-3) / 1e9

    # ---- second leg: 64 streams in total, 64 / world per GPU (the strong-scaling case of the benchmark definition)
    s64 = None
    if not args.no_streams64 and 64 % world == 0:
        sess.close()
        sess = None
        S64 = 64 // world
        max_ctx64 = CONTEXT + 12 * (K + 1) + 64
        t64 = tsb.Model(ctx, tsb.config_8b_target(max_ctx64))
        t64.share(-1, target, -1)
        d64 = tsb.Model(ctx, tsb.config_8b_draft(max_ctx64))
        d64.share(-1, draft, -1)
        for l in range(32):
            t64.share(l, target, l)
        for l in range(16):
            d64.share(l, draft, l)
        sess64 = tsb.Session(ctx, t64, d64, S64, K + 1, page_tokens=64)
        sess64.fill_context(CONTEXT, seed=70 + rank)
        nxt64 = rng.integers(0, target.cfg.vocab, size=S64).astype(np.int32)
        ctr64 = np.zeros(S64, dtype=np.uint64)
        for _ in range(3):
            sess64.round(rc, nxt64, ctr64)
        barrier()
        n64, com64, ms64 = 5, 0, 0.0
        for _ in range(n64):
            acc = sess64.round(rc, nxt64, ctr64)
            com64 += int(acc.sum()) + S64
            ms64 += sess64.round_times()[3]
        sess64.set_graph(False)
        sess64.round(rc, nxt64, ctr64)
        ver64 = sess64.round_times()[1]
        t = torch.tensor([ms64, float(com64), ver64], dtype=torch.float64, device="cuda")
        if dist:
            mx = t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = t.clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            ms64, com64, ver64 = float(mx[0]), float(sm[1]), float(mx[2])
        bytes64 = target.weight_bytes + 32 * CONTEXT * 8 * 128 * 2 * 2 * S64
        s64 = {"streams_total": 64, "streams_per_gpu": S64, "rounds": n64, "tok_s": com64 / (ms64 * 1e-3), "ms_per_round": ms64 / n64,
               "verify_ms": ver64, "verify_rows_per_gpu": S64 * (K + 1), "verify_bytes_per_gpu": bytes64,
               "verify_frac": bytes64 / (ver64 * 1e-3) / 1e9 / peak}
        sess64.close(), t64.close(), d64.close()

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            secs, desc = cpu_round_estimate(threads)
            cpr = committed / (args.steps * S)
            cpu = {"value": cpr / secs, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc}
        n_rounds = args.steps
        line = {
            "metric": METRIC, "value": committed_all / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / n_rounds, "rounds_per_s": world * S * n_rounds / (dev_ms * 1e-3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 accumulate over Q4_K blocks, f16 activations", "data": "synthetic",
            "config": {"workload": "configs[2] dense 8B-shape speculative decode: 32-layer Q4_K target, 16-layer Q4_K drafter, "
                                   "chain K=5, context 4096 fp16 paged KV, %d stream(s) per GPU, temperature 1.0" % S,
                       "streams_per_gpu": S, "block": K, "context": CONTEXT,
                       "l2": "weights per pass (4.2 GB) exceed the 126 MB L2; no flush needed",
                       "accepted_per_round": accepted / (n_rounds * S), "committed_per_round": committed / (n_rounds * S),
                       "value_definition": "tokens committed per second (accepted proposals + the corrected/bonus token), SUMMED over all "
                                           "GPUs of the run (the metric's '/GPU' figure is value / n_gpus); with random unrelated "
                                           "draft and target weights the acceptance is a floor, so value ~ committed_per_round / ms_per_step"},
            "e2e": {"value": committed_all / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / n_rounds,
                    "h2d_bytes_per_step": S * ((K + 3) * 4 + (3 * K + 1) * 8 + (2 * K + 2) * 32), "d2h_bytes_per_step": S * 96},
            "gpu_launches": launches,
            "phases_ms_per_step": {"draft": phase[0] / n_rounds, "verify": phase[1] / n_rounds, "accept": phase[2] / n_rounds},
            "verify_pass": {"ms": verify_ms / n_rounds, "algorithmic_bytes": verify_bytes, "gbs": verify_gbs, "frac_of_peak": verify_gbs / peak,
                            "matmul_ms": mm_ms, "other_ms": verify_ms / n_rounds - mm_ms, "rest_ms": rest_ms,
                            "note": "matmul_ms = the pass's 128 layer matmuls back to back (roofline block); other_ms = attention, "
                                    "embedding, head and the gaps between launches; rest_ms = embedding, the 32 attention "
                                    "launch pairs and the head back to back, without the layer matmuls"},
            "roofline": {"bound": "hbm", "kernel": "gemm_quant_kernel<Q4_K> with the pass's fused epilogues (q|k|v + RoPE/store, o_proj and "
                                                    "down + residual/norm, gate|up + SiLU: all layer matmuls of one verify pass, %d rows)" % (S * (K + 1)),
                         "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                         "in_pass_frac": mm_bytes / (max(verify_ms / n_rounds - rest_ms, 1e-6) * 1e-3) / 1e9 / peak,
                         "in_pass_definition": "the same bytes over (the verify pass's time - rest_ms): what the layer matmuls "
                                               "reach between the pass's other launches",
                         "launches": mm_launches, "us_per_launch": mm_ms * 1e3 / mm_launches,
                         "bytes_per_launch": mm_bytes / mm_launches,
                         "traffic": NCU_TRAFFIC_RATIO * mm_bytes / mm_launches,
                         "traffic_source": "ncu capture of a 132 MB launch, scaled by algorithmic bytes"},
            "clocks": clocks,
            "weights_bytes": {"target": tb, "draft": db},
        }
        if S * (K + 1) >= 24:
            line["roofline"] = None
            for k_ in ("matmul_ms", "other_ms", "rest_ms", "note"):
                line["verify_pass"].pop(k_, None)
        if cpu:
            line["cpu_baseline"] = cpu
        if s64:
            line["streams64"] = s64
        print(json.dumps(line), flush=True)
    if sess is not None:
        sess.close()
    target.close(), draft.close(), ctx.close()
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--streams", type=int, default=1, help="independent request streams per GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-streams64", action="store_true", help="skip the 64-streams-in-total leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
