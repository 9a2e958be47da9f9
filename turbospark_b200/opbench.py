"""Operator timing: the quantized matmul, the split-KV attention and the acceptance kernel on their own.

    python -m turbospark_b200.opbench --op gemm --qtype q4k --rows 14336 --cols 4096 --tokens 6
    python -m turbospark_b200.opbench --op gemm --sweep            # the operator-sweep shapes
    python -m turbospark_b200.opbench --op attention --context 4096 --tokens 6
    python -m turbospark_b200.opbench --op accept --batch 64
    python -m turbospark_b200.opbench --op sample --batch 1

Each line reports the launch time (CUDA events around `--iters` back-to-back launches that rotate over weight
copies larger than the L2 cache, minimum of five repeats after warm-up) and the algorithmic bytes over that time.
The matmul is timed through tsb_gemm_quant_prepared (operand converted once, as a model pass does once per three or
four matrices); --whole-call times the one-call operator, which allocates and converts on every call.
Weights are random valid blocks (finite scales, random quants); values do not matter for timing.
"""
import argparse
import json

import numpy as np

from . import capi

QTYPES = {"q4k": (0, 256, 144), "q6k": (1, 256, 210), "mxfp4": (2, 32, 17), "q5k": (3, 256, 176), "q8_0": (4, 32, 34)}
L2_BYTES = 126 << 20


def random_blocks(qtype, rows, cols, rng):
    """[rows, cols/block * block_bytes] u8 of valid blocks: every byte random except the f16/e8m0 scale fields."""
    _, blk, nbytes = QTYPES[qtype]
    nb = cols // blk
    base_rows = min(rows, 64)
    b = rng.integers(0, 256, size=(base_rows, nb, nbytes), dtype=np.uint8)
    if qtype == "q4k":
        b[:, :, 0:2] = np.frombuffer(np.float16(7.7e-5).tobytes(), np.uint8)
        b[:, :, 2:4] = np.frombuffer(np.float16(5.8e-4).tobytes(), np.uint8)
    elif qtype == "q6k":
        b[:, :, 208:210] = np.frombuffer(np.float16(1.5e-5).tobytes(), np.uint8)
    elif qtype == "q5k":
        b[:, :, 0:2] = np.frombuffer(np.float16(3.7e-5).tobytes(), np.uint8)
        b[:, :, 2:4] = np.frombuffer(np.float16(5.7e-4).tobytes(), np.uint8)
    elif qtype == "q8_0":
        b[:, :, 0:2] = np.frombuffer(np.float16(2.7e-4).tobytes(), np.uint8)
    else:
        b[:, :, 0] = 119
    flat = b.reshape(base_rows, nb * nbytes)
    reps = (rows + base_rows - 1) // base_rows
    return np.ascontiguousarray(np.tile(flat, (reps, 1))[:rows])


def f16_bits(a):
    return np.asarray(a, dtype=np.float16).view(np.uint16)


def time_launches(fn, iters, repeats=5, warm=3):
    import torch
    torch.zeros(1, device="cuda")
    best = None
    for r in range(warm + repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if r >= warm:
            best = ms if best is None else min(best, ms)
    return best


def bench_gemm(ctx, qtype, rows, cols, tokens, iters, rng, repeats=5, warm=3, whole_call=False):
    kind, blk, nbytes = QTYPES[qtype]
    w_bytes = rows * (cols // blk) * nbytes
    copies = max(2, -(-2 * L2_BYTES // w_bytes))  # rotate over more than an L2's worth of distinct weights
    host = random_blocks(qtype, rows, cols, rng)
    ws = [ctx.upload_weights(host) for _ in range(copies)]
    x = ctx.to_device(f16_bits(rng.standard_normal((tokens, cols))))
    y = ctx.alloc(tokens * rows * 2)
    if whole_call:  # the one-call operator: stream-ordered allocation + operand conversion + matmul every time
        ms = time_launches(lambda i: ctx.gemm_quant(kind, ws[i % copies], rows, cols, x, y, tokens), iters, repeats, warm)
    else:  # the operand converted once into the caller's workspace, the matmul launch alone timed
        work = ctx.alloc(ctx.gemm_workspace_bytes(kind, rows, cols, tokens))
        ctx.gemm_prepare(kind, rows, cols, x, tokens, work)
        ms = time_launches(lambda i: ctx.gemm_quant_prepared(kind, ws[i % copies], rows, cols, x, work, y, tokens), iters, repeats, warm)
        work.free()
    algo = w_bytes + tokens * cols * 2 + tokens * rows * 2
    for w in ws:
        w.free()
    return {"op": "gemm", "qtype": qtype, "rows": rows, "cols": cols, "tokens": tokens, "us": round(ms * 1e3, 2),
            "bytes": algo, "gbs": round(algo / ms / 1e6, 1), "weight_copies": copies,
            "timed": "tsb_gemm_quant" if whole_call else "tsb_gemm_quant_prepared"}


def bench_attention(ctx, hd, nq, nkv, context, tokens, streams, iters, repeats=5, warm=3):
    page = 64
    pages_per = (context + tokens + page - 1) // page + 1
    layers = max(2, -(-2 * L2_BYTES // (streams * context * nkv * hd * 4)))
    kv = capi.KvCache(ctx, layers, nkv, hd, page, pages_per * streams + 2, streams, pages_per)
    for s in range(streams):
        kv.reserve(s, context + tokens)
        kv.fill_random(s, context + tokens, 7 + s)
    rows = streams * tokens
    rng = np.random.default_rng(5)
    q = ctx.to_device(f16_bits(rng.standard_normal((rows, nq * hd))))
    out = ctx.alloc(rows * nq * hd * 2)
    entries = [(s, context, m, context + m, (1 << (m + 1)) - 1) for s in range(streams) for m in range(tokens)]
    rd = ctx.to_device(capi.row_descs(entries))
    scratch = ctx.alloc(ctx.attn_scratch_bytes(rows, nq, hd))
    scale = float(1.0 / np.sqrt(hd))
    ms = time_launches(lambda i: ctx.attn_decode_rows(kv, i % layers, q, nq * hd, out, rd, rows, tokens, nq, scale,
                                                      context + tokens, scratch), iters, repeats, warm)
    algo = streams * (context + tokens) * nkv * hd * 4 + 2 * rows * nq * hd * 2
    kv.close()
    return {"op": "attention", "head_dim": hd, "q_heads": nq, "kv_heads": nkv, "context": context, "tokens": tokens,
            "streams": streams, "us": round(ms * 1e3, 2), "bytes": algo, "gbs": round(algo / ms / 1e6, 1), "kv_layers": layers}


def bench_accept(ctx, batch, k, vocab, iters, repeats=5, warm=3):
    rng = np.random.default_rng(4)
    t = rng.standard_normal((batch * (k + 1), vocab), dtype=np.float32) * 3.0
    d = t.reshape(batch, k + 1, vocab)[:, :k].reshape(batch * k, vocab) + rng.standard_normal((batch * k, vocab), dtype=np.float32)
    tl, dl = ctx.to_device(f16_bits(t)), ctx.to_device(f16_bits(d))
    props = ctx.to_device(rng.integers(0, vocab, size=batch * k).astype(np.int32))
    uni = ctx.to_device(rng.integers(0, 1 << 63, size=batch * (2 * k + 1), dtype=np.uint64))
    out = ctx.alloc(batch * 96)
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, k, vocab))
    cfg = capi.shaping(temperature=1.0)
    ms = time_launches(lambda i: ctx.accept(tl, dl, props, uni, batch, k, vocab, cfg, out, scratch), iters, repeats, warm)
    algo = batch * (2 * k + 1) * vocab * 2
    return {"op": "accept", "batch": batch, "k": k, "vocab": vocab, "us": round(ms * 1e3, 2), "bytes": algo,
            "gbs": round(algo / ms / 1e6, 1)}


def bench_sample(ctx, batch, vocab, iters, repeats=5, warm=3):
    rng = np.random.default_rng(6)
    lg = ctx.to_device(f16_bits(rng.standard_normal((batch, vocab), dtype=np.float32) * 3.0))
    uni = ctx.to_device(rng.integers(0, 1 << 63, size=batch, dtype=np.uint64))
    toks = ctx.alloc(batch * 4)
    margins = ctx.alloc(batch * 8)
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, 1, vocab))
    cfg = capi.shaping(temperature=1.0)
    ms = time_launches(lambda i: ctx.sample(lg, uni, batch, vocab, cfg, toks, margins, scratch), iters, repeats, warm)
    algo = batch * vocab * 2
    return {"op": "sample", "batch": batch, "vocab": vocab, "us": round(ms * 1e3, 2), "bytes": algo, "gbs": round(algo / ms / 1e6, 1)}


SWEEP_SHAPES = [(14336, 4096), (4096, 14336), (128256, 4096)]
SWEEP_TOKENS = [1, 2, 4, 6, 8, 16, 32, 64]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="gemm", choices=["gemm", "attention", "accept", "sample"])
    ap.add_argument("--qtype", default="q4k", choices=sorted(QTYPES))
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=6)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--warm", type=int, default=3)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--whole-call", action="store_true", help="time tsb_gemm_quant (allocation + conversion + matmul) instead of the prepared matmul")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--k", type=int, default=5)
    ap.add_argument("--vocab", type=int, default=128256)
    a = ap.parse_args()
    ctx = capi.Ctx(0)
    rng = np.random.default_rng(3)
    if a.op == "gemm":
        cases = [(q, r, c, t) for q in ("q4k", "mxfp4") for (r, c) in SWEEP_SHAPES for t in SWEEP_TOKENS] if a.sweep \
            else [(a.qtype, a.rows, a.cols, a.tokens)]
        for q, r, c, t in cases:
            print(json.dumps(bench_gemm(ctx, q, r, c, t, a.iters, rng, a.repeats, a.warm, a.whole_call)), flush=True)
    elif a.op == "attention":
        print(json.dumps(bench_attention(ctx, a.head_dim, a.q_heads, a.kv_heads, a.context, a.tokens, a.streams, a.iters,
                                         a.repeats, a.warm)), flush=True)
    elif a.op == "sample":
        print(json.dumps(bench_sample(ctx, a.batch, a.vocab, a.iters, a.repeats, a.warm)), flush=True)
    else:
        batches = [1, 4, 16, 64, 256] if a.sweep else [a.batch]
        for b in batches:
            print(json.dumps(bench_accept(ctx, b, a.k, a.vocab, a.iters, a.repeats, a.warm)), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
