"""The device acceptance / sampling kernels against the CPU oracle's restatement of the reference sampler.

Accepted lengths and token ids must be identical; the decision margins the kernel reports must
show that no uniform sat on a boundary (otherwise equality would be luck).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    yield c
    c.close()


def _logits(oracle, rng, batch, k, vocab, noise=1.0):
    tgt = rng.standard_normal((batch, k + 1, vocab)).astype(np.float32) * 3.0
    drf = tgt[:, :k, :] + rng.standard_normal((batch, k, vocab)).astype(np.float32) * noise
    return oracle.f32_to_f16_bits(tgt), oracle.f32_to_f16_bits(drf)


def _run_accept(ctx, oracle, t16, d16, props, unis, temperature, **shape):
    import turbospark_b200 as tsb
    batch, kp1, vocab = t16.shape
    k = kp1 - 1
    cfg = tsb.shaping(temperature=temperature, seed=4, **shape)
    out = ctx.alloc(batch * C.sizeof(tsb.AcceptOut))
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, k, vocab))
    ctx.accept(ctx.to_device(t16), ctx.to_device(d16) if k else None, ctx.to_device(props) if k else None,
               ctx.to_device(unis), batch, k, vocab, cfg, out, scratch)
    ctx.sync()
    raw = out.download(np.uint8, batch * C.sizeof(tsb.AcceptOut))
    return [tsb.AcceptOut.from_buffer_copy(raw[i * C.sizeof(tsb.AcceptOut):(i + 1) * C.sizeof(tsb.AcceptOut)].tobytes())
            for i in range(batch)]


@pytest.mark.parametrize("temperature", [1.0, 0.7, 0.0])
@pytest.mark.parametrize("vocab,batch,k", [(8192, 16, 4), (128256, 6, 5), (151936, 3, 4)])
def test_accept_matches_the_oracle(ctx, oracle, temperature, vocab, batch, k):
    rng = np.random.default_rng(vocab + int(temperature * 10))
    t16, d16 = _logits(oracle, rng, batch, k, vocab)
    ocfg = oracle.shaping(temperature=temperature, seed=4)
    # proposals drawn from q, as the loop does (argmax at temperature 0)
    props = np.zeros((batch, k), dtype=np.int32)
    unis = np.zeros((batch, 2 * k + 1), dtype=np.uint64)
    for b in range(batch):
        for i in range(k):
            props[b, i] = oracle.sample(d16[b, i], ocfg, oracle.uniform_u64(1, 4, 1000 * b + i))[0]
        for j in range(2 * k + 1):
            unis[b, j] = oracle.uniform_u64(1, 4, 5000 + 100 * b + j)  # Philox4x32-10, seed 4
    outs = _run_accept(ctx, oracle, t16, d16, props, unis, temperature)
    rejected = 0
    for b in range(batch):
        acc, toks, draws, margins = oracle.accept_round(t16[b], d16[b], props[b], ocfg, unis[b])
        o = outs[b]
        assert o.status == 0
        assert o.accepted == acc, (b, o.accepted, acc)
        assert list(o.tokens[:acc + 1]) == list(toks), (b, list(o.tokens[:acc + 1]), list(toks))
        assert o.draws == draws
        if temperature != 0.0:
            assert o.margin_draw > 1e-12 and margins[1] > 1e-12
            if np.isfinite(margins[0]):
                assert abs(o.margin_accept - margins[0]) <= 1e-9 * max(1.0, margins[0]) + 1e-15
        rejected += acc < k
    if temperature != 0.0:
        assert rejected > 0  # the residual path was exercised


def test_identical_distributions_accept_everything_and_draw_the_bonus_from_p(ctx, oracle):
    rng = np.random.default_rng(2)
    batch, k, vocab = 4, 3, 4096
    t16, _ = _logits(oracle, rng, batch, k, vocab)
    d16 = t16[:, :k, :].copy()
    ocfg = oracle.shaping(temperature=1.0, seed=1)
    props = rng.integers(0, vocab, size=(batch, k)).astype(np.int32)
    unis = rng.integers(0, 2**63, size=(batch, 2 * k + 1)).astype(np.uint64)
    outs = _run_accept(ctx, oracle, t16, d16, props, unis, 1.0)
    for b in range(batch):
        acc, toks, draws, _ = oracle.accept_round(t16[b], d16[b], props[b], ocfg, unis[b])
        assert acc == k and outs[b].accepted == k
        assert list(outs[b].tokens[:k + 1]) == list(toks)


def test_residual_fallback_tail_and_extreme_logits(ctx, oracle):
    # a row of +-60000 logits: underflowed exps tie by index, the draw must still land on the peak;
    # a uniform of all ones exercises the tail fallback (last support entry in rank order)
    vocab, k = 1024, 1
    ocfg = oracle.shaping(temperature=1.0, seed=1)
    tgt = np.full((1, 2, vocab), -60000.0, dtype=np.float32)
    tgt[0, 0, 7] = 60000.0
    tgt[0, 1, 9] = 60000.0
    drf = np.zeros((1, 1, vocab), dtype=np.float32)
    t16, d16 = oracle.f32_to_f16_bits(tgt), oracle.f32_to_f16_bits(drf)
    for prop, u in ((3, 0), (7, 0), (3, 2**64 - 1), (7, 2**64 - 1), (3, 1 << 63)):
        props = np.array([[prop]], dtype=np.int32)
        unis = np.array([[u, u, u]], dtype=np.uint64)
        outs = _run_accept(ctx, oracle, t16, d16, props, unis, 1.0)
        acc, toks, draws, _ = oracle.accept_round(t16[0], d16[0], props[0], ocfg, unis[0])
        assert outs[0].accepted == acc and list(outs[0].tokens[:acc + 1]) == list(toks), (prop, u)
    # flat distribution, uniform at the very top of [0,1): tail or last bin, both sides must agree
    flat = oracle.f32_to_f16_bits(np.zeros((1, 1, vocab), dtype=np.float32))
    unis = np.array([[2**64 - 1]], dtype=np.uint64)
    outs = _run_accept(ctx, oracle, flat, None, None, unis, 1.0)
    acc, toks, _, _ = oracle.accept_round(flat[0], np.zeros((0, vocab), np.uint16), [], ocfg, unis[0])
    assert outs[0].tokens[0] == toks[0]


def test_non_finite_logits_are_reported_not_sampled(ctx, oracle):
    vocab, k = 512, 2
    rng = np.random.default_rng(1)
    t16, d16 = _logits(oracle, rng, 2, k, vocab)
    t16[1, 1, 5] = 0x7C00  # +inf
    props = np.zeros((2, k), dtype=np.int32)
    unis = np.ones((2, 2 * k + 1), dtype=np.uint64)
    outs = _run_accept(ctx, oracle, t16, d16, props, unis, 1.0)
    assert outs[0].status == 0 and outs[1].status != 0


def test_unsupported_shaping_is_refused(ctx, oracle):
    import turbospark_b200 as tsb
    out = ctx.alloc(256)
    scratch = ctx.alloc(ctx.accept_scratch_bytes(1, 1, 64))
    buf = ctx.alloc(4096)
    for cfg in (tsb.shaping(temperature=0.7, top_k=300), tsb.shaping(temperature=0.7, top_p=1.5), tsb.shaping(temperature=0.7, min_p=2.0),
                tsb.shaping(temperature=1.0, repetition_penalty=1.1), tsb.shaping(temperature=1.0, presence_penalty=0.5),
                tsb.shaping(temperature=-1.0)):
        with pytest.raises(tsb.TsbError):
            ctx.accept(buf, buf, buf, buf, 1, 1, 64, cfg, out, scratch)


@pytest.mark.parametrize("temperature", [1.0, 0.7, 0.0])
def test_sample_matches_the_oracle_draw(ctx, oracle, temperature):
    import turbospark_b200 as tsb
    rng = np.random.default_rng(11)
    batch, vocab = 24, 128256
    lg = oracle.f32_to_f16_bits(rng.standard_normal((batch, vocab)).astype(np.float32) * 3.0)
    unis = np.array([oracle.uniform_u64(0, 2, i) for i in range(batch)], dtype=np.uint64)  # derive_step_value(seed 2, i)
    toks = ctx.alloc(batch * 4)
    margins = ctx.alloc(batch * 8)
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, 0, vocab))
    ctx.sample(ctx.to_device(lg), ctx.to_device(unis), batch, vocab, tsb.shaping(temperature=temperature), toks, margins,
               scratch)
    ctx.sync()
    got = toks.download(np.int32, batch)
    ocfg = oracle.shaping(temperature=temperature, seed=2)
    for b in range(batch):
        want, margin = oracle.sample(lg[b], ocfg, int(unis[b]))
        assert got[b] == want, (b, got[b], want, margin)
    # the reference's own identity: the materialised distribution draws what select draws
    if temperature != 0.0:
        for b in range(4):
            assert oracle.select(lg[b], ocfg, None, b) == got[b]


SHAPES = [dict(top_k=64, top_p=0.95), dict(top_p=0.9), dict(top_k=8), dict(min_p=0.05), dict(top_k=40, top_p=0.8, min_p=0.02),
          dict(top_k=1), dict(top_p=1.0)]


@pytest.mark.parametrize("shape", SHAPES, ids=[str(sorted(d.items())) for d in SHAPES])
@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_truncated_sampling_matches_the_oracle_draw(ctx, oracle, temperature, shape):
    """top-k, top-p and min-p on the device: the support is the same rank-order prefix the reference keeps
    (crates/selection/src/choose.rs:176-222) and the draw over it lands on the same token."""
    import turbospark_b200 as tsb
    rng = np.random.default_rng(21)
    batch, vocab = 32, 32000
    lg = oracle.f32_to_f16_bits(rng.standard_normal((batch, vocab)).astype(np.float32) * 3.0)
    lg[0, :] = lg[0, 0]                # every logit equal: the rank order is the index order
    lg[1, 100:200] = lg[1, 100]        # a run of ties crossing the top-k cut
    unis = np.array([oracle.uniform_u64(0, 2, i) for i in range(batch)], dtype=np.uint64)
    toks = ctx.alloc(batch * 4)
    margins = ctx.alloc(batch * 8)
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, 0, vocab))
    ctx.sample(ctx.to_device(lg), ctx.to_device(unis), batch, vocab, tsb.shaping(temperature=temperature, **shape), toks, margins, scratch)
    ctx.sync()
    got = toks.download(np.int32, batch)
    ocfg = oracle.shaping(temperature=temperature, seed=2, **shape)
    for b in range(batch):
        want, margin = oracle.sample(lg[b], ocfg, int(unis[b]))
        assert got[b] == want, (b, got[b], want, margin)


@pytest.mark.parametrize("shape", SHAPES[:5], ids=[str(sorted(d.items())) for d in SHAPES[:5]])
@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_truncated_acceptance_matches_the_oracle(ctx, oracle, temperature, shape):
    rng = np.random.default_rng(31)
    vocab, batch, k = 32000, 12, 4
    t16, d16 = _logits(oracle, rng, batch, k, vocab, noise=0.5)
    ocfg = oracle.shaping(temperature=temperature, seed=4, **shape)
    props = np.zeros((batch, k), dtype=np.int32)
    unis = np.zeros((batch, 2 * k + 1), dtype=np.uint64)
    for b in range(batch):
        for i in range(k):
            props[b, i] = oracle.sample(d16[b, i], ocfg, oracle.uniform_u64(1, 4, 1000 * b + i))[0]
        for j in range(2 * k + 1):
            unis[b, j] = oracle.uniform_u64(1, 4, 5000 + 100 * b + j)
    props[0, 1] = int(np.argmin(oracle.f16_bits_to_f32(t16[0, 1])))  # a proposal outside the target's support: p(x) = 0
    outs = _run_accept(ctx, oracle, t16, d16, props, unis, temperature, **shape)
    for b in range(batch):
        acc, toks, draws, margins = oracle.accept_round(t16[b], d16[b], props[b], ocfg, unis[b])
        o = outs[b]
        assert o.status == 0
        assert o.accepted == acc, (b, o.accepted, acc)
        assert list(o.tokens[:acc + 1]) == list(toks), (b, list(o.tokens[:acc + 1]), list(toks))
        assert o.draws == draws


def _run_accept_history(ctx, t16, d16, props, unis, cfg, history, generated):
    import turbospark_b200 as tsb
    batch, kp1, vocab = t16.shape
    k = kp1 - 1
    stride = max(len(h) for h in history) + 1
    hist = np.zeros((batch, stride), dtype=np.int32)
    for b, h in enumerate(history):
        hist[b, :len(h)] = h
    hl = np.array([len(h) for h in history], dtype=np.int32)
    gen = np.array(generated, dtype=np.int32)
    out = ctx.alloc(batch * C.sizeof(tsb.AcceptOut))
    scratch = ctx.alloc(ctx.accept_history_scratch_bytes(batch, k, vocab))
    ctx.accept_history(ctx.to_device(t16), ctx.to_device(d16), ctx.to_device(props), ctx.to_device(unis), batch, k, vocab, cfg,
                       ctx.to_device(hist), stride, ctx.to_device(hl), ctx.to_device(gen), out, scratch)
    ctx.sync()
    raw = out.download(np.uint8, batch * C.sizeof(tsb.AcceptOut))
    sz = C.sizeof(tsb.AcceptOut)
    return [tsb.AcceptOut.from_buffer_copy(raw[i * sz:(i + 1) * sz].tobytes()) for i in range(batch)]


@pytest.mark.parametrize("vocab,batch,k", [(8192, 8, 4), (128256, 3, 5)])
@pytest.mark.parametrize("shape", [dict(repetition_penalty=1.1, presence_penalty=0.5, frequency_penalty=0.3, top_k=64, top_p=0.95),
                                   dict(repetition_penalty=1.3), dict(presence_penalty=0.7, frequency_penalty=0.2, min_p=0.02),
                                   dict(repetition_penalty=0.8, frequency_penalty=1.5)])
def test_acceptance_with_history_penalties_matches_the_oracle(ctx, oracle, vocab, batch, k, shape):
    """Repetition over the whole history (each distinct id once), presence / frequency over the generated suffix
    (crates/selection/src/penalty.rs:15-82), before the softmax; target row i sees the proposals accepted before it, a
    drafter row the history of the round's start (crates/runtime/src/speculative.rs:636-648,701-734)."""
    import turbospark_b200 as tsb
    temperature = 0.7
    rng = np.random.default_rng(vocab + k + len(shape))
    t16, d16 = _logits(oracle, rng, batch, k, vocab)
    ocfg = oracle.shaping(temperature=temperature, seed=4, **shape)
    cfg = tsb.shaping(temperature=temperature, seed=4, **shape)
    history, generated = [], []
    for b in range(batch):
        n = int(rng.integers(5, 60))
        h = rng.integers(0, vocab, size=n).astype(np.int32)
        # repeats, among them the likeliest tokens of the rows (so the penalties move decisions, not only tails)
        top = np.argsort(-oracle.f16_bits_to_f32(t16[b, 0]))[:6].astype(np.int32)
        h = np.concatenate([h, top, top[:3], h[:4]])
        history.append(h)
        generated.append(int(rng.integers(0, len(h) + 1)))
    props = np.zeros((batch, k), dtype=np.int32)
    unis = np.zeros((batch, 2 * k + 1), dtype=np.uint64)
    for b in range(batch):
        for i in range(k):  # drawn from q under the round-start history, as the loop does
            props[b, i] = oracle.sample(d16[b, i], ocfg, oracle.uniform_u64(1, 4, 1000 * b + i), history[b], generated[b])[0]
        for j in range(2 * k + 1):
            unis[b, j] = oracle.uniform_u64(1, 4, 5000 + 100 * b + j)
    outs = _run_accept_history(ctx, t16, d16, props, unis, cfg, history, generated)
    plain = _run_accept(ctx, oracle, t16, d16, props, unis, temperature, **{k_: v for k_, v in shape.items() if k_ in ("top_k", "top_p", "min_p")})
    moved = 0
    for b in range(batch):
        acc, toks, draws, margins = oracle.accept_round(t16[b], d16[b], props[b], ocfg, unis[b], history[b], generated[b])
        o = outs[b]
        assert o.status == 0
        assert o.accepted == acc, (b, o.accepted, acc)
        assert list(o.tokens[:acc + 1]) == list(toks), (b, list(o.tokens[:acc + 1]), list(toks))
        assert o.draws == draws
        assert o.margin_draw > 1e-12 and margins[1] > 1e-12
        moved += (plain[b].accepted != acc) or list(plain[b].tokens[:acc + 1]) != list(toks)
    if batch >= 8:
        assert moved > 0  # the penalties changed at least one decision, so the test is not vacuous


def test_identity_penalties_through_the_history_path_equal_the_plain_path(ctx, oracle):
    import turbospark_b200 as tsb
    rng = np.random.default_rng(12)
    batch, k, vocab = 4, 3, 32000
    t16, d16 = _logits(oracle, rng, batch, k, vocab)
    ocfg = oracle.shaping(temperature=1.0, seed=4)
    props = np.array([[oracle.sample(d16[b, i], ocfg, oracle.uniform_u64(1, 4, 10 * b + i))[0] for i in range(k)] for b in range(batch)],
                     dtype=np.int32)
    unis = rng.integers(0, 2**63, size=(batch, 2 * k + 1)).astype(np.uint64)
    hist = [rng.integers(0, vocab, size=20).astype(np.int32) for _ in range(batch)]
    a = _run_accept_history(ctx, t16, d16, props, unis, tsb.shaping(temperature=1.0, seed=4), hist, [7] * batch)
    b_ = _run_accept(ctx, oracle, t16, d16, props, unis, 1.0)
    for x, y in zip(a, b_):
        assert (x.accepted, list(x.tokens), x.draws, x.margin_accept, x.margin_draw) == (y.accepted, list(y.tokens), y.draws, y.margin_accept, y.margin_draw)


@pytest.mark.parametrize("shape", [dict(repetition_penalty=1.2, presence_penalty=0.4, frequency_penalty=0.25, top_k=40),
                                   dict(repetition_penalty=1.5)])
def test_sampling_with_history_penalties_matches_the_oracle(ctx, oracle, shape):
    import turbospark_b200 as tsb
    rng = np.random.default_rng(8)
    batch, vocab = 16, 128256
    lg = oracle.f32_to_f16_bits((rng.standard_normal((batch, vocab)) * 3.0).astype(np.float32))
    ocfg = oracle.shaping(temperature=0.9, seed=1, **shape)
    cfg = tsb.shaping(temperature=0.9, seed=1, **shape)
    stride = 80
    hist = np.zeros((batch, stride), dtype=np.int32)
    hl = np.zeros(batch, dtype=np.int32)
    gen = np.zeros(batch, dtype=np.int32)
    for b in range(batch):
        top = np.argsort(-oracle.f16_bits_to_f32(lg[b]))[:8].astype(np.int32)
        h = np.concatenate([rng.integers(0, vocab, size=int(rng.integers(0, 50))).astype(np.int32), top, top[:2], [vocab + 5, -3]])
        hist[b, :len(h)], hl[b], gen[b] = h, len(h), int(rng.integers(0, len(h) + 1))
    unis = np.array([oracle.uniform_u64(1, 9, b) for b in range(batch)], dtype=np.uint64)
    toks, margins = ctx.alloc(batch * 4), ctx.alloc(batch * 8)
    scratch = ctx.alloc(ctx.accept_history_scratch_bytes(batch, 0, vocab))
    ctx.sample_history(ctx.to_device(lg), ctx.to_device(unis), batch, vocab, cfg, ctx.to_device(hist), stride, ctx.to_device(hl),
                       ctx.to_device(gen), toks, margins, scratch)
    ctx.sync()
    got = toks.download(np.int32, batch)
    want = [oracle.sample(lg[b], ocfg, int(unis[b]), hist[b, :hl[b]], int(gen[b]))[0] for b in range(batch)]
    assert list(got) == want
    # the plain entry point refuses what it cannot apply
    with pytest.raises(tsb.TsbError):
        ctx.sample(ctx.to_device(lg), ctx.to_device(unis), batch, vocab, cfg, toks, margins, ctx.alloc(ctx.accept_scratch_bytes(batch, 1, vocab)))
