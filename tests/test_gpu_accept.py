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
