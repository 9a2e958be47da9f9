"""Mixture-of-experts routing and routed feed-forward on the GPU against the oracle's restatement of
router_topk_gemma4 and the two MoE kernels (crates/gpu/src/shaders/moe_gguf.metal:561-678)."""
import numpy as np
import pytest

from tests import weights

pytestmark = pytest.mark.gpu
REL, ABS = 2e-3, 1e-3


@pytest.fixture(scope="module")
def ctx():
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    yield c
    c.close()


@pytest.mark.parametrize("tokens,experts,k", [(1, 8, 2), (6, 128, 8), (40, 32, 4)])
def test_routing_matches_the_oracle_bit_for_bit(ctx, oracle, tokens, experts, k):
    rng = np.random.default_rng(tokens + experts)
    lg = rng.standard_normal((tokens, experts)).astype(np.float32)
    lg[0, min(3, experts - 1)] = lg[0, experts - 1] = 4.0  # a tie for first place: the lower index wins
    scale = (0.5 + rng.random(experts)).astype(np.float32)
    for sc in (None, scale):
        want_ids, want_w = oracle.moe_route(lg, k, sc)
        ids = ctx.alloc(tokens * k * 4)
        w = ctx.alloc(tokens * k * 2)
        ctx.moe_route(ctx.to_device(lg), tokens, experts, k, ids, w, scale=None if sc is None else ctx.to_device(sc))
        ctx.sync()
        got_ids = ids.download(np.int32, tokens * k).reshape(tokens, k)
        got_w = w.download(np.uint16, tokens * k).reshape(tokens, k)
        assert np.array_equal(got_ids, want_ids)
        # the weights are f16 roundings of an f32 softmax; the device uses a correctly rounded exp, glibc's expf may be
        # one ulp off before the rounding to f16
        d = np.abs(oracle.f16_bits_to_f32(got_w) - oracle.f16_bits_to_f32(want_w))
        assert np.all(d <= 1e-3 * np.abs(oracle.f16_bits_to_f32(want_w)) + 1e-7)
    assert got_ids[0, 0] == min(3, experts - 1)


@pytest.mark.parametrize("kind,tokens,experts,k,d,f", [(2, 5, 16, 4, 512, 256), (2, 6, 128, 8, 2048, 768), (0, 3, 8, 2, 512, 512),
                                                   (2, 150, 4, 2, 512, 256), (0, 40, 16, 4, 256, 256)])
def test_routed_feed_forward_matches_the_oracle(ctx, oracle, kind, tokens, experts, k, d, f):
    rng = np.random.default_rng(100 + tokens)
    gu = np.concatenate([oracle.quantize(kind, (rng.standard_normal((2 * f, d)) * 0.05).astype(np.float32)) for _ in range(experts)])
    dn = np.concatenate([oracle.quantize(kind, (rng.standard_normal((d, f)) * 0.05).astype(np.float32)) for _ in range(experts)])
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((tokens, d)).astype(np.float32))
    r16 = oracle.f32_to_f16_bits(rng.standard_normal((tokens, d)).astype(np.float32))
    lg = rng.standard_normal((tokens, experts)).astype(np.float32)
    ids, w16 = oracle.moe_route(lg, k)
    want = oracle.f16_bits_to_f32(oracle.moe_ffn(kind, gu, dn, experts, d, f, x16, r16, ids, w16, threads=8))
    y = ctx.alloc(tokens * d * 2)
    ctx.moe_ffn(kind, ctx.upload_weights(gu), ctx.upload_weights(dn), experts, d, f, ctx.to_device(x16), ctx.to_device(r16),
                ctx.to_device(ids), ctx.to_device(w16), tokens, k, y)
    ctx.sync()
    got = oracle.f16_bits_to_f32(y.download(np.uint16, tokens * d).reshape(tokens, d))
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    assert np.all(err <= ABS + REL * np.abs(want)), float(err.max())


def test_routed_feed_forward_flags_an_expert_id_outside_the_table(ctx, oracle):
    import turbospark_b200 as tsb
    d, f, experts = 256, 256, 4
    rng = np.random.default_rng(1)
    gu = np.concatenate([oracle.quantize(0, (rng.standard_normal((2 * f, d)) * 0.05).astype(np.float32)) for _ in range(experts)])
    dn = np.concatenate([oracle.quantize(0, (rng.standard_normal((d, f)) * 0.05).astype(np.float32)) for _ in range(experts)])
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((2, d)).astype(np.float32))
    ids = np.array([[0, 9], [1, 2]], dtype=np.int32)
    w16 = oracle.f32_to_f16_bits(np.full((2, 2), 0.5, np.float32))
    y = ctx.alloc(2 * d * 2)
    ctx.moe_ffn(0, ctx.upload_weights(gu), ctx.upload_weights(dn), experts, d, f, ctx.to_device(x16), ctx.to_device(x16),
                ctx.to_device(ids), ctx.to_device(w16), 2, 2, y)
    with pytest.raises(tsb.TsbError):
        ctx.sync()


def test_router_logits_match_the_oracle(ctx, oracle):
    import turbospark_b200 as tsb
    cfg = tsb.config_tiny()
    moe = weights.random_moe_weights(cfg, 8, 256, 3, oracle)
    q, sc, bi, _, _ = moe[0]
    rng = np.random.default_rng(4)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((5, cfg.d_model)).astype(np.float32))
    want = oracle.router_logits(q, sc, bi, x16, 8)
    out = ctx.alloc(5 * 8 * 4)
    ctx.router_logits(ctx.to_device(q), ctx.to_device(sc), ctx.to_device(bi), ctx.to_device(x16), 5, 8, cfg.d_model, out)
    ctx.sync()
    got = out.download(np.float32, 40).reshape(5, 8)
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-5), float(np.abs(got - want).max())


def test_a_model_with_a_routed_feed_forward_matches_the_oracle_forward(oracle):
    """4-layer decoder whose feed-forward is 8 MXFP4 experts, top-2 (the MoE configuration's layer, small):
    token-by-token decode, a 6-row verify that equals the single-row steps bit for bit, a speculative run that
    equals the sequential one, all against the oracle's forward over the same bytes."""
    import turbospark_b200 as tsb
    E, K, F = 8, 2, 256
    ctx = tsb.Ctx(0)
    cfg = tsb.config_tiny(max_context=256)
    mats, norms = weights.random_weights(cfg, 7, oracle, real_ffn=1408)
    moe = weights.random_moe_weights(cfg, E, F, 8, oracle)
    target = tsb.Model(ctx, cfg)
    target.set_moe(E, K, F)
    weights.load_weights(target, mats, norms, skip=weights.DENSE_FFN)
    weights.load_moe_weights(target, moe)
    ocfg = oracle.ModelCfg(cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                           cfg.max_context, cfg.rms_eps, cfg.rope_theta)
    ot = oracle.Model(ocfg, threads=8)
    ot.set_moe(E, K, F)
    weights.load_weights(ot, mats, norms, skip=weights.DENSE_FFN)
    weights.load_moe_weights(ot, moe)
    sess = tsb.Session(ctx, target, None, 1, 8)
    ost = oracle.State(ot)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab, size=8).astype(np.int32)

    def close(got16, want16):
        got, want = oracle.f16_bits_to_f32(got16), oracle.f16_bits_to_f32(want16)
        assert not np.isnan(got).any()
        # the routed layer adds rounding points (f16 routing weights, the f16 routed sum, its add onto the stream):
        # the reference's own bound for chained f16 reductions (compute/src/tolerance.rs:70-83, 1e-2) applies;
        # the observed error is 0.2-0.4 % rms of the logit scale
        err = np.abs(got - want)
        assert np.all(err <= 1e-2 + 1e-2 * np.abs(want)), float(err.max())
        assert np.sqrt((err ** 2).mean()) <= 4e-3 * np.sqrt((want ** 2).mean())

    for i, t in enumerate(prompt):
        close(sess.produce(int(t), i), ost.forward([int(t)], i)[0])
    feed = rng.integers(0, cfg.vocab, size=6).astype(np.int32)
    point = sess.checkpoint()
    batch = sess.verify(feed, point)
    sess.rollback_retaining(point, 0)
    single = np.stack([sess.produce(int(t), point + i) for i, t in enumerate(feed)])
    assert np.array_equal(batch, single)
    close(batch, ost.forward(feed, point))
    sess.close()
    # the round loop over a routed target with a routed 2-layer drafter sharing its trunk
    dcfg = tsb.ModelConfig(2, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.max_context,
                           cfg.rms_eps, cfg.rope_theta)
    draft = tsb.Model(ctx, dcfg)
    draft.set_moe(E, K, F)
    for l in range(2):
        draft.share(l, target, l)
    draft.share(-1, target, -1)
    sess = tsb.Session(ctx, target, draft, 1, 16)
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 24, 4)
    seq_hist, seq_emit, _ = sess.sequential_run(prompt, rc)
    spec_hist, spec_emit, res = sess.spec_run(prompt, rc)
    assert np.array_equal(seq_emit, spec_emit) and res.new_tokens == 24
    sess.close(), draft.close(), target.close(), ctx.close()
