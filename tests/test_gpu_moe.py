"""Mixture-of-experts routing and routed feed-forward on the GPU against the oracle's restatement of
router_topk_gemma4 and the two MoE kernels (crates/gpu/src/shaders/moe_gguf.metal:561-678)."""
import numpy as np
import pytest

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
