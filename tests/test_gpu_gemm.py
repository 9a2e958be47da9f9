"""Quantized matmul and row operators on the GPU against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# north-star tolerance for GEMV/GEMM with fp32 accumulation
REL, ABS = 2e-3, 1e-3


@pytest.fixture(scope="module")
def ctx():
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    yield c
    c.close()


def _weights(oracle, kind, rows, cols, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    return oracle.quantize(kind, w)


def _check(got, want):
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    tol = ABS + REL * np.abs(want)
    assert np.all(err <= tol), "max err %g at %s (want %g)" % (err.max(), np.unravel_index(err.argmax(), err.shape),
                                                                 want.flat[err.argmax()])


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("rows,cols,tokens", [(64, 512, 1), (48, 2048, 6), (40, 4096, 3), (16, 14336, 6), (100, 1536, 8)])
def test_gemm_matches_oracle(ctx, oracle, kind, rows, cols, tokens):
    q = _weights(oracle, kind, rows, cols, 3)
    rng = np.random.default_rng(7)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((tokens, cols)).astype(np.float32))
    want = oracle.gemm_quant(kind, q, rows, cols, oracle.f16_bits_to_f32(x16), threads=8)
    w = ctx.upload_weights(q)
    xd = ctx.to_device(x16)
    yd = ctx.alloc(tokens * rows * 4)
    ctx.gemm_quant(kind, w, rows, cols, xd, yd, tokens, y_f32=True)
    got = yd.download(np.float32, tokens * rows).reshape(tokens, rows)
    _check(got, want)
    # f16 output is the same sums rounded once
    yh = ctx.alloc(tokens * rows * 2)
    ctx.gemm_quant(kind, w, rows, cols, xd, yh, tokens, y_f32=False)
    got16 = yh.download(np.uint16, tokens * rows).reshape(tokens, rows)
    assert np.array_equal(got16, oracle.f32_to_f16_bits(got))


@pytest.mark.parametrize("rows,cols,tokens", [(128, 256, 24), (256, 2048, 40), (1024, 4096, 64), (384, 1536, 100), (128, 14336, 33),
                                              (19200, 512, 130), (640, 2048, 300)])
def test_many_token_rows_take_the_tensor_memory_path_and_match_the_oracle(ctx, oracle, rows, cols, tokens):
    """24 token rows and more of a Q4_K matrix whose rows are a multiple of 128 run on tcgen05 with the dequantised
    operand in tensor memory; q*sc is exact in f16 and d, dmin are applied in fp32, so the sums match as closely as
    the few-row path's."""
    q = _weights(oracle, 0, rows, cols, 5)
    rng = np.random.default_rng(tokens)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((tokens, cols)).astype(np.float32))
    want = oracle.gemm_quant(0, q, rows, cols, oracle.f16_bits_to_f32(x16), threads=8)
    w = ctx.upload_weights(q)
    xd = ctx.to_device(x16)
    yd = ctx.alloc(tokens * rows * 4)
    ctx.gemm_quant(0, w, rows, cols, xd, yd, tokens, y_f32=True)
    ctx.sync()
    got = yd.download(np.float32, tokens * rows).reshape(tokens, rows)
    _check(got, want)
    yh = ctx.alloc(tokens * rows * 2)
    ctx.gemm_quant(0, w, rows, cols, xd, yh, tokens, y_f32=False)
    ctx.sync()
    assert np.array_equal(yh.download(np.uint16, tokens * rows).reshape(tokens, rows), oracle.f32_to_f16_bits(got))
    # a token's row does not depend on its batch mates: the first 24 rows alone give the same bits
    y2 = ctx.alloc(24 * rows * 4)
    ctx.gemm_quant(0, w, rows, cols, xd, y2, 24, y_f32=True)
    ctx.sync()
    assert np.array_equal(y2.download(np.float32, 24 * rows).reshape(24, rows), got[:24])


@pytest.mark.parametrize("kind,rows,cols,tokens", [(0, 48, 2048, 6), (2, 100, 1536, 8), (1, 64, 512, 1), (0, 256, 2048, 40), (4, 40, 4096, 17)])
def test_the_matmul_over_a_caller_workspace_gives_the_one_call_operators_bits(ctx, oracle, kind, rows, cols, tokens):
    """tsb_gemm_prepare + tsb_gemm_quant_prepared (no allocation, the operand converted once and reused over two
    matrices) against tsb_gemm_quant; a short workspace and a misaligned one are refused."""
    import turbospark_b200 as tsb
    qa, qb = _weights(oracle, kind, rows, cols, 3), _weights(oracle, kind, rows, cols, 4)
    rng = np.random.default_rng(11)
    xd = ctx.to_device(oracle.f32_to_f16_bits(rng.standard_normal((tokens, cols)).astype(np.float32)))
    need = ctx.gemm_workspace_bytes(kind, rows, cols, tokens)
    assert need > 0 and ctx.gemm_workspace_bytes(kind, rows, cols + 32, tokens) == 0
    work = ctx.alloc(need)
    ctx.gemm_prepare(kind, rows, cols, xd, tokens, work)
    for q in (qa, qb):
        w = ctx.upload_weights(q)
        y1, y2 = ctx.alloc(tokens * rows * 4), ctx.alloc(tokens * rows * 4)
        ctx.gemm_quant(kind, w, rows, cols, xd, y1, tokens, y_f32=True)
        ctx.gemm_quant_prepared(kind, w, rows, cols, xd, work, y2, tokens, y_f32=True)
        ctx.sync()
        assert np.array_equal(y1.download(np.uint32, tokens * rows), y2.download(np.uint32, tokens * rows))
    short = ctx.alloc(need - 256)
    with pytest.raises(tsb.TsbError):
        ctx.gemm_prepare(kind, rows, cols, xd, tokens, short)


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_a_tokens_result_does_not_depend_on_the_batch(ctx, oracle, kind):
    # the verify batch must reproduce the decode step bit for bit, at every width
    rows, cols = 96, 4096
    q = _weights(oracle, kind, rows, cols, 5)
    rng = np.random.default_rng(11)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((64, cols)).astype(np.float32))
    w = ctx.upload_weights(q)
    single = []
    yd = ctx.alloc(64 * rows * 4)
    for t in range(8):
        xd = ctx.to_device(x16[t])
        ctx.gemm_quant(kind, w, rows, cols, xd, yd, 1, y_f32=True)
        single.append(yd.download(np.uint32, rows))
    for width in (2, 3, 6, 8, 9, 16, 17, 33, 64):
        xd = ctx.to_device(x16[:width])
        ctx.gemm_quant(kind, w, rows, cols, xd, yd, width, y_f32=True)
        got = yd.download(np.uint32, width * rows).reshape(width, rows)
        for t in range(min(width, 8)):
            assert np.array_equal(got[t], single[t]), (width, t)


def test_q4k_finite_but_wrong_cases(ctx, oracle):
    # split 6-bit scales, the min carries the sign, per-superblock scales differ, offset != 0
    rows, cols = 32, 1024
    rng = np.random.default_rng(23)
    factors = np.array([1.0, 0.5, 4.0, 2.0, 0.5, 8.0, 1.0, 2.0], dtype=np.float32)
    w = rng.standard_normal((rows, cols)).astype(np.float32) * 0.05
    w = w * np.repeat(np.tile(factors, cols // 256), 32)[None, :]
    w[:, 256:512] = -np.abs(w[:, 256:512]) - 0.1  # all negative: the min term alone makes it negative
    w[:, 512:768] *= 7.0                          # a superblock with a very different d
    q = oracle.quantize(0, w)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((2, cols)).astype(np.float32))
    want = oracle.gemm_quant(0, q, rows, cols, oracle.f16_bits_to_f32(x16))
    pad = np.zeros(144 * 5, dtype=np.uint8)
    region = ctx.upload_weights(np.concatenate([pad, q.reshape(-1)]))
    xd = ctx.to_device(x16)
    yd = ctx.alloc(2 * rows * 4)
    ctx.gemm_quant(0, region, rows, cols, xd, yd, 2, y_f32=True, w_off=pad.size)
    _check(yd.download(np.float32, 2 * rows).reshape(2, rows), want)


def test_gemm_refuses_bad_shapes(ctx, oracle):
    import turbospark_b200 as tsb
    q = _weights(oracle, 0, 16, 256, 1)
    w = ctx.upload_weights(q)
    xd = ctx.alloc(4096)
    yd = ctx.alloc(4096)
    with pytest.raises(tsb.TsbError):
        ctx.gemm_quant(0, w, 16, 200, xd, yd, 1)
    with pytest.raises(tsb.TsbError):
        ctx.gemm_quant(7, w, 16, 256, xd, yd, 1)
    with pytest.raises(tsb.TsbError):
        ctx.gemm_quant(0, w, 16, 256, xd, yd, 0)


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_dequant_rows_is_bit_exact(ctx, oracle, kind):
    rows, cols = 24, 1024
    q = _weights(oracle, kind, rows, cols, 9)
    w = ctx.upload_weights(q)
    ids = np.array([3, 0, 23, 7, 7], dtype=np.int32)
    idd = ctx.to_device(ids)
    out = ctx.alloc(ids.size * cols * 4)
    ctx.dequant_rows(kind, w, cols, idd, ids.size, out)
    got = out.download(np.uint32, ids.size * cols).reshape(ids.size, cols)
    for i, r in enumerate(ids):
        want = oracle.dequantize(kind, q[r], cols)
        assert np.array_equal(got[i], want.view(np.uint32)), (kind, r)


def test_q5k_dequant_matches_ggml_golden_on_device(ctx, oracle):
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "q5k_ggml.json")))
    w = ctx.upload_weights(np.array(g["bytes"], dtype=np.uint8))
    out = ctx.alloc(512 * 4)
    ctx.dequant_rows(3, w, 512, None, 1, out)
    assert np.array_equal(out.download(np.uint32, 512), np.array(g["floats"], dtype=np.float32).view(np.uint32))
    # and the matmul over the same two superblocks against the decoded floats
    rng = np.random.default_rng(2)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((3, 512)).astype(np.float32))
    want = oracle.f16_bits_to_f32(x16) @ np.array(g["floats"], dtype=np.float32)
    rows16 = ctx.upload_weights(np.tile(np.array(g["bytes"], dtype=np.uint8), 16))
    yd = ctx.alloc(3 * 16 * 4)
    ctx.gemm_quant(3, rows16, 16, 512, ctx.to_device(x16), yd, 3, y_f32=True)
    got = yd.download(np.float32, 48).reshape(3, 16)
    _check(got, np.repeat(want[:, None], 16, axis=1))


def test_mxfp4_dequant_matches_ggml_golden_on_device(ctx, oracle):
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "mxfp4_ggml.json")))
    w = ctx.upload_weights(np.array(g["bytes"], dtype=np.uint8))
    out = ctx.alloc(128 * 4)
    ctx.dequant_rows(2, w, 128, None, 1, out)
    got = out.download(np.uint32, 128)
    assert np.array_equal(got, np.array(g["floats"], dtype=np.float32).view(np.uint32))
    # every shared exponent, through a one-block row whose first code is 1
    blocks = np.zeros((256, 17), dtype=np.uint8)
    blocks[:, 0] = np.arange(256)
    blocks[:, 1] = 1
    w = ctx.upload_weights(blocks.reshape(-1))
    out = ctx.alloc(256 * 32 * 4)
    ctx.dequant_rows(2, w, 32, None, 256, out)
    got = out.download(np.float32, 256 * 32).reshape(256, 32)[:, 0]
    assert np.array_equal(got.view(np.uint32), np.array(g["e8m0"], dtype=np.float32).view(np.uint32))


def test_q4k_hand_packed_superblock_on_device(ctx, oracle):
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "q4k_handpacked.json")))
    quants = [(e * 7 + 3) % 16 for e in range(256)]
    block = bytearray(g["d_bits"] + g["dmin_bits"] + g["packed"])
    for grp in range(4):
        for l in range(32):
            block.append(quants[grp * 64 + l] | (quants[grp * 64 + l + 32] << 4))
    w = ctx.upload_weights(np.frombuffer(bytes(block), dtype=np.uint8))
    out = ctx.alloc(256 * 4)
    ctx.dequant_rows(0, w, 256, None, 1, out)
    got = out.download(np.float32, 256)
    for e in range(256):
        j = e // 32
        assert got[e] == np.float32(0.5) * np.float32(g["ls"][j]) * np.float32(quants[e]) - np.float32(0.25) * np.float32(g["lm"][j])
    # and through the matmul: x = one-hot picks single weights out exactly
    x = np.zeros((8, 256), dtype=np.float32)
    for t in range(8):
        x[t, t * 37 % 256] = 1.0
    xd = ctx.to_device(oracle.f32_to_f16_bits(x))
    yd = ctx.alloc(8 * 4)
    ctx.gemm_quant(0, w, 1, 256, xd, yd, 8, y_f32=True)
    y = yd.download(np.float32, 8)
    for t in range(8):
        assert y[t] == got[t * 37 % 256]


def test_q6k_hand_packed_superblock_on_device(ctx, oracle):
    import json, os
    from tests.test_oracle_quant import q6k_hand_packed_block
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "q6k_handpacked.json")))
    block, want = q6k_hand_packed_block(g)
    w = ctx.upload_weights(block)
    out = ctx.alloc(256 * 4)
    ctx.dequant_rows(1, w, 256, None, 1, out)
    got = out.download(np.float32, 256)
    assert np.array_equal(got, want)
    # through the matmul: one-hot activations pick single weights out exactly
    x = np.zeros((8, 256), dtype=np.float32)
    for t in range(8):
        x[t, (t * 37 + 5) % 256] = 1.0
    xd = ctx.to_device(oracle.f32_to_f16_bits(x))
    yd = ctx.alloc(8 * 4)
    ctx.gemm_quant(1, w, 1, 256, xd, yd, 8, y_f32=True)
    y = yd.download(np.float32, 8)
    for t in range(8):
        assert y[t] == want[(t * 37 + 5) % 256]


def test_embed_rows(ctx, oracle):
    vocab, d = 50, 512
    q = _weights(oracle, 0, vocab, d, 2)
    w = ctx.upload_weights(q)
    ids = np.array([49, 1, 0, 17], dtype=np.int32)
    out = ctx.alloc(ids.size * d * 2)
    ctx.embed_rows(0, w, vocab, d, ctx.to_device(ids), ids.size, out)
    got = out.download(np.uint16, ids.size * d).reshape(ids.size, d)
    for i, r in enumerate(ids):
        assert np.array_equal(got[i], oracle.f32_to_f16_bits(oracle.dequantize(0, q[r], d)))


def test_rmsnorm_rope_silu_residual(ctx, oracle):
    rng = np.random.default_rng(5)
    rows, d = 6, 4096
    x = oracle.f32_to_f16_bits(rng.standard_normal((rows, d)).astype(np.float32))
    res = oracle.f32_to_f16_bits(rng.standard_normal((rows, d)).astype(np.float32) * 0.1)
    wbf = np.array([oracle.lib().tso_f32_to_bf16(float(v)) for v in 1.0 + 0.1 * rng.standard_normal(d)], dtype=np.uint16)
    wf = np.array([oracle.lib().tso_bf16_to_f32(int(b)) for b in wbf], dtype=np.float32)
    xd, rd, wd, od = ctx.to_device(x), ctx.to_device(res), ctx.to_device(wbf), ctx.alloc(rows * d * 2)
    ctx.rmsnorm_rows(xd, rd, wd, od, rows, d, 1e-6)
    summed = oracle.f32_to_f16_bits(oracle.f16_bits_to_f32(x) + oracle.f16_bits_to_f32(res))
    assert np.array_equal(xd.download(np.uint16, rows * d).reshape(rows, d), summed)
    got = oracle.f16_bits_to_f32(od.download(np.uint16, rows * d).reshape(rows, d))
    for r in range(rows):
        want = oracle.rms_norm(oracle.f16_bits_to_f32(summed[r]), wf, 1e-6)
        assert np.all(np.abs(got[r] - want) <= 1e-3 * np.abs(want) + 1e-4)

    heads, hd = 8, 128
    q = oracle.f32_to_f16_bits(rng.standard_normal((rows, heads * hd)).astype(np.float32))
    pos = np.array([0, 1, 17, 4095, 4096, 32767], dtype=np.int32)
    qd = ctx.to_device(q)
    ctx.rope_rows(qd, rows, heads, hd, hd // 2, heads * hd, ctx.to_device(pos), 10000.0)
    got = qd.download(np.uint16, rows * heads * hd).reshape(rows, heads * hd)
    mism = 0
    for r in range(rows):
        want = oracle.f32_to_f16_bits(oracle.rope_neox(oracle.f16_bits_to_f32(q[r]), 1, heads, hd, hd // 2, int(pos[r]), 10000.0))
        mism += int((got[r] != want).sum())
        assert np.all(np.abs(oracle.f16_bits_to_f32(got[r]) - oracle.f16_bits_to_f32(want)) <= 2e-3)
    assert mism <= 4, mism  # double-rounded libm calls reproduce the f32 reference almost everywhere

    n = 1536
    g = oracle.f32_to_f16_bits(rng.standard_normal((rows, n)).astype(np.float32) * 3)
    u = oracle.f32_to_f16_bits(rng.standard_normal((rows, n)).astype(np.float32))
    out = ctx.alloc(rows * n * 2)
    ctx.silu_mul(ctx.to_device(g), ctx.to_device(u), out, rows, n, n, n)
    want = oracle.f32_to_f16_bits(oracle.silu_mul(oracle.f16_bits_to_f32(g), oracle.f16_bits_to_f32(u)))
    got = out.download(np.uint16, rows * n).reshape(rows, n)
    assert (got != want).sum() <= 2

    a = ctx.to_device(x)
    ctx.residual_add(a, ctx.to_device(res), rows * d)
    assert np.array_equal(a.download(np.uint16, rows * d).reshape(rows, d), summed)


def test_a_wait_nobody_answers_gives_up_reports_and_leaves_the_context_usable(oracle):
    """Every device-side wait is bounded by time.  A barrier nobody arrives on makes the bound run out: the kernel
    returns, the next synchronisation reports the device error word, and the same context still computes."""
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    try:
        c.set_wait_limit_us(2000)
        flag = c.to_device(np.array([7], dtype=np.uint32))
        c.debug_wait_nobody(flag)
        with pytest.raises(tsb.TsbError) as ei:
            c.sync()
        assert "wait gave up" in str(ei.value)
        assert flag.download(np.uint32, 1)[0] == 0  # the wait did not claim success
        c.set_wait_limit_us(1000000)
        rows, cols = 32, 4096
        q = _weights(oracle, 0, rows, cols, 1)
        x16 = oracle.f32_to_f16_bits(np.random.default_rng(1).standard_normal((2, cols)).astype(np.float32))
        yd = c.alloc(2 * rows * 4)
        c.gemm_quant(0, c.upload_weights(q), rows, cols, c.to_device(x16), yd, 2, y_f32=True)
        c.sync()
        _check(yd.download(np.float32, 2 * rows).reshape(2, rows),
               oracle.gemm_quant(0, q, rows, cols, oracle.f16_bits_to_f32(x16)))
    finally:
        c.close()
