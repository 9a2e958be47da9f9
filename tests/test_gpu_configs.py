"""The operator shapes, token counts, context lengths and batch sizes the benchmark configurations name,
against the CPU oracle through the C ABI.

Weight matrices here are raw block bytes (random codes, scale fields set so the dequantised weights are
zero-mean with a standard deviation near 0.02): the oracle decodes the same bytes, so no quantiser runs.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL, ABS = 2e-3, 1e-3  # GEMV/GEMM and attention with fp32 accumulation


@pytest.fixture(scope="module")
def ctx():
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    yield c
    c.close()


def raw_blocks(kind, rows, cols, seed):
    """[rows, row_bytes] uint8 of valid Q4_K (kind 0) or MXFP4 (kind 2) blocks."""
    rng = np.random.default_rng(seed)
    if kind == 0:
        nb = rows * cols // 256
        b = rng.integers(0, 256, size=(nb, 144), dtype=np.uint8)
        d = (7.7e-5 * (0.5 + rng.random(nb))).astype(np.float16)
        b[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        b[:, 2:4] = (d.astype(np.float32) * 7.5).astype(np.float16).view(np.uint8).reshape(nb, 2)
        return b.reshape(rows, -1)
    if kind == 2:
        nb = rows * cols // 32
        b = rng.integers(0, 256, size=(nb, 17), dtype=np.uint8)
        b[:, 0] = 119 + (b[:, 0] & 1)
        return b.reshape(rows, -1)
    raise ValueError(kind)


def _check(got, want):
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    tol = ABS + REL * np.abs(want)
    assert np.all(err <= tol), "max err %g at %s (want %g)" % (err.max(), np.unravel_index(err.argmax(), err.shape),
                                                                 want.flat[err.argmax()])


TOKEN_COUNTS = (1, 2, 4, 8, 16, 32, 64)


@pytest.mark.parametrize("kind", [0, 2])
@pytest.mark.parametrize("rows,cols", [(14336, 4096), (4096, 14336)])
def test_sweep_shapes_match_the_oracle_at_every_token_count(ctx, oracle, kind, rows, cols):
    q = raw_blocks(kind, rows, cols, rows + kind)
    rng = np.random.default_rng(cols)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((64, cols)).astype(np.float32))
    want = oracle.gemm_quant(kind, q, rows, cols, oracle.f16_bits_to_f32(x16), threads=8)  # rows are independent
    w = ctx.upload_weights(q)
    yd = ctx.alloc(64 * rows * 4)
    for tokens in TOKEN_COUNTS:
        xd = ctx.to_device(x16[:tokens])
        ctx.gemm_quant(kind, w, rows, cols, xd, yd, tokens, y_f32=True)
        ctx.sync()
        got = yd.download(np.float32, tokens * rows).reshape(tokens, rows)
        _check(got, want[:tokens])


@pytest.mark.parametrize("kind", [0, 2])
def test_head_shape_matches_the_oracle_on_a_row_sample(ctx, oracle, kind):
    # 128256 x 4096: the persistent CTAs walk more tiles than they are; the oracle checks the first and last
    # tiles and every 29th row between them
    rows, cols = 128256, 4096
    q = raw_blocks(kind, rows, cols, 77 + kind)
    pick = np.unique(np.concatenate([np.arange(0, 160), np.arange(rows - 160, rows), np.arange(0, rows, 29)]))
    assert pick.size >= 4096
    rng = np.random.default_rng(5)
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((64, cols)).astype(np.float32))
    want = oracle.gemm_quant(kind, q[pick], pick.size, cols, oracle.f16_bits_to_f32(x16), threads=8)
    w = ctx.upload_weights(q)
    yd = ctx.alloc(64 * rows * 4)
    for tokens in TOKEN_COUNTS:
        xd = ctx.to_device(x16[:tokens])
        ctx.gemm_quant(kind, w, rows, cols, xd, yd, tokens, y_f32=True)
        ctx.sync()
        got = yd.download(np.float32, tokens * rows).reshape(tokens, rows)
        _check(got[:, pick], want[:tokens])


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("tokens", [9, 16, 17, 23, 24, 40, 64])
def test_token_counts_between_the_tile_widths_match_the_oracle(ctx, oracle, kind, tokens):
    # two and three token tiles of the register path (9..23), and above 23 the formats that never take tcgen05
    rows, cols = 144, 2048
    rng = np.random.default_rng(100 * kind + tokens)
    q = oracle.quantize(kind, (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((tokens, cols)).astype(np.float32))
    want = oracle.gemm_quant(kind, q, rows, cols, oracle.f16_bits_to_f32(x16), threads=4)
    w = ctx.upload_weights(q)
    xd = ctx.to_device(x16)
    yd = ctx.alloc(tokens * rows * 4)
    ctx.gemm_quant(kind, w, rows, cols, xd, yd, tokens, y_f32=True)
    ctx.sync()
    _check(yd.download(np.float32, tokens * rows).reshape(tokens, rows), want)


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_every_row_of_a_batch_equals_the_single_row_call(ctx, oracle, kind):
    # rows = 96 keeps Q4_K on the register path at every width, so all widths share one arithmetic
    rows, cols = 96, 4096
    rng = np.random.default_rng(11 + kind)
    q = oracle.quantize(kind, (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((64, cols)).astype(np.float32))
    w = ctx.upload_weights(q)
    yd = ctx.alloc(64 * rows * 4)
    single = np.empty((64, rows), dtype=np.uint32)
    for t in range(64):
        ctx.gemm_quant(kind, w, rows, cols, ctx.to_device(x16[t]), yd, 1, y_f32=True)
        ctx.sync()
        single[t] = yd.download(np.uint32, rows)
    for width in (2, 6, 8, 9, 16, 17, 23, 33, 64):
        ctx.gemm_quant(kind, w, rows, cols, ctx.to_device(x16[:width]), yd, width, y_f32=True)
        ctx.sync()
        got = yd.download(np.uint32, width * rows).reshape(width, rows)
        assert np.array_equal(got, single[:width]), width


def _attend(ctx, kv, layer, q16, entries, rows_per_seq, nq, hd, max_len):
    import turbospark_b200 as tsb
    rows = len(entries)
    qd = ctx.to_device(q16)
    out = ctx.alloc(rows * nq * hd * 2)
    rd = ctx.to_device(tsb.row_descs(entries))
    scratch = ctx.alloc(ctx.attn_scratch_bytes(rows, nq, hd))
    ctx.attn_decode_rows(kv, layer, qd, nq * hd, out, rd, rows, rows_per_seq, nq, 1.0 / np.sqrt(hd), max_len, scratch)
    ctx.sync()
    return out.download(np.uint16, rows * nq * hd).reshape(rows, nq * hd)


def _kv(ctx, oracle, nkv, hd, ctx_len, seed):
    import turbospark_b200 as tsb
    pages = (ctx_len + 63) // 64 + 1
    kv = tsb.KvCache(ctx, 1, nkv, hd, 64, pages + 2, 1, pages)
    kv.reserve(0, ctx_len)
    rng = np.random.default_rng(seed)
    k = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
    v = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
    kv.write_rows(0, 0, 0, k, v)
    return kv, oracle.f16_bits_to_f32(k), oracle.f16_bits_to_f32(v)


@pytest.mark.parametrize("base", [8190, 32762])
def test_chain_rows_at_long_contexts_match_the_oracle(ctx, oracle, base):
    hd, nq, nkv, rows = 128, 32, 8, 6
    ctx_len = base + rows
    kv, kf, vf = _kv(ctx, oracle, nkv, hd, ctx_len, base)
    rng = np.random.default_rng(base + 1)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((rows, nq * hd)).astype(np.float32))
    entries = [(0, base, m, base + m, (1 << (m + 1)) - 1) for m in range(rows)]
    got = oracle.f16_bits_to_f32(_attend(ctx, kv, 0, q16, entries, rows, nq, hd, ctx_len))
    for m in range(rows):
        want = oracle.causal_attention(oracle.f16_bits_to_f32(q16[m]), kf[:base + m + 1], vf[:base + m + 1], hd, nq, nkv,
                                       base + m + 1, 1.0 / np.sqrt(hd))
        _check(got[m], want)
    kv.close()


def static_tree(branching, nodes):
    """Parent of every node of a level-by-level tree (node 0 = the anchor row) cut at `nodes` drafted nodes."""
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


@pytest.mark.parametrize("base", [2000, 8127])
def test_a_65_row_tree_matches_indexed_attention(ctx, oracle, base):
    # the anchor plus 64 drafted nodes, branching 4,4,2,1,1,1 cut at 64: masks reach into the second 64-bit word
    hd, nq, nkv = 128, 32, 8
    parent = static_tree((4, 4, 2, 1, 1, 1), 64)
    n = len(parent)
    assert n == 65
    paths, depth = [], []
    for s in range(n):
        p, cur = [], s
        while cur >= 0:
            p.append(cur)
            cur = parent[cur]
        paths.append(p[::-1])
        depth.append(len(p) - 1)
    ctx_len = base + n
    kv, kf, vf = _kv(ctx, oracle, nkv, hd, ctx_len, base + 3)
    rng = np.random.default_rng(base)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((n, nq * hd)).astype(np.float32))
    entries = [(0, base, s, base + depth[s], sum(1 << j for j in paths[s])) for s in range(n)]
    got = oracle.f16_bits_to_f32(_attend(ctx, kv, 0, q16, entries, n, nq, hd, ctx_len))
    for s in list(range(0, n, 5)) + [n - 1]:
        pos = list(range(base)) + [base + j for j in paths[s]]
        want = oracle.indexed_attention(oracle.f16_bits_to_f32(q16[s]), kf, vf, pos, hd, nq, nkv, 1.0 / np.sqrt(hd))
        _check(got[s], want)
    kv.close()


def test_acceptance_over_256_streams_at_the_full_vocabulary(ctx, oracle):
    import turbospark_b200 as tsb
    batch, k, vocab = 256, 5, 128256
    rng = np.random.default_rng(9)
    # target logits N(0, 3), draft = target + N(0, 1): one stream's rows generated, the others permute it
    base_t = (rng.standard_normal((k + 1, vocab)) * 3.0).astype(np.float32)
    base_d = base_t[:k] + rng.standard_normal((k, vocab)).astype(np.float32)
    t16 = np.empty((batch, k + 1, vocab), dtype=np.uint16)
    d16 = np.empty((batch, k, vocab), dtype=np.uint16)
    bt, bd = oracle.f32_to_f16_bits(base_t), oracle.f32_to_f16_bits(base_d)
    for b in range(batch):
        t16[b] = np.roll(bt, 37 * b, axis=1)
        d16[b] = np.roll(bd, 37 * b, axis=1)
    ocfg = oracle.shaping(temperature=1.0, seed=4)
    check = list(range(0, batch, 8))  # the oracle runs on every eighth stream
    props = np.empty((batch, k), dtype=np.int32)
    unis = np.empty((batch, 2 * k + 1), dtype=np.uint64)
    for b in range(batch):
        for j in range(2 * k + 1):
            unis[b, j] = oracle.uniform_u64(1, 4, 7000 + 100 * b + j)
    # proposals: drawn from q on the checked streams (as the loop does), the rolled copy of stream 0's elsewhere
    p0 = [oracle.sample(d16[0, i], ocfg, oracle.uniform_u64(1, 4, i))[0] for i in range(k)]
    for b in range(batch):
        for i in range(k):
            props[b, i] = (p0[i] + 37 * b) % vocab
    cfg = tsb.shaping(temperature=1.0, seed=4)
    out = ctx.alloc(batch * C.sizeof(tsb.AcceptOut))
    scratch = ctx.alloc(ctx.accept_scratch_bytes(batch, k, vocab))
    ctx.accept(ctx.to_device(t16), ctx.to_device(d16), ctx.to_device(props), ctx.to_device(unis), batch, k, vocab, cfg, out, scratch)
    ctx.sync()
    raw = out.download(np.uint8, batch * C.sizeof(tsb.AcceptOut))
    sz = C.sizeof(tsb.AcceptOut)
    outs = [tsb.AcceptOut.from_buffer_copy(raw[i * sz:(i + 1) * sz].tobytes()) for i in range(batch)]
    assert all(o.status == 0 for o in outs)
    rejected = 0
    for b in check:
        acc, toks, draws, margins = oracle.accept_round(t16[b], d16[b], props[b], ocfg, unis[b])
        o = outs[b]
        assert o.accepted == acc and list(o.tokens[:acc + 1]) == list(toks) and o.draws == draws, b
        rejected += acc < k
    assert rejected > 0
