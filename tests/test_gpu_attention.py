"""Paged KV cache, RoPE + store, split-KV attention with the tree mask, path compaction (GPU vs oracle)."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL, ABS = 2e-3, 1e-3  # north-star tolerance for attention with fp32 accumulation


@pytest.fixture(scope="module")
def ctx():
    import turbospark_b200 as tsb
    c = tsb.Ctx(0)
    yield c
    c.close()


def xorshift_values(oracle, seed, n):
    # crates/gpu/tests/attention_tree_parity.rs:27-37 value generator
    s = (seed | 1) & 0xFFFFFFFFFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        out[i] = ((s % 2000) / 1000.0 - 1.0) * 0.5
    return oracle.f32_to_f16_bits(out)


def _setup(ctx, oracle, layers, nkv, hd, ctx_len, seqs=1, page_tokens=64, seed=1):
    import turbospark_b200 as tsb
    pages_per_seq = (ctx_len + page_tokens - 1) // page_tokens + 1
    kv = tsb.KvCache(ctx, layers, nkv, hd, page_tokens, pages_per_seq * seqs + 2, seqs, pages_per_seq)
    rng = np.random.default_rng(seed)
    data = {}
    for s in range(seqs):
        kv.reserve(s, ctx_len)
        for l in range(layers):
            k = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
            v = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
            kv.write_rows(s, l, 0, k, v)
            data[(s, l)] = (k, v)
    return kv, data


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


def _close(oracle, got16, want):
    got = oracle.f16_bits_to_f32(got16)
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    assert np.all(err <= ABS + REL * np.abs(want)), err.max()


@pytest.mark.parametrize("hd,nq,nkv", [(128, 32, 8), (64, 8, 2), (128, 24, 4)])
@pytest.mark.parametrize("base,rows", [(0, 1), (1, 1), (15, 5), (63, 6), (64, 6), (257, 6), (1000, 6), (4090, 6)])
def test_chain_rows_match_the_oracle(ctx, oracle, hd, nq, nkv, base, rows):
    ctx_len = base + rows
    kv, data = _setup(ctx, oracle, 2, nkv, hd, ctx_len, seed=base + hd)
    k, v = data[(0, 1)]
    rng = np.random.default_rng(base)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((rows, nq * hd)).astype(np.float32))
    entries = [(0, base, m, base + m, (1 << (m + 1)) - 1) for m in range(rows)]
    got = _attend(ctx, kv, 1, q16, entries, rows, nq, hd, ctx_len)
    kf, vf = oracle.f16_bits_to_f32(k), oracle.f16_bits_to_f32(v)
    for m in range(rows):
        want = oracle.causal_attention(oracle.f16_bits_to_f32(q16[m]), kf[:base + m + 1], vf[:base + m + 1], hd, nq, nkv,
                                       base + m + 1, 1.0 / np.sqrt(hd))
        _close(oracle, got[m], want)
    kv.close()


@pytest.mark.parametrize("hd,nq,nkv,rows", [(128, 32, 8, 3), (64, 32, 8, 1)])
def test_many_streams_fill_the_device_and_match_the_oracle(ctx, oracle, hd, nq, nkv, rows):
    """48 streams x 8 kv heads are more CTAs than the device holds.  At head_dim 64 the context is then not cut and the
    one launch finishes the queries itself (no merge launch); at head_dim 128 such a pass takes the tensor-memory kernel.
    Streams of different lengths; a sample of them against the oracle."""
    seqs = 48
    lens = [150 + 37 * (s % 5) for s in range(seqs)]
    import turbospark_b200 as tsb
    page = 64
    pages_per = (max(lens) + rows) // page + 2
    kv = tsb.KvCache(ctx, 1, nkv, hd, page, pages_per * seqs + 2, seqs, pages_per)
    rng = np.random.default_rng(hd + rows)
    keep = {}
    for s in range(seqs):
        n = lens[s] + rows
        kv.reserve(s, n)
        k = oracle.f32_to_f16_bits(rng.standard_normal((n, nkv * hd)).astype(np.float32))
        v = oracle.f32_to_f16_bits(rng.standard_normal((n, nkv * hd)).astype(np.float32))
        kv.write_rows(s, 0, 0, k, v)
        if s % 11 == 0 or s == seqs - 1:
            keep[s] = (k, v)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((seqs * rows, nq * hd)).astype(np.float32))
    entries = [(s, lens[s], m, lens[s] + m, (1 << (m + 1)) - 1) for s in range(seqs) for m in range(rows)]
    got = _attend(ctx, kv, 0, q16, entries, rows, nq, hd, max(lens) + rows)
    for s, (k, v) in keep.items():
        kf, vf = oracle.f16_bits_to_f32(k), oracle.f16_bits_to_f32(v)
        for m in range(rows):
            n = lens[s] + m + 1
            want = oracle.causal_attention(oracle.f16_bits_to_f32(q16[s * rows + m]), kf[:n], vf[:n], hd, nq, nkv, n, 1.0 / np.sqrt(hd))
            _close(oracle, got[s * rows + m], want)
    kv.close()


def test_tree_rows_match_indexed_attention_and_identity_equals_chain(ctx, oracle):
    # crates/gpu/tests/attention_tree_parity.rs:136-206
    parent = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "tree_parent.json")))["parent"]
    depth, paths = oracle.tree_spec(parent)
    hd, nq, nkv = 128, 24, 4
    for base in (0, 3, 64, 300, 1023):
        n = len(parent)
        ctx_len = base + n
        import turbospark_b200 as tsb
        kv = tsb.KvCache(ctx, 1, nkv, hd, 64, ctx_len // 64 + 3, 1, ctx_len // 64 + 2)
        kv.reserve(0, ctx_len)
        k = xorshift_values(oracle, 11 + base, ctx_len * nkv * hd).reshape(ctx_len, -1)
        v = xorshift_values(oracle, 23 + base, ctx_len * nkv * hd).reshape(ctx_len, -1)
        kv.write_rows(0, 0, 0, k, v)
        q16 = xorshift_values(oracle, 5 + base, n * nq * hd).reshape(n, -1)
        masks = []
        for s in range(n):
            m = 0
            for i in range(depth[s] + 1):
                m |= 1 << int(paths[s][i])
            masks.append(m)
        entries = [(0, base, s, base + int(depth[s]), masks[s]) for s in range(n)]
        got = _attend(ctx, kv, 0, q16, entries, n, nq, hd, ctx_len)
        kf, vf = oracle.f16_bits_to_f32(k), oracle.f16_bits_to_f32(v)
        for s in range(n):
            pos = list(range(base)) + [base + int(p) for p in paths[s][:depth[s] + 1]]
            want = oracle.indexed_attention(oracle.f16_bits_to_f32(q16[s]), kf, vf, pos, hd, nq, nkv, 1.0 / np.sqrt(hd))
            _close(oracle, got[s], want)
        # identity paths (slots 0..4 form a chain 0-1-2-3-4) must equal the chain dispatch bit for bit
        chain_entries = [(0, base, s, base + s, (1 << (s + 1)) - 1) for s in range(5)]
        chain = _attend(ctx, kv, 0, q16[:5], chain_entries, 5, nq, hd, base + 5)
        tree5 = _attend(ctx, kv, 0, q16[:5], entries[:5], 5, nq, hd, base + 5)
        assert np.array_equal(chain, tree5)
        # a branching node differs from the chain row of the same depth (the mask matters)
        chain8 = _attend(ctx, kv, 0, q16, [(0, base, s, base + s, (1 << (s + 1)) - 1) for s in range(n)], n, nq, hd, ctx_len)
        for s in (5, 6, 7):
            assert not np.array_equal(chain8[s], got[s])
        kv.close()


def test_many_streams_with_different_lengths(ctx, oracle):
    import turbospark_b200 as tsb
    hd, nq, nkv, rows = 128, 32, 8, 6
    bases = [0, 70, 513, 129]
    kv = tsb.KvCache(ctx, 1, nkv, hd, 32, 80, len(bases), 20)
    rng = np.random.default_rng(3)
    ks, vs = [], []
    for s, b in enumerate(bases):
        kv.reserve(s, b + rows)
        k = oracle.f32_to_f16_bits(rng.standard_normal((b + rows, nkv * hd)).astype(np.float32))
        v = oracle.f32_to_f16_bits(rng.standard_normal((b + rows, nkv * hd)).astype(np.float32))
        kv.write_rows(s, 0, 0, k, v)
        ks.append(k), vs.append(v)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((len(bases) * rows, nq * hd)).astype(np.float32))
    entries = [(s, b, m, b + m, (1 << (m + 1)) - 1) for s, b in enumerate(bases) for m in range(rows)]
    got = _attend(ctx, kv, 0, q16, entries, rows, nq, hd, max(bases) + rows)
    for s, b in enumerate(bases):
        kf, vf = oracle.f16_bits_to_f32(ks[s]), oracle.f16_bits_to_f32(vs[s])
        for m in range(rows):
            want = oracle.causal_attention(oracle.f16_bits_to_f32(q16[s * rows + m]), kf[:b + m + 1], vf[:b + m + 1], hd, nq,
                                           nkv, b + m + 1, 1.0 / np.sqrt(hd))
            _close(oracle, got[s * rows + m], want)
    kv.close()


@pytest.mark.parametrize("rows", [17, 40, 128])
def test_many_rows_per_stream_take_the_tensor_memory_kernel_and_match_the_oracle(ctx, oracle, rows):
    """More than 64 queries per (stream, kv head) at head_dim 128 (17 rows x 4 heads and up): chain rows of streams of
    different lengths, one of them starting at position 0, pages of 32 tokens."""
    import turbospark_b200 as tsb
    hd, nq, nkv = 128, 32, 8
    bases = [0, 70, 513]
    kv = tsb.KvCache(ctx, 1, nkv, hd, 32, 80, len(bases), 24)
    rng = np.random.default_rng(rows)
    ks, vs = [], []
    for s, b in enumerate(bases):
        kv.reserve(s, b + rows)
        k = oracle.f32_to_f16_bits(rng.standard_normal((b + rows, nkv * hd)).astype(np.float32))
        v = oracle.f32_to_f16_bits(rng.standard_normal((b + rows, nkv * hd)).astype(np.float32))
        kv.write_rows(s, 0, 0, k, v)
        ks.append(k), vs.append(v)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((len(bases) * rows, nq * hd)).astype(np.float32))
    entries = [(s, b, m, b + m, (1 << (m + 1)) - 1) for s, b in enumerate(bases) for m in range(rows)]
    got = _attend(ctx, kv, 0, q16, entries, rows, nq, hd, max(bases) + rows)
    for s, b in enumerate(bases):
        kf, vf = oracle.f16_bits_to_f32(ks[s]), oracle.f16_bits_to_f32(vs[s])
        for m in sorted(set([0, 1, rows // 2, 63 % rows, 64 % rows, rows - 2, rows - 1])):
            want = oracle.causal_attention(oracle.f16_bits_to_f32(q16[s * rows + m]), kf[:b + m + 1], vf[:b + m + 1], hd, nq,
                                           nkv, b + m + 1, 1.0 / np.sqrt(hd))
            _close(oracle, got[s * rows + m], want)
    kv.close()


def test_rope_store_kv_writes_rotated_k_and_plain_v(ctx, oracle):
    import turbospark_b200 as tsb
    hd, nq, nkv = 128, 8, 2
    kv = tsb.KvCache(ctx, 2, nkv, hd, 16, 12, 2, 6)
    kv.reserve(1, 70)
    rng = np.random.default_rng(9)
    rows = 4
    qkv = oracle.f32_to_f16_bits(rng.standard_normal((rows, (nq + 2 * nkv) * hd)).astype(np.float32))
    base = 60
    positions = [60, 61, 61, 62]  # two rows share a depth, as tree siblings do
    entries = [(1, base, m, positions[m], 1) for m in range(rows)]
    qd = ctx.to_device(qkv)
    ctx.rope_store_kv(kv, 1, qd, ctx.to_device(tsb.row_descs(entries)), rows, nq, 10000.0)
    ctx.sync()
    got = qd.download(np.uint16, qkv.size).reshape(qkv.shape)
    k_rows, v_rows = kv.read_rows(1, 1, base, rows)
    for m in range(rows):
        qf = oracle.f16_bits_to_f32(qkv[m, :nq * hd])
        kf = oracle.f16_bits_to_f32(qkv[m, nq * hd:(nq + nkv) * hd])
        want_q = oracle.f32_to_f16_bits(oracle.rope_neox(qf, 1, nq, hd, hd // 2, positions[m], 10000.0))
        want_k = oracle.f32_to_f16_bits(oracle.rope_neox(kf, 1, nkv, hd, hd // 2, positions[m], 10000.0))
        assert (got[m, :nq * hd] != want_q).sum() <= 1
        assert (k_rows[m] != want_k).sum() <= 1
        assert np.array_equal(v_rows[m], qkv[m, (nq + nkv) * hd:])
    # a row outside the reserved pages is reported, not written
    bad = [(1, 200, 0, 200, 1)]
    ctx.rope_store_kv(kv, 1, qd, ctx.to_device(tsb.row_descs(bad)), 1, nq, 10000.0)
    with pytest.raises(tsb.TsbError):
        ctx.sync()
    ctx.sync()  # the error word is cleared and the context stays usable
    kv.close()


def test_kv_cursor_and_paging(ctx, oracle):
    import turbospark_b200 as tsb
    kv = tsb.KvCache(ctx, 1, 2, 64, 16, 7, 2, 4)
    kv.reserve(0, 40)
    kv.set_cursor(0, 40)
    kv.rewind_by(0, 3)
    assert kv.cursor(0) == 37
    with pytest.raises(tsb.TsbError):
        kv.rewind_by(0, 38)
    with pytest.raises(tsb.TsbError):
        kv.reserve(0, 65)  # more pages than the table holds
    kv.reserve(1, 64)
    with pytest.raises(tsb.TsbError):
        kv.reserve(0, 64)  # pool exhausted: 3 + 4 + 1 > 7
    rng = np.random.default_rng(0)
    k = rng.integers(0, 65536, size=(40, 128), dtype=np.uint16)
    v = rng.integers(0, 65536, size=(40, 128), dtype=np.uint16)
    kv.write_rows(0, 0, 0, k, v)
    k2, v2 = kv.read_rows(0, 0, 5, 30)
    assert np.array_equal(k2, k[5:35]) and np.array_equal(v2, v[5:35])
    kv.reset(1)
    kv.reserve(0, 64)
    kv.close()


def test_commit_path_compacts_every_layer_in_place(ctx, oracle):
    # crates/gpu/tests/gather_rows_parity.rs, crates/gpu/src/dflash_conv.rs:192-234
    import turbospark_b200 as tsb
    layers, nkv, hd = 3, 2, 64
    kv = tsb.KvCache(ctx, layers, nkv, hd, 16, 10, 1, 8)
    n = 100
    kv.reserve(0, n)
    rng = np.random.default_rng(4)
    data = []
    for l in range(layers):
        k = rng.integers(0, 65536, size=(n, nkv * hd), dtype=np.uint16)
        v = rng.integers(0, 65536, size=(n, nkv * hd), dtype=np.uint16)
        kv.write_rows(0, l, 0, k, v)
        data.append((k, v))
    base, path = 37, [0, 2, 5, 6, 30]
    kv.commit_path(0, base, path)
    ctx.sync()
    for l in range(layers):
        for which in range(2):
            want = data[l][which].copy()
            assert oracle.gather_rows_inplace(want[base:], path) == 0
            got = kv.read_rows(0, l, 0, n)[which]
            assert np.array_equal(got[:base + len(path)], want[:base + len(path)])
    for bad in ([1, 2], [0, 2, 2], [0, 3, 1], [0, 200]):
        with pytest.raises(tsb.TsbError):
            kv.commit_path(0, base, bad)
    kv.commit_path(0, base, [0, 1, 2])  # a chain moves nothing
    kv.close()
