"""tsb_attn_decode_rows_static: the attention entry point whose scratch is a fixed area inside the library.

Collected last on purpose (it shares one device-wide area with every other caller in the process), but it also
passes on its own.  Two calls in a row through the C ABI must give what the entry point with a caller-supplied
buffer gives: the area keeps the first call's contents when the second one starts.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL, ABS = 2e-3, 1e-3  # the attention tests' tolerance


def _case(ctx, oracle, tsb, hd, nq, nkv, base, rows, seed):
    page_tokens = 64
    ctx_len = base + rows
    pages = (ctx_len + page_tokens - 1) // page_tokens + 1
    kv = tsb.KvCache(ctx, 1, nkv, hd, page_tokens, pages + 2, 1, pages)
    kv.reserve(0, ctx_len)
    rng = np.random.default_rng(seed)
    k = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
    v = oracle.f32_to_f16_bits(rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32))
    kv.write_rows(0, 0, 0, k, v)
    q16 = oracle.f32_to_f16_bits(rng.standard_normal((rows, nq * hd)).astype(np.float32))
    entries = [(0, base, m, base + m, (1 << (m + 1)) - 1) for m in range(rows)]
    return kv, q16, entries, ctx_len


def _run(ctx, tsb, kv, q16, entries, nq, hd, max_len, static):
    rows = len(entries)
    qd = ctx.to_device(q16)
    out = ctx.alloc(rows * nq * hd * 2)
    rd = ctx.to_device(tsb.row_descs(entries))
    scale = 1.0 / np.sqrt(hd)
    if static:
        ctx.attn_decode_rows_static(kv, 0, qd, nq * hd, out, rd, rows, rows, nq, scale, max_len)
    else:
        scratch = ctx.alloc(ctx.attn_scratch_bytes(rows, nq, hd))
        ctx.attn_decode_rows(kv, 0, qd, nq * hd, out, rd, rows, rows, nq, scale, max_len, scratch)
    ctx.sync()
    return out.download(np.uint16, rows * nq * hd).reshape(rows, nq * hd)


def test_two_calls_in_a_row_match_the_caller_buffer_entry_point(oracle):
    import turbospark_b200 as tsb
    ctx = tsb.Ctx(0)
    try:
        # the second shape is smaller and differently split, so it reads an area still full of the first call's data
        for hd, nq, nkv, base, rows, seed in [(128, 32, 8, 1500, 6, 11), (64, 8, 2, 300, 3, 12)]:
            kv, q16, entries, ctx_len = _case(ctx, oracle, tsb, hd, nq, nkv, base, rows, seed)
            want = oracle.f16_bits_to_f32(_run(ctx, tsb, kv, q16, entries, nq, hd, ctx_len, static=False))
            for _ in range(2):
                got = oracle.f16_bits_to_f32(_run(ctx, tsb, kv, q16, entries, nq, hd, ctx_len, static=True))
                assert not np.isnan(got).any()
                assert np.all(np.abs(got - want) <= ABS + REL * np.abs(want)), float(np.abs(got - want).max())
    finally:
        ctx.close()


def test_a_shape_beyond_the_built_in_area_is_refused_with_both_sizes_named(oracle):
    import turbospark_b200 as tsb
    ctx = tsb.Ctx(0)
    try:
        hd, nq, nkv, base, rows = 128, 32, 8, 100, 12  # 12 rows x 32 heads need about 12.8 MB, the area holds 8 MiB
        kv, q16, entries, ctx_len = _case(ctx, oracle, tsb, hd, nq, nkv, base, rows, 13)
        assert ctx.attn_scratch_bytes(rows, nq, hd) > 8 << 20
        with pytest.raises(tsb.TsbError) as info:
            _run(ctx, tsb, kv, q16, entries, nq, hd, ctx_len, static=True)
        assert "8388608" in str(info.value) and str(ctx.attn_scratch_bytes(rows, nq, hd)) in str(info.value)
    finally:
        ctx.close()
