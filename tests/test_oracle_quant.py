"""The CPU oracle against the reference's own golden vectors for the block formats."""
import json
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def lcg_weights(n, seed):
    # crates/compute/tests/quant_gguf.rs weight generator shape: values in about [-1, 1)
    s = np.uint64(seed * 2654435761 + 1)
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = np.uint64((int(s) * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF)
        out[i] = ((int(s) >> 40) / float(1 << 24)) * 2.0 - 1.0
    return out


def test_q4k_hand_packed_superblock_decodes_to_the_documented_formula(oracle):
    g = json.load(open(os.path.join(GOLD, "q4k_handpacked.json")))
    quants = [(e * 7 + 3) % 16 for e in range(256)]
    block = bytearray(g["d_bits"] + g["dmin_bits"] + g["packed"])
    for grp in range(4):
        for l in range(32):
            at = grp * 64 + l
            block.append(quants[at] | (quants[at + 32] << 4))
    assert len(block) == 144
    got = oracle.dequantize(oracle.Q4K, np.frombuffer(bytes(block), dtype=np.uint8), 256)
    for e in range(256):
        j = e // 32
        want = np.float32(g["d"]) * np.float32(g["ls"][j]) * np.float32(quants[e]) - np.float32(g["dmin"]) * np.float32(g["lm"][j])
        assert got[e] == want, (e, j)


def test_q4k_scale_min_split_bytes(oracle):
    import ctypes as C
    g = json.load(open(os.path.join(GOLD, "q4k_handpacked.json")))
    packed = (C.c_uint8 * 12)(*g["packed"])
    for j in range(8):
        sc, m = C.c_uint8(), C.c_uint8()
        oracle.lib().tso_q4k_scale_min(j, packed, C.byref(sc), C.byref(m))
        assert (sc.value, m.value) == (g["ls"][j], g["lm"][j])


def test_q4k_round_trip_stays_inside_one_step(oracle):
    w = lcg_weights(512, 11)
    out = oracle.dequantize(oracle.Q4K, oracle.quantize(oracle.Q4K, w.reshape(1, -1)), 512)
    for j in range(16):
        sub = w[j * 32:(j + 1) * 32]
        lo = min(0.0, sub.min())
        hi = max(lo, sub.max())
        bound = (hi - lo) / 15.0 * 0.5 + (hi - lo) * 0.05
        assert np.all(np.abs(out[j * 32:(j + 1) * 32] - sub) <= bound)


def test_q4k_min_term_carries_the_sign_and_zero_block(oracle):
    w = np.array([-1.0 + (e % 32) / 64.0 for e in range(256)], dtype=np.float32)
    out = oracle.dequantize(oracle.Q4K, oracle.quantize(oracle.Q4K, w.reshape(1, -1)), 256)
    assert np.all(out < 0) and np.all(np.abs(out - w) < 0.05)
    z = oracle.dequantize(oracle.Q4K, oracle.quantize(oracle.Q4K, np.zeros((1, 256), np.float32)), 256)
    assert np.all(z == 0)


def test_q6k_round_trip(oracle):
    w = lcg_weights(512, 31)
    out = oracle.dequantize(oracle.Q6K, oracle.quantize(oracle.Q6K, w.reshape(1, -1)), 512)
    assert np.max(np.abs(out - w)) < 0.05
    z = oracle.dequantize(oracle.Q6K, oracle.quantize(oracle.Q6K, np.zeros((1, 256), np.float32)), 256)
    assert np.all(z == 0)


def q6k_hand_packed_block(g):
    """The literal superblock of crates/compute/tests/quant_gguf.rs:390-445 and the values its formula gives."""
    block = bytes([g["ql_byte"]] * 128 + [g["qh_byte"]] * 64 + [s & 0xFF for s in g["scales"]]) + int(g["d_bits"]).to_bytes(2, "little")
    assert len(block) == 210
    want = np.empty(256, dtype=np.float32)
    for h in range(2):
        for k in range(4):
            for l in range(32):
                want[h * 128 + k * 32 + l] = np.float32(g["d"]) * np.float32(g["scales"][h * 8 + l // 16 + 2 * k]) * np.float32(g["quants"][k])
    return np.frombuffer(block, dtype=np.uint8), want


def test_q6k_hand_packed_superblock_decodes_to_the_documented_formula(oracle):
    # split 6-bit levels, the bias of 32, signed scales, the scale index striding by 2, the 32-element spacing
    g = json.load(open(os.path.join(GOLD, "q6k_handpacked.json")))
    block, want = q6k_hand_packed_block(g)
    got = oracle.dequantize(oracle.Q6K, block, 256)
    assert np.array_equal(got, want)
    assert got[0] == np.float32(g["spot"]["0"]) and got[176] == np.float32(g["spot"]["176"])


def test_mxfp4_decoder_matches_ggml_bytes_floats_codebook_and_exponents(oracle):
    g = json.load(open(os.path.join(GOLD, "mxfp4_ggml.json")))
    got = oracle.dequantize(oracle.MXFP4, np.array(g["bytes"], dtype=np.uint8), 128)
    want = np.array(g["floats"], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    for i in range(16):
        assert np.float32(oracle.lib().tso_mxfp4_value(i)) == np.float32(g["codebook"][i])
    # index 8 is +0, not -0
    assert np.float32(oracle.lib().tso_mxfp4_value(8)).view(np.uint32) == 0
    for e in range(256):
        got_e = np.float32(oracle.lib().tso_mxfp4_value(1)) * np.float32(oracle.lib().tso_mxfp4_scale(e))
        assert got_e == np.float32(g["e8m0"][e]), e


def test_mxfp4_own_encoder_round_trips(oracle):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal(32 * 64) * 0.02).astype(np.float32)
    q = oracle.quantize(oracle.MXFP4, w.reshape(1, -1))
    out = oracle.dequantize(oracle.MXFP4, q, w.size)
    for b in range(64):
        blk, o = w[b * 32:(b + 1) * 32], out[b * 32:(b + 1) * 32]
        amax = np.abs(blk).max()
        # the coarsest code gap is 4 units of the block scale, and 12*scale < 2*amax
        assert np.all(np.abs(o - blk) <= amax / 3.0 + 1e-9)
    # idempotent in value: re-encoding decoded values decodes to the same floats
    again = oracle.dequantize(oracle.MXFP4, oracle.quantize(oracle.MXFP4, out.reshape(1, -1)), w.size)
    assert np.array_equal(again, out)


def test_gemv_matches_dequantize_then_multiply(oracle):
    n = 512
    x = lcg_weights(n, 5)
    for kind in (oracle.Q4K, oracle.Q6K, oracle.MXFP4):
        rows = np.stack([lcg_weights(n, 20 + r) for r in range(4)])
        q = oracle.quantize(kind, rows)
        got = oracle.gemm_quant(kind, q, 4, n, x.reshape(1, -1))[0]
        for i in range(4):
            deq = oracle.dequantize(kind, q[i], n)
            want = np.float32(0)
            for c in range(n):
                want = np.float32(want + np.float32(deq[c] * x[c]))
            assert got[i] == want


def test_f16_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 65519.99, 5.96e-8, 2.98e-8, 2.9802322e-8], np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16_bits(x)
    assert np.array_equal(got, want)
    allbits = np.arange(65536, dtype=np.uint16)
    back = oracle.f16_bits_to_f32(allbits)
    ref = allbits.view(np.float16).astype(np.float32)
    assert np.array_equal(back.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])


def ref_weights(n, seed):
    """The reference tests' own weight generator (crates/compute/tests/quant_gguf.rs:24-33): 32-bit LCG, values in [-1, 1)."""
    s = (seed * 2654435761 + 1) & 0xFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(s >> 8) / np.float32(1 << 23)) - np.float32(1.0)
    return out


def test_q5k_decodes_exactly_what_ggml_decodes(oracle):
    # crates/compute/tests/quant_gguf.rs:548-555: compared with ==, two superblocks
    g = json.load(open(os.path.join(GOLD, "q5k_ggml.json")))
    raw = np.array(g["bytes"], dtype=np.uint8)
    assert raw.size == 2 * 176 and oracle.row_bytes(oracle.Q5K, 512) == raw.size
    got = oracle.dequantize(oracle.Q5K, raw, 512)
    want = np.array(g["floats"], dtype=np.float32)
    assert np.array_equal(got, want)
    assert (got < 0).any() and (got > 0).any()                      # :592-597 the min term carries the sign
    stripped = raw.copy()                                           # :575-590 the fifth bit matters and only lowers
    for b in range(2):
        stripped[b * 176 + 16:b * 176 + 48] = 0
    without = oracle.dequantize(oracle.Q5K, stripped, 512)
    assert not np.array_equal(got, without) and np.all(got >= without)


def test_q5k_own_encoder_round_trips_inside_one_step(oracle):
    w = (ref_weights(1024, 9) * 0.05).reshape(2, 512)
    q = oracle.quantize(oracle.Q5K, w)
    assert q.shape == (2, 2 * 176)
    back = oracle.dequantize(oracle.Q5K, q, 1024).reshape(2, 512)
    for sub in range(1024 // 32):
        blk = w.reshape(-1, 32)[sub]
        step = (max(blk.max(), 0) - min(blk.min(), 0)) / 31.0
        assert np.abs(back.reshape(-1, 32)[sub] - blk).max() <= step * 1.1 + 1e-4
    assert np.array_equal(oracle.dequantize(oracle.Q5K, oracle.quantize(oracle.Q5K, np.zeros((1, 256), np.float32)), 256), np.zeros(256, np.float32))


def test_q8_0_block_shape_round_trip_idempotence_signs_and_zeros(oracle):
    # crates/compute/tests/quant_gguf.rs:36-42, 93-155
    assert oracle.row_bytes(oracle.Q8_0, 96) == 3 * 34
    w = ref_weights(256, 11)
    out = oracle.dequantize(oracle.Q8_0, oracle.quantize(oracle.Q8_0, w.reshape(1, -1)), 256)
    for b in range(8):
        blk = w[b * 32:(b + 1) * 32]
        amax = np.abs(blk).max()
        assert np.abs(out[b * 32:(b + 1) * 32] - blk).max() <= amax / 127.0 * 0.5 + amax * 1e-3
    once = oracle.quantize(oracle.Q8_0, ref_weights(512, 3).reshape(1, -1))
    twice = oracle.quantize(oracle.Q8_0, oracle.dequantize(oracle.Q8_0, once, 512).reshape(1, -1))
    assert np.array_equal(once, twice)
    w = np.array([-1.0 if i % 2 == 0 else 0.5 for i in range(32)], dtype=np.float32)
    out = oracle.dequantize(oracle.Q8_0, oracle.quantize(oracle.Q8_0, w.reshape(1, -1)), 32)
    assert np.array_equal(out < 0, w < 0) and np.abs(out - w).max() < 0.02
    z = oracle.dequantize(oracle.Q8_0, oracle.quantize(oracle.Q8_0, np.zeros((1, 64), np.float32)), 64)
    assert np.all(z == 0.0)


def test_q5k_q8_0_gemv_is_dequantize_then_multiply_in_index_order(oracle):
    # crates/compute/src/quant_gguf/q5_k.rs:104-118, q8_0.rs:82-96
    for kind, n in ((oracle.Q5K, 512), (oracle.Q8_0, 128)):
        x = ref_weights(n, 5)
        w = np.stack([ref_weights(n, 20 + r) for r in range(4)])
        q = oracle.quantize(kind, w)
        got = oracle.gemm_quant(kind, q.reshape(-1), 4, n, x.reshape(1, n))[0]
        for r in range(4):
            deq = oracle.dequantize(kind, q[r], n)
            acc = np.float32(0)
            for c in range(n):
                acc = np.float32(acc + np.float32(deq[c] * x[c]))
            assert got[r] == acc
