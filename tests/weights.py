"""Seeded weight sets for the tests and the smoke run: random matrices quantized by the ORACLE's encoders and
pushed into a library Model or an oracle Model through the same builder interface.  Test scaffolding - the product
package never imports this module (or the oracle)."""
import numpy as np

from turbospark_b200 import capi
from turbospark_b200.model import (W_EMBED, W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_LM_HEAD, N_ATTN, N_FFN, N_OUT)


def random_weights(cfg, seed, oracle, qtype=capi.Q4_K, std=0.02, real_ffn=None, qtype_of=None):
    """Seeded N(0, std) weights quantized by the oracle's encoder (test / small-model set-up).  Returns a dict
    (layer, which) -> (blocks uint8 [rows, row_bytes], rows, cols, qtype) and norms (layer, which) -> bf16 bits.
    real_ffn < cfg.ffn zero-pads the FFN (rows of gate/up and columns of down beyond real_ffn are zero).
    qtype_of maps a tensor kind (W_V, W_DOWN, ...) to a block format other than `qtype`, as mixed recipes do."""
    rng = np.random.default_rng(seed)
    qd, kd, d, f = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.d_model, cfg.ffn
    rf = real_ffn or f
    mats, norms = {}, {}

    def mk(rows, cols, zero_rows_from=None, zero_cols_from=None, which=None):
        qt = (qtype_of or {}).get(which, qtype)
        w = (rng.standard_normal((rows, cols)) * std).astype(np.float32)
        if zero_rows_from is not None:
            w[zero_rows_from:] = 0
        if zero_cols_from is not None:
            w[:, zero_cols_from:] = 0
        return oracle.quantize(qt, w), rows, cols, qt

    mats[(-1, W_EMBED)] = mk(cfg.vocab, d, which=W_EMBED)
    for l in range(cfg.n_layers):
        mats[(l, W_Q)] = mk(qd, d, which=W_Q)
        mats[(l, W_K)] = mk(kd, d, which=W_K)
        mats[(l, W_V)] = mk(kd, d, which=W_V)
        mats[(l, W_O)] = mk(d, qd, which=W_O)
        mats[(l, W_GATE)] = mk(f, d, zero_rows_from=rf, which=W_GATE)
        mats[(l, W_UP)] = mk(f, d, zero_rows_from=rf, which=W_UP)
        mats[(l, W_DOWN)] = mk(d, f, zero_cols_from=rf, which=W_DOWN)
        for which in (N_ATTN, N_FFN):
            norms[(l, which)] = np.array([oracle.lib().tso_f32_to_bf16(float(v)) for v in 1.0 + 0.05 * rng.standard_normal(d)], dtype=np.uint16)
    mats[(-1, W_LM_HEAD)] = mk(cfg.vocab, d, which=W_LM_HEAD)
    norms[(-1, N_OUT)] = np.array([oracle.lib().tso_f32_to_bf16(float(v)) for v in 1.0 + 0.05 * rng.standard_normal(d)], dtype=np.uint16)
    return mats, norms


DENSE_FFN = (W_GATE, W_UP, W_DOWN)


def load_weights(model, mats, norms, qtype=None, layers=None, order=None, skip=()):
    """Push a random_weights() set into a tsb Model or an oracle Model (same builder interface).  Each matrix goes
    up in the format it was quantized in (`qtype` overrides it); `order` lists tensor kinds to upload first."""
    n_layers = model.cfg.n_layers if layers is None else layers
    first = list(order or [])
    keys = sorted(mats, key=lambda k: first.index(k[1]) if k[1] in first else len(first))  # stable: the rest keep their order
    for (l, which) in keys:
        blocks, rows, cols, qt = mats[(l, which)]
        if l >= n_layers or which in skip:
            continue
        model.set_matrix(max(l, 0), which, qt if qtype is None else qtype, blocks, rows, cols)
    for (l, which), bits in norms.items():
        if l >= n_layers:
            continue
        model.set_norm(max(l, 0), which, bits)


def random_moe_weights(cfg, n_experts, moe_ffn, seed, oracle, qtype=capi.MXFP4, std=0.05):
    """Seeded routers (8-bit affine: u8 [E, d], bf16 scale and bias per 64 columns) and experts (block rows, per
    expert gate then up [2F, d], and down [d, F]) for every layer: {layer: (q, scale, bias, gate_up, down)}."""
    rng = np.random.default_rng(seed)
    d = cfg.d_model
    bf16 = np.vectorize(lambda v: oracle.lib().tso_f32_to_bf16(float(v)), otypes=[np.uint16])
    out = {}
    for l in range(cfg.n_layers):
        q = rng.integers(0, 256, size=(n_experts, d), dtype=np.uint8)
        sc = bf16(0.004 * (0.5 + rng.random((n_experts, d // 64))))
        bi = bf16(-0.5 * (0.5 + rng.random((n_experts, d // 64))))   # about -128 * scale: zero-mean weights
        gu = np.concatenate([oracle.quantize(qtype, (rng.standard_normal((2 * moe_ffn, d)) * std).astype(np.float32)) for _ in range(n_experts)])
        dn = np.concatenate([oracle.quantize(qtype, (rng.standard_normal((d, moe_ffn)) * std).astype(np.float32)) for _ in range(n_experts)])
        out[l] = (q, sc, bi, gu, dn)
    return out


def load_moe_weights(model, moe, qtype=capi.MXFP4):
    """Push a random_moe_weights() set into a tsb Model or an oracle Model (set_moe must have been called)."""
    for l, (q, sc, bi, gu, dn) in moe.items():
        model.set_router(l, q, sc, bi)
        model.set_experts(l, qtype, gu, dn)
