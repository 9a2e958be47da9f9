"""ctypes front end for the CPU oracle (oracle/libtsb_oracle.so).

Test infrastructure only: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtsb_oracle.so")

Q4K, Q6K, MXFP4, Q5K, Q8_0 = 0, 1, 2, 3, 4
W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_EMBED, W_LM_HEAD = range(9)
N_ATTN, N_FFN, N_OUT = range(3)


def build(force=False):
    """Compile the oracle with the Makefile beside this file."""
    srcs = [os.path.join(_HERE, f) for f in ("tsb_oracle.cpp", "tsb_oracle_model.inc", "Makefile")]
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= max(os.path.getmtime(s) for s in srcs)):
        return _LIB_PATH
    subprocess.check_call(["make", "-C", _HERE, "-B", "libtsb_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class Shaping(C.Structure):
    _fields_ = [("temperature", C.c_double), ("top_k", C.c_uint32), ("_pad", C.c_uint32), ("top_p", C.c_double),
                ("repetition_penalty", C.c_double), ("presence_penalty", C.c_double),
                ("frequency_penalty", C.c_double), ("min_p", C.c_double), ("seed", C.c_uint64)]


def shaping(temperature=1.0, top_k=0, top_p=0.0, repetition_penalty=1.0, presence_penalty=0.0,
            frequency_penalty=0.0, min_p=0.0, seed=0):
    return Shaping(temperature, top_k, 0, top_p, repetition_penalty, presence_penalty, frequency_penalty, min_p, seed)


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d_model", "n_q_heads", "n_kv_heads", "head_dim", "ffn",
                                         "vocab", "max_context")] + [("rms_eps", C.c_float), ("rope_theta", C.c_float)]


class RunConfig(C.Structure):
    _fields_ = [("shaping", Shaping), ("max_new_tokens", C.c_int32), ("block", C.c_int32),
                ("uniform_mode", C.c_int32), ("n_stop", C.c_int32), ("stop_tokens", C.c_int32 * 8),
                ("adaptive", C.c_int32)]


class RunResult(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("new_tokens", "reason", "rounds", "accepted_total", "rollbacks",
                                         "history_len")] + [("kv_position", C.c_int64), ("draws", C.c_uint64)]


class Adaptive(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("floor", "cap", "cur", "climb", "pressure")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        L = _lib
        L.tso_f16_to_f32.restype = C.c_float
        L.tso_f16_to_f32.argtypes = [C.c_uint16]
        L.tso_f32_to_f16.restype = C.c_uint16
        L.tso_f32_to_f16.argtypes = [C.c_float]
        L.tso_bf16_to_f32.restype = C.c_float
        L.tso_bf16_to_f32.argtypes = [C.c_uint16]
        L.tso_f32_to_bf16.restype = C.c_uint16
        L.tso_f32_to_bf16.argtypes = [C.c_float]
        L.tso_mxfp4_scale.restype = C.c_float
        L.tso_mxfp4_scale.argtypes = [C.c_uint8]
        L.tso_mxfp4_value.restype = C.c_float
        L.tso_row_bytes.restype = C.c_int64
        L.tso_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.tso_derive_step_value.restype = C.c_uint64
        L.tso_derive_step_value.argtypes = [C.c_uint64, C.c_uint64]
        L.tso_to_unit_interval.restype = C.c_double
        L.tso_to_unit_interval.argtypes = [C.c_uint64]
        L.tso_uniform_u64.restype = C.c_uint64
        L.tso_uniform_u64.argtypes = [C.c_int, C.c_uint64, C.c_uint64]
        L.tso_shaped_distribution.restype = C.c_int64
        L.tso_residual.restype = C.c_int64
        L.tso_draw.restype = C.c_uint32
        L.tso_model_create.restype = C.c_void_p
        L.tso_state_create.restype = C.c_void_p
        L.tso_state_create.argtypes = [C.c_void_p]
        L.tso_state_cursor.restype = C.c_int64
        L.tso_state_cursor.argtypes = [C.c_void_p]
        L.tso_state_k.restype = C.c_void_p
        L.tso_state_v.restype = C.c_void_p
        L.tso_adaptive_tile_cap.restype = C.c_int64
        L.tso_adaptive_tile_cap.argtypes = [C.c_int64, C.c_int64]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def f32_to_f16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().tso_f32_to_f16_n(_p(x), _p(y), C.c_int64(x.size))
    return y


def f16_bits_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    y = np.empty(x.shape, dtype=np.float32)
    lib().tso_f16_to_f32_n(_p(x), _p(y), C.c_int64(x.size))
    return y


def row_bytes(kind, cols):
    return int(lib().tso_row_bytes(kind, cols))


_QUANT = {Q4K: "tso_quantize_q4k", Q6K: "tso_quantize_q6k", MXFP4: "tso_quantize_mxfp4", Q5K: "tso_quantize_q5k",
          Q8_0: "tso_quantize_q8_0"}
_DEQUANT = {Q4K: "tso_dequantize_q4k", Q6K: "tso_dequantize_q6k", MXFP4: "tso_dequantize_mxfp4", Q5K: "tso_dequantize_q5k",
            Q8_0: "tso_dequantize_q8_0"}


def quantize(kind, w):
    """w: [rows, cols] f32 -> uint8 [rows, row_bytes]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    rb = row_bytes(kind, cols)
    out = np.zeros((rows, rb), dtype=np.uint8)
    assert cols % (32 if kind in (MXFP4, Q8_0) else 256) == 0, "row is not a whole number of blocks"
    # rows are contiguous block runs, so the whole matrix quantizes as one long row
    getattr(lib(), _QUANT[kind])(_p(w), C.c_int64(rows * cols), _p(out))
    return out


def dequantize(kind, blocks, n):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    getattr(lib(), _DEQUANT[kind])(_p(blocks), C.c_int64(n), _p(out))
    return out


def gemm_quant(kind, w_bytes, rows, cols, x, threads=1):
    """x: [tokens, cols] f32 -> y [tokens, rows] f32 (sequential f32 sums)."""
    w_bytes = np.ascontiguousarray(w_bytes, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, cols)
    y = np.empty((x.shape[0], rows), dtype=np.float32)
    lib().tso_gemm_quant(kind, _p(w_bytes), C.c_int64(rows), C.c_int64(cols), _p(x), C.c_int64(x.shape[0]), _p(y),
                         C.c_int(threads))
    return y


def moe_route(logits, k, scale=None):
    """router_topk_gemma4: ids [tokens, k] in rank order, weights [tokens, k] as f16 bits."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tokens, n_experts = logits.shape
    ids = np.empty((tokens, k), dtype=np.int32)
    w = np.empty((tokens, k), dtype=np.uint16)
    sc = None if scale is None else np.ascontiguousarray(scale, dtype=np.float32)
    lib().tso_moe_route(_p(logits), C.c_int64(tokens), C.c_int64(n_experts), C.c_int64(k), _p(sc) if sc is not None else None,
                        _p(ids), _p(w))
    return ids, w


def moe_ffn(kind, gate_up, down, n_experts, d_model, ffn, x16, resid16, ids, w16, threads=1):
    gate_up = np.ascontiguousarray(gate_up, dtype=np.uint8)
    down = np.ascontiguousarray(down, dtype=np.uint8)
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    resid16 = np.ascontiguousarray(resid16, dtype=np.uint16)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    w16 = np.ascontiguousarray(w16, dtype=np.uint16)
    tokens, k = ids.shape
    y = np.empty((tokens, d_model), dtype=np.uint16)
    lib().tso_moe_ffn(C.c_int(kind), _p(gate_up), _p(down), C.c_int64(n_experts), C.c_int64(d_model), C.c_int64(ffn), _p(x16),
                      _p(resid16), _p(ids), _p(w16), C.c_int64(tokens), C.c_int64(k), _p(y), C.c_int(threads))
    return y


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    lib().tso_rms_norm(_p(x), _p(w), C.c_int64(x.size), C.c_float(eps), _p(out))
    return out


def rope_neox(x, num_tokens, num_heads, head_dim, rotated_pairs, position, theta):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().tso_rope_neox(_p(x), C.c_int64(num_tokens), C.c_int64(num_heads), C.c_int64(head_dim),
                        C.c_int64(rotated_pairs), C.c_int64(position), C.c_float(theta), _p(out))
    return out


def silu_mul(g, u):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    out = np.empty_like(g)
    lib().tso_silu_mul(_p(g), _p(u), C.c_int64(g.size), _p(out))
    return out


def causal_attention(q, k, v, hd, nq, nkv, seq_len, scale):
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    out = np.empty(nq * hd, dtype=np.float32)
    lib().tso_causal_attention(_p(q), _p(k), _p(v), C.c_int64(hd), C.c_int64(nq), C.c_int64(nkv), C.c_int64(seq_len),
                               C.c_float(scale), _p(out))
    return out


def indexed_attention(q, k, v, positions, hd, nq, nkv, scale):
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    out = np.empty(nq * hd, dtype=np.float32)
    lib().tso_indexed_attention(_p(q), _p(k), _p(v), _p(pos), C.c_int64(pos.size), C.c_int64(hd), C.c_int64(nq),
                                C.c_int64(nkv), C.c_float(scale), _p(out))
    return out


def _hist(history):
    h = np.ascontiguousarray(history if history is not None else [], dtype=np.int32)
    return h


def select(logits_f16, cfg, history=None, position=0):
    lg = np.ascontiguousarray(logits_f16, dtype=np.uint16)
    h = _hist(history)
    out = C.c_int32(-1)
    rc = lib().tso_select(_p(lg), C.c_int64(lg.size), C.byref(cfg), _p(h), C.c_int64(h.size), C.c_uint64(position),
                          C.byref(out))
    if rc:
        raise ValueError("select error %d" % rc)
    return out.value


def shaped_distribution(logits_f16, cfg, history=None, position=0):
    lg = np.ascontiguousarray(logits_f16, dtype=np.uint16)
    h = _hist(history)
    sup = np.empty(lg.size, dtype=np.uint32)
    pr = np.empty(lg.size, dtype=np.float64)
    n = lib().tso_shaped_distribution(_p(lg), C.c_int64(lg.size), C.byref(cfg), _p(h), C.c_int64(h.size),
                                      C.c_uint64(position), _p(sup), _p(pr), C.c_int64(lg.size))
    if n < 0:
        raise ValueError("shaped_distribution error %d" % -n)
    return sup[:n].copy(), pr[:n].copy()


def residual(p, q):
    ps, pp = (np.ascontiguousarray(p[0], dtype=np.uint32), np.ascontiguousarray(p[1], dtype=np.float64))
    qs, qp = (np.ascontiguousarray(q[0], dtype=np.uint32), np.ascontiguousarray(q[1], dtype=np.float64))
    os_ = np.empty(ps.size, dtype=np.uint32)
    op = np.empty(ps.size, dtype=np.float64)
    n = lib().tso_residual(_p(ps), _p(pp), C.c_int64(ps.size), _p(qs), _p(qp), C.c_int64(qs.size), _p(os_), _p(op))
    if n == 0:
        return None
    return os_[:n].copy(), op[:n].copy()


def draw(dist, target):
    s = np.ascontiguousarray(dist[0], dtype=np.uint32)
    p = np.ascontiguousarray(dist[1], dtype=np.float64)
    return int(lib().tso_draw(_p(s), _p(p), C.c_int64(s.size), C.c_double(target)))


def derive_step_value(seed, position):
    return int(lib().tso_derive_step_value(seed, position))


def to_unit_interval(v):
    return float(lib().tso_to_unit_interval(v))


def uniform_u64(mode, seed, step):
    return int(lib().tso_uniform_u64(mode, seed, step))


def accept_round(target_logits, draft_logits, proposals, cfg, uniforms, history=None, generated=0):
    """target_logits [(k+1), V] u16, draft_logits [k, V] u16 -> (accepted, tokens[accepted+1], draws, margins)."""
    tl = np.ascontiguousarray(target_logits, dtype=np.uint16)
    dl = np.ascontiguousarray(draft_logits, dtype=np.uint16)
    pr = np.ascontiguousarray(proposals, dtype=np.int32)
    un = np.ascontiguousarray(uniforms, dtype=np.uint64)
    h = _hist(history)
    k = pr.size
    v = tl.shape[-1]
    acc = C.c_int32(0)
    toks = np.full(k + 1, -1, dtype=np.int32)
    margins = np.zeros(2, dtype=np.float64)
    draws = lib().tso_accept_round(_p(tl), _p(dl), C.c_int64(v), C.c_int(k), _p(pr), C.byref(cfg), _p(un), _p(h),
                                   C.c_int64(h.size), C.c_uint64(generated), C.byref(acc), _p(toks), _p(margins))
    if draws < 0:
        raise ValueError("accept_round error %d" % -draws)
    return acc.value, toks[:acc.value + 1].copy(), draws, margins


def sample(logits_f16, cfg, uniform, history=None, generated=0):
    lg = np.ascontiguousarray(logits_f16, dtype=np.uint16)
    h = _hist(history)
    tok = C.c_int32(-1)
    margin = C.c_double(0)
    rc = lib().tso_sample(_p(lg), C.c_int64(lg.size), C.byref(cfg), C.c_uint64(uniform), _p(h), C.c_int64(h.size),
                          C.c_uint64(generated), C.byref(tok), C.byref(margin))
    if rc:
        raise ValueError("sample error %d" % rc)
    return tok.value, margin.value


def tree_spec(parent, max_depth=None):
    par = np.ascontiguousarray(parent, dtype=np.int32)
    n = par.size
    md = max_depth or n
    depth = np.zeros(n, dtype=np.int32)
    paths = np.zeros((n, md), dtype=np.int32)
    rc = lib().tso_tree_spec(_p(par), C.c_int(n), _p(depth), _p(paths), C.c_int(md))
    if rc:
        raise ValueError("slot %d's parent must precede it" % (rc - 1))
    return depth, paths


def tree_slot_parents(node_parent):
    np_ = np.ascontiguousarray(node_parent, dtype=np.int32)
    out = np.zeros(np_.size + 1, dtype=np.int32)
    lib().tso_tree_slot_parents(_p(np_), C.c_int(np_.size), _p(out))
    return out


def tree_accept(node_parent, node_token, target_pick):
    a = np.ascontiguousarray(node_parent, dtype=np.int32)
    b = np.ascontiguousarray(node_token, dtype=np.int32)
    c = np.ascontiguousarray(target_pick, dtype=np.int32)
    out = np.zeros(a.size + 1, dtype=np.int32)
    n = lib().tso_tree_accept(_p(a), _p(b), C.c_int(a.size), _p(c), _p(out))
    return out[:n].copy()


def best_first_tree(scores, nodes):
    s = np.ascontiguousarray(scores, dtype=np.float32)
    depth_max, branch = s.shape
    d = np.zeros(nodes, dtype=np.int32)
    c = np.zeros(nodes, dtype=np.int32)
    p = np.zeros(nodes, dtype=np.int32)
    n = lib().tso_best_first_tree(_p(s), C.c_int(depth_max), C.c_int(branch), C.c_int(nodes), _p(d), _p(c), _p(p))
    return d[:n].copy(), c[:n].copy(), p[:n].copy()


def gather_rows_inplace(rows_u16, map_):
    m = np.ascontiguousarray(map_, dtype=np.uint32)
    assert rows_u16.dtype == np.uint16 and rows_u16.flags.c_contiguous
    return int(lib().tso_gather_rows_inplace(_p(rows_u16), C.c_int64(rows_u16.shape[1]), _p(m), C.c_int(m.size)))


def router_logits(q_u8, scale_bf16, bias_bf16, x16, experts):
    """router_gemv_gemma4 with the all-ones effective scale: [tokens, experts] f32."""
    x = np.ascontiguousarray(x16, dtype=np.uint16)
    tokens, d = x.shape
    q = np.ascontiguousarray(q_u8, dtype=np.uint8)
    sc, bi = np.ascontiguousarray(scale_bf16, dtype=np.uint16), np.ascontiguousarray(bias_bf16, dtype=np.uint16)
    out = np.empty((tokens, experts), dtype=np.float32)
    lib().tso_router_logits(_p(q), _p(sc), _p(bi), _p(x), C.c_int64(tokens), C.c_int64(experts), C.c_int64(d), _p(out))
    return out


class Model:
    """CPU model: Llama-style decoder over quantized matrices, dense or with a routed feed-forward."""

    def __init__(self, cfg: ModelCfg, threads=1):
        self.cfg = cfg
        self.h = C.c_void_p(lib().tso_model_create(C.byref(cfg), C.c_int(threads)))

    def set_matrix(self, layer, which, kind, data, rows, cols):
        data = np.ascontiguousarray(data, dtype=np.uint8)
        assert data.size == rows * row_bytes(kind, cols)
        lib().tso_model_set_matrix(self.h, C.c_int(layer), C.c_int(which), C.c_int(kind), _p(data), C.c_int64(rows),
                                   C.c_int64(cols))

    def set_norm(self, layer, which, bf16):
        bf16 = np.ascontiguousarray(bf16, dtype=np.uint16)
        lib().tso_model_set_norm(self.h, C.c_int(layer), C.c_int(which), _p(bf16), C.c_int64(bf16.size))

    def set_moe(self, n_experts, top_k, moe_ffn):
        """Every layer's feed-forward becomes routed (families/llama/moe.rs)."""
        self.n_experts, self.top_k, self.moe_ffn = n_experts, top_k, moe_ffn
        lib().tso_model_set_moe(self.h, C.c_int(n_experts), C.c_int(top_k), C.c_int(moe_ffn))

    def set_router(self, layer, q_u8, scale_bf16, bias_bf16):
        q = np.ascontiguousarray(q_u8, dtype=np.uint8)
        sc, bi = np.ascontiguousarray(scale_bf16, dtype=np.uint16), np.ascontiguousarray(bias_bf16, dtype=np.uint16)
        assert q.size == self.n_experts * self.cfg.d_model and sc.size == q.size // 64 == bi.size
        lib().tso_model_set_router(self.h, C.c_int(layer), _p(q), _p(sc), _p(bi))

    def set_experts(self, layer, kind, gate_up, down):
        gu, dn = np.ascontiguousarray(gate_up, dtype=np.uint8), np.ascontiguousarray(down, dtype=np.uint8)
        assert gu.size == self.n_experts * 2 * self.moe_ffn * row_bytes(kind, self.cfg.d_model)
        assert dn.size == self.n_experts * self.cfg.d_model * row_bytes(kind, self.moe_ffn)
        lib().tso_model_set_experts(self.h, C.c_int(layer), C.c_int(kind), _p(gu), _p(dn))

    def __del__(self):
        if getattr(self, "h", None):
            lib().tso_model_destroy(self.h)
            self.h = None


class State:
    def __init__(self, model: Model):
        self.model = model
        self.h = C.c_void_p(lib().tso_state_create(model.h))

    @property
    def cursor(self):
        return int(lib().tso_state_cursor(self.h))

    @cursor.setter
    def cursor(self, v):
        lib().tso_state_set_cursor(self.h, C.c_int64(v))

    def kv(self, layer):
        cfg = self.model.cfg
        n = cfg.max_context * cfg.n_kv_heads * cfg.head_dim
        kp = lib().tso_state_k(self.h, C.c_int(layer))
        vp = lib().tso_state_v(self.h, C.c_int(layer))
        k = np.ctypeslib.as_array(C.cast(kp, C.POINTER(C.c_uint16)), shape=(n,))
        v = np.ctypeslib.as_array(C.cast(vp, C.POINTER(C.c_uint16)), shape=(n,))
        return k, v

    def forward(self, tokens, start, parent=None, want_logits=True):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        v = self.model.cfg.vocab
        out = np.empty((t.size, v), dtype=np.uint16) if want_logits else None
        par = np.ascontiguousarray(parent, dtype=np.int32) if parent is not None else None
        rc = lib().tso_forward(self.h, _p(t), C.c_int(t.size), C.c_int64(start), _p(par) if par is not None else None,
                               _p(out) if out is not None else None)
        if rc:
            raise RuntimeError("oracle forward error %d" % rc)
        return out

    def __del__(self):
        if getattr(self, "h", None):
            lib().tso_state_destroy(self.h)
            self.h = None


def run_config(cfg_shaping, max_new_tokens, block, uniform_mode=0, stop_tokens=(), adaptive=0):
    rc = RunConfig()
    rc.shaping = cfg_shaping
    rc.max_new_tokens = max_new_tokens
    rc.block = block
    rc.uniform_mode = uniform_mode
    rc.n_stop = len(stop_tokens)
    for i, t in enumerate(stop_tokens):
        rc.stop_tokens[i] = t
    rc.adaptive = adaptive
    return rc


def _run_out(n_prompt, rc):
    cap = n_prompt + rc.max_new_tokens + 8
    return np.zeros(cap, dtype=np.int32), np.zeros(rc.max_new_tokens + 8, dtype=np.int32), RunResult()


def run_speculative_model(target: State, draft: State, prompt, rc: RunConfig):
    p = np.ascontiguousarray(prompt, dtype=np.int32)
    toks, emitted, res = _run_out(p.size, rc)
    err = lib().tso_run_speculative_model(target.h, draft.h, _p(p), C.c_int(p.size), C.byref(rc), _p(toks),
                                          _p(emitted), C.byref(res))
    if err:
        raise RuntimeError("oracle run_speculative error %d" % err)
    return toks[:res.history_len].copy(), emitted[:res.new_tokens].copy(), res


def run_sequential_model(target: State, prompt, rc: RunConfig):
    p = np.ascontiguousarray(prompt, dtype=np.int32)
    toks, emitted, res = _run_out(p.size, rc)
    err = lib().tso_run_sequential_model(target.h, _p(p), C.c_int(p.size), C.byref(rc), _p(toks), _p(emitted),
                                         C.byref(res))
    if err:
        raise RuntimeError("oracle run_sequential error %d" % err)
    return toks[:res.history_len].copy(), emitted[:res.new_tokens].copy(), res


def run_scripted(vocab, quality, graded, speculative, prompt, rc: RunConfig, max_context):
    p = np.ascontiguousarray(prompt, dtype=np.int32)
    toks, emitted, res = _run_out(p.size, rc)
    counters = np.zeros(8, dtype=np.int32)
    err = lib().tso_run_scripted(C.c_int64(vocab), C.c_int(quality), C.c_int(graded), C.c_int(speculative), _p(p),
                                 C.c_int(p.size), C.byref(rc), C.c_int64(max_context), _p(toks), _p(emitted),
                                 C.byref(res), _p(counters))
    return err, toks[:max(res.history_len, 0)].copy(), emitted[:max(res.new_tokens, 0)].copy(), res, counters
