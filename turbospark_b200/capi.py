"""ctypes binding of libtsb.so (include/tsb.h)."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
Q4_K, Q6_K, MXFP4, Q5_K, Q8_0 = 0, 1, 2, 3, 4

_lib = None


class TsbError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("tsb status %d: %s" % (code, message))
        self.code = code


def lib_path():
    # TSB_LIB points at another build of the same library (kernel experiments); the default is the in-tree one
    return os.environ.get("TSB_LIB") or os.path.join(_HERE, "libtsb.so")


class RowDesc(C.Structure):
    _fields_ = [("seq", C.c_int32), ("base", C.c_int32), ("slot", C.c_int32), ("position", C.c_int32),
                ("mask", C.c_uint64 * 2)]


class Shaping(C.Structure):
    _fields_ = [("temperature", C.c_double), ("top_k", C.c_uint32), ("_pad", C.c_uint32), ("top_p", C.c_double),
                ("repetition_penalty", C.c_double), ("presence_penalty", C.c_double),
                ("frequency_penalty", C.c_double), ("min_p", C.c_double), ("seed", C.c_uint64)]


def shaping(temperature=1.0, top_k=0, top_p=0.0, repetition_penalty=1.0, presence_penalty=0.0,
            frequency_penalty=0.0, min_p=0.0, seed=0):
    return Shaping(temperature, top_k, 0, top_p, repetition_penalty, presence_penalty, frequency_penalty, min_p, seed)


class AcceptOut(C.Structure):
    _fields_ = [("accepted", C.c_int32), ("draws", C.c_int32), ("tokens", C.c_int32 * 16), ("status", C.c_int32),
                ("_pad", C.c_int32), ("margin_accept", C.c_double), ("margin_draw", C.c_double)]


def row_descs(entries):
    """entries: iterable of (seq, base, slot, position, mask_int) -> ctypes array of RowDesc."""
    entries = list(entries)
    arr = (RowDesc * len(entries))()
    for i, (seq, base, slot, position, mask) in enumerate(entries):
        arr[i].seq, arr[i].base, arr[i].slot, arr[i].position = seq, base, slot, position
        arr[i].mask[0] = mask & 0xFFFFFFFFFFFFFFFF
        arr[i].mask[1] = (mask >> 64) & 0xFFFFFFFFFFFFFFFF
    return arr


def lib():
    """Loads libtsb.so; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError("libtsb.so is missing: build it with `python -m turbospark_b200.build` "
                              "(no CPU fallback exists)")
        L = C.CDLL(path)
        L.tsb_last_error.restype = C.c_char_p
        L.tsb_last_error.argtypes = [C.c_void_p]
        L.tsb_row_bytes.restype = C.c_int64
        L.tsb_row_bytes.argtypes = [C.c_int32, C.c_int64]
        L.tsb_launch_count.restype = C.c_uint64
        L.tsb_launch_count.argtypes = [C.c_void_p]
        L.tsb_uniform_u64.restype = C.c_uint64
        L.tsb_uniform_u64.argtypes = [C.c_int32, C.c_uint64, C.c_uint64]
        for name in ("tsb_attn_scratch_bytes", "tsb_accept_scratch_bytes", "tsb_accept_history_scratch_bytes", "tsb_gemm_workspace_bytes"):
            if hasattr(L, name):
                getattr(L, name).restype = C.c_size_t
        if hasattr(L, "tsb_kv_cursor"):
            L.tsb_kv_cursor.restype = C.c_int64
            L.tsb_kv_cursor.argtypes = [C.c_void_p, C.c_int32]
        _lib = L
    return _lib


def _vp(x):
    if x is None:
        return None
    if isinstance(x, DeviceBuffer):
        return C.c_void_p(x.ptr)
    if isinstance(x, np.ndarray):
        return x.ctypes.data_as(C.c_void_p)
    if isinstance(x, int):
        return C.c_void_p(x)
    return x


class DeviceBuffer:
    """Device memory owned through tsb_alloc / tsb_free."""

    def __init__(self, ctx, nbytes):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        ctx.check(lib().tsb_alloc(ctx.h, C.c_size_t(self.nbytes), C.byref(p)))
        self.ptr = p.value

    def upload(self, arr, stream=None):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        self.ctx.check(lib().tsb_memcpy_h2d(self.ctx.h, stream, C.c_void_p(self.ptr), _vp(arr), C.c_size_t(arr.nbytes)))
        self.ctx.sync(stream)
        return self

    def download(self, dtype, count, stream=None, offset=0):
        out = np.empty(count, dtype=dtype)
        self.ctx.check(lib().tsb_memcpy_d2h(self.ctx.h, stream, _vp(out), C.c_void_p(self.ptr + offset),
                                            C.c_size_t(out.nbytes)))
        self.ctx.sync(stream)
        return out

    def free(self):
        if self.ptr:
            lib().tsb_free(self.ctx.h, C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Ctx:
    def __init__(self, device=0):
        h = C.c_void_p()
        rc = lib().tsb_ctx_create(C.c_int32(device), C.byref(h))
        if rc:
            raise TsbError(rc, "tsb_ctx_create failed (no CUDA device, or not an sm_100 GPU)")
        self.h = h

    def check(self, rc):
        if rc:
            raise TsbError(rc, lib().tsb_last_error(self.h).decode())

    def sync(self, stream=None):
        self.check(lib().tsb_stream_sync(self.h, stream))

    def alloc(self, nbytes):
        return DeviceBuffer(self, nbytes)

    def to_device(self, arr):
        if isinstance(arr, C.Array):
            arr = np.frombuffer(bytes(arr), dtype=np.uint8)
        arr = np.ascontiguousarray(arr)
        return DeviceBuffer(self, max(arr.nbytes, 16)).upload(arr)

    def upload_weights(self, arr):
        arr = np.ascontiguousarray(arr, dtype=np.uint8)
        p = C.c_void_p()
        self.check(lib().tsb_weights_upload(self.h, _vp(arr), C.c_size_t(arr.nbytes), C.byref(p)))
        b = DeviceBuffer.__new__(DeviceBuffer)
        b.ctx, b.nbytes, b.ptr = self, arr.nbytes, p.value
        return b

    @property
    def launches(self):
        return int(lib().tsb_launch_count(self.h))

    def set_wait_limit_us(self, microseconds):
        """Bound of every wait inside a kernel; when it runs out the kernel reports an error and returns."""
        self.check(lib().tsb_ctx_set_wait_limit_us(self.h, C.c_uint32(microseconds)))

    def debug_wait_nobody(self, out_u32, stream=None):
        self.check(lib().tsb_debug_wait_nobody(self.h, stream, _vp(out_u32)))

    # ---- operators
    def gemm_quant(self, qtype, w, rows, cols, x, y, tokens, y_f32=False, w_off=0, stream=None):
        self.check(lib().tsb_gemm_quant(self.h, stream, C.c_int32(qtype), _vp(w), C.c_uint64(w_off), C.c_int64(rows),
                                        C.c_int64(cols), _vp(x), _vp(y), C.c_int32(tokens), C.c_int32(int(y_f32))))

    def gemm_workspace_bytes(self, qtype, rows, cols, tokens):
        return int(lib().tsb_gemm_workspace_bytes(C.c_int32(qtype), C.c_int64(rows), C.c_int64(cols), C.c_int32(tokens)))

    def gemm_prepare(self, qtype, rows, cols, x, tokens, workspace, stream=None):
        self.check(lib().tsb_gemm_prepare(self.h, stream, C.c_int32(qtype), C.c_int64(rows), C.c_int64(cols), _vp(x), C.c_int32(tokens),
                                          _vp(workspace), C.c_size_t(workspace.nbytes)))

    def gemm_quant_prepared(self, qtype, w, rows, cols, x, workspace, y, tokens, y_f32=False, w_off=0, stream=None):
        self.check(lib().tsb_gemm_quant_prepared(self.h, stream, C.c_int32(qtype), _vp(w), C.c_uint64(w_off), C.c_int64(rows),
                                                 C.c_int64(cols), _vp(x), _vp(workspace), _vp(y), C.c_int32(tokens), C.c_int32(int(y_f32))))

    def dequant_rows(self, qtype, w, cols, row_ids, n_rows, out, w_off=0, stream=None):
        self.check(lib().tsb_dequant_rows(self.h, stream, C.c_int32(qtype), _vp(w), C.c_uint64(w_off), C.c_int64(cols),
                                          _vp(row_ids), C.c_int32(n_rows), _vp(out)))

    def embed_rows(self, qtype, w, vocab_rows, cols, token_ids, n, out, out_scale=1.0, w_off=0, stream=None):
        self.check(lib().tsb_embed_rows(self.h, stream, C.c_int32(qtype), _vp(w), C.c_uint64(w_off),
                                        C.c_int64(vocab_rows), C.c_int64(cols), _vp(token_ids), C.c_int32(n), _vp(out),
                                        C.c_float(out_scale)))

    def rmsnorm_rows(self, x, residual, w_bf16, out, rows, d, eps, stream=None):
        self.check(lib().tsb_rmsnorm_rows(self.h, stream, _vp(x), _vp(residual), _vp(w_bf16), _vp(out), C.c_int32(rows),
                                          C.c_int32(d), C.c_float(eps)))

    def rope_rows(self, x, rows, heads, head_dim, rotated_pairs, row_stride, positions, theta, stream=None):
        self.check(lib().tsb_rope_neox_rows_positions(self.h, stream, _vp(x), C.c_int32(rows), C.c_int32(heads),
                                                      C.c_int32(head_dim), C.c_int32(rotated_pairs),
                                                      C.c_int64(row_stride), _vp(positions), C.c_float(theta)))

    def silu_mul(self, gate, up, out, rows, n, in_stride, out_stride, stream=None):
        self.check(lib().tsb_silu_mul(self.h, stream, _vp(gate), _vp(up), _vp(out), C.c_int32(rows), C.c_int32(n),
                                      C.c_int64(in_stride), C.c_int64(out_stride)))

    def attn_scratch_bytes(self, rows, n_q_heads, head_dim):
        return int(lib().tsb_attn_scratch_bytes(C.c_int32(rows), C.c_int32(n_q_heads), C.c_int32(head_dim)))

    def rope_store_kv(self, kv, layer, qkv, rows_dev, rows, n_q_heads, theta, stream=None):
        self.check(lib().tsb_rope_store_kv(self.h, stream, kv.h, C.c_int32(layer), _vp(qkv), _vp(rows_dev),
                                           C.c_int32(rows), C.c_int32(n_q_heads), C.c_float(theta)))

    def attn_decode_rows(self, kv, layer, q, q_stride, out, rows_dev, rows, rows_per_seq, n_q_heads, scale, max_len,
                         scratch, stream=None):
        self.check(lib().tsb_attn_decode_rows(self.h, stream, kv.h, C.c_int32(layer), _vp(q), C.c_int64(q_stride),
                                              _vp(out), _vp(rows_dev), C.c_int32(rows), C.c_int32(rows_per_seq),
                                              C.c_int32(n_q_heads), C.c_float(scale), C.c_int32(max_len), _vp(scratch),
                                              C.c_size_t(scratch.nbytes)))

    def attn_decode_rows_static(self, kv, layer, q, q_stride, out, rows_dev, rows, rows_per_seq, n_q_heads, scale, max_len,
                                stream=None):
        """tsb_attn_decode_rows with the library's built-in scratch area (no buffer argument, no allocation)."""
        self.check(lib().tsb_attn_decode_rows_static(self.h, stream, kv.h, C.c_int32(layer), _vp(q), C.c_int64(q_stride),
                                                     _vp(out), _vp(rows_dev), C.c_int32(rows), C.c_int32(rows_per_seq),
                                                     C.c_int32(n_q_heads), C.c_float(scale), C.c_int32(max_len)))

    def accept_scratch_bytes(self, batch, k, vocab):
        return int(lib().tsb_accept_scratch_bytes(C.c_int32(batch), C.c_int32(k), C.c_int32(vocab)))

    def accept(self, target_logits, draft_logits, proposals, uniforms, batch, k, vocab, shaping_cfg, out, scratch,
               stream=None):
        self.check(lib().tsb_accept(self.h, stream, _vp(target_logits), _vp(draft_logits), _vp(proposals), _vp(uniforms),
                                    C.c_int32(batch), C.c_int32(k), C.c_int32(vocab), C.byref(shaping_cfg), _vp(out),
                                    _vp(scratch), C.c_size_t(scratch.nbytes)))

    def sample(self, logits, uniforms, batch, vocab, shaping_cfg, tokens, margins, scratch, stream=None):
        self.check(lib().tsb_sample(self.h, stream, _vp(logits), _vp(uniforms), C.c_int32(batch), C.c_int32(vocab),
                                    C.byref(shaping_cfg), _vp(tokens), _vp(margins), _vp(scratch),
                                    C.c_size_t(scratch.nbytes)))

    def accept_history_scratch_bytes(self, batch, k, vocab):
        return int(lib().tsb_accept_history_scratch_bytes(C.c_int32(batch), C.c_int32(k), C.c_int32(vocab)))

    def accept_history(self, target_logits, draft_logits, proposals, uniforms, batch, k, vocab, shaping_cfg, history, hist_stride,
                       hist_len, generated, out, scratch, stream=None):
        """tsb_accept with the history penalties: history [batch, hist_stride] i32, hist_len / generated [batch] i32 (device)."""
        self.check(lib().tsb_accept_history(self.h, stream, _vp(target_logits), _vp(draft_logits), _vp(proposals), _vp(uniforms),
                                            C.c_int32(batch), C.c_int32(k), C.c_int32(vocab), C.byref(shaping_cfg), _vp(history),
                                            C.c_int32(hist_stride), _vp(hist_len), _vp(generated), _vp(out), _vp(scratch),
                                            C.c_size_t(scratch.nbytes)))

    def sample_history(self, logits, uniforms, batch, vocab, shaping_cfg, history, hist_stride, hist_len, generated, tokens, margins,
                       scratch, stream=None):
        self.check(lib().tsb_sample_history(self.h, stream, _vp(logits), _vp(uniforms), C.c_int32(batch), C.c_int32(vocab),
                                            C.byref(shaping_cfg), _vp(history), C.c_int32(hist_stride), _vp(hist_len), _vp(generated),
                                            _vp(tokens), _vp(margins), _vp(scratch), C.c_size_t(scratch.nbytes)))

    def moe_route(self, router_logits, tokens, n_experts, k, ids_out, weights_out, scale=None, stream=None):
        self.check(lib().tsb_moe_route(self.h, stream, _vp(router_logits), C.c_int32(tokens), C.c_int32(n_experts), C.c_int32(k),
                                       _vp(scale) if scale is not None else None, _vp(ids_out), _vp(weights_out)))

    def router_logits(self, q_u8, scale_bf16, bias_bf16, x, tokens, n_experts, d_model, logits_out, stream=None):
        self.check(lib().tsb_router_logits(self.h, stream, _vp(q_u8), _vp(scale_bf16), _vp(bias_bf16), _vp(x), C.c_int32(tokens),
                                           C.c_int32(n_experts), C.c_int32(d_model), _vp(logits_out)))

    def moe_ffn(self, qtype, gate_up, down, n_experts, d_model, ffn, x, residual, ids, weights, tokens, k, y, stream=None):
        self.check(lib().tsb_moe_ffn(self.h, stream, C.c_int32(qtype), _vp(gate_up), C.c_uint64(0), _vp(down), C.c_uint64(0),
                                     C.c_int32(n_experts), C.c_int32(d_model), C.c_int32(ffn), _vp(x), _vp(residual), _vp(ids),
                                     _vp(weights), C.c_int32(tokens), C.c_int32(k), _vp(y)))

    def residual_add(self, x, y, n, stream=None):
        self.check(lib().tsb_residual_add(self.h, stream, _vp(x), _vp(y), C.c_int64(n)))

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        pass  # explicit close only: buffers may outlive the Python object order at interpreter exit


class KvCache:
    def __init__(self, ctx, layers, kv_heads, head_dim, page_tokens, num_pages, max_seqs, max_pages_per_seq):
        self.ctx = ctx
        self.layers, self.kv_heads, self.head_dim = layers, kv_heads, head_dim
        h = C.c_void_p()
        ctx.check(lib().tsb_kv_create(ctx.h, C.c_int32(layers), C.c_int32(kv_heads), C.c_int32(head_dim),
                                      C.c_int32(page_tokens), C.c_int32(num_pages), C.c_int32(max_seqs),
                                      C.c_int32(max_pages_per_seq), C.byref(h)))
        self.h = h

    def reserve(self, seq, tokens):
        self.ctx.check(lib().tsb_kv_reserve(self.h, C.c_int32(seq), C.c_int64(tokens)))

    def reset(self, seq):
        self.ctx.check(lib().tsb_kv_reset(self.h, C.c_int32(seq)))

    def cursor(self, seq):
        return int(lib().tsb_kv_cursor(self.h, C.c_int32(seq)))

    def set_cursor(self, seq, pos):
        self.ctx.check(lib().tsb_kv_set_cursor(self.h, C.c_int32(seq), C.c_int64(pos)))

    def rewind_by(self, seq, count):
        self.ctx.check(lib().tsb_kv_rewind_by(self.h, C.c_int32(seq), C.c_int64(count)))

    def write_rows(self, seq, layer, pos0, k, v, stream=None):
        k = np.ascontiguousarray(k, dtype=np.uint16)
        v = np.ascontiguousarray(v, dtype=np.uint16)
        n = k.size // (self.kv_heads * self.head_dim)
        self.ctx.check(lib().tsb_kv_write_rows(self.h, stream, C.c_int32(seq), C.c_int32(layer), C.c_int64(pos0),
                                               C.c_int32(n), _vp(k), _vp(v)))

    def read_rows(self, seq, layer, pos0, n, stream=None):
        k = np.empty((n, self.kv_heads * self.head_dim), dtype=np.uint16)
        v = np.empty_like(k)
        self.ctx.check(lib().tsb_kv_read_rows(self.h, stream, C.c_int32(seq), C.c_int32(layer), C.c_int64(pos0),
                                              C.c_int32(n), _vp(k), _vp(v)))
        return k, v

    def fill_random(self, seq, tokens, seed, stream=None):
        self.ctx.check(lib().tsb_kv_fill_random(self.h, stream, C.c_int32(seq), C.c_int64(tokens), C.c_uint64(seed)))

    def commit_path(self, seq, base, path, stream=None):
        p = np.ascontiguousarray(path, dtype=np.uint32)
        self.ctx.check(lib().tsb_kv_commit_path(self.ctx.h, stream, self.h, C.c_int32(seq), C.c_int64(base), _vp(p),
                                                C.c_int32(p.size)))

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_kv_destroy(self.h)
            self.h = None
