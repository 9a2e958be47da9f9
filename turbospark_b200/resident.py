"""The resident weight file: the reader (through the C ABI) and a writer of the same layout.

Layout (reference: crates/model-io/src/resident_index.rs:19-67, crates/repack/src/resident_writer.rs:375-470):
24-byte header (index size, resident size, entry count), 72-byte entries, the string table, zero padding to a
16 KiB page with the 16-byte format trailer ("GTURBIDX", version, reserved) in its last bytes, then the tensor
bytes, each entry starting on a 4-byte boundary.  The writer exists so installs can be produced for this backend
and so the reader has files to read in tests; block bytes go through untouched.
"""
import ctypes as C
import struct

import numpy as np

from . import capi
from .capi import lib

HEADER_BYTES, ENTRY_BYTES, TRAILER_BYTES, PAGE_BYTES = 24, 72, 16, 16384
INDEX_MAGIC, INDEX_FORMAT_VERSION = b"GTURBIDX", 1
DTYPE_BF16 = 1
# dtype tag bytes of the block formats (crates/repack/src/resident_writer.rs:103-162)
DTYPE_OF_QTYPE = {capi.Q4_K: 7, capi.Q6_K: 8, capi.MXFP4: 14, capi.Q5_K: 13, capi.Q8_0: 6}


class ResidentEntry(C.Structure):
    _fields_ = [("dtype", C.c_uint8), ("_pad", C.c_uint8 * 3), ("shape", C.c_uint32 * 4), ("file_offset", C.c_uint64),
                ("size_bytes", C.c_uint64), ("scale_offset", C.c_uint64), ("scale_size", C.c_uint64),
                ("bias_offset", C.c_uint64), ("bias_size", C.c_uint64)]


class ResidentError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("tsb_resident error %d: %s" % (code, message))
        self.code, self.message = code, message


def _check(rc):
    if rc != 0:
        lib().tsb_resident_last_error.restype = C.c_char_p
        raise ResidentError(rc, (lib().tsb_resident_last_error() or b"").decode("utf-8", "replace"))


class ResidentIndex:
    """An opened index: `len()`, `names()`, `find(name)`; `load_into(model)` uploads a Llama-family tensor set."""

    def __init__(self, path):
        h = C.c_void_p()
        _check(lib().tsb_resident_open(str(path).encode(), C.byref(h)))
        self.h = h
        L = lib()
        L.tsb_resident_count.restype = C.c_int64
        L.tsb_resident_index_size.restype = C.c_uint64
        L.tsb_resident_data_size.restype = C.c_uint64

    def __len__(self):
        return int(lib().tsb_resident_count(self.h))

    @property
    def index_size(self):
        return int(lib().tsb_resident_index_size(self.h))

    @property
    def data_size(self):
        return int(lib().tsb_resident_data_size(self.h))

    def entry_at(self, i):
        e, name = ResidentEntry(), C.create_string_buffer(65536 + 1)
        _check(lib().tsb_resident_entry_at(self.h, C.c_int64(i), C.byref(e), name, C.c_int32(len(name))))
        return name.value.decode("utf-8", "replace"), e

    def names(self):
        return [self.entry_at(i)[0] for i in range(len(self))]

    def find(self, name):
        e = ResidentEntry()
        _check(lib().tsb_resident_find(self.h, name.encode(), C.byref(e)))
        return e

    def load_into(self, model, tie_word_embeddings=False):
        model.ctx.check(lib().tsb_model_load_resident(model.h, self.h, C.c_int32(1 if tie_word_embeddings else 0)))

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_resident_close(self.h)
            self.h = None

    __del__ = close


def build_resident_file(tensors, trailer_version=INDEX_FORMAT_VERSION):
    """tensors: list of (name, dtype_tag, shape tuple (<= 4), payload bytes) -> the file's bytes."""
    table_end = HEADER_BYTES + len(tensors) * ENTRY_BYTES
    names = [t[0].encode() for t in tensors]
    string_end = table_end + sum(len(n) for n in names)
    index_size = -(-(string_end + TRAILER_BYTES) // PAGE_BYTES) * PAGE_BYTES
    cursor, placed = 0, []
    for _, _, _, payload in tensors:
        cursor += (4 - cursor % 4) % 4
        placed.append(index_size + cursor)
        cursor += len(payload)
    out = bytearray(struct.pack("<QQQ", index_size, cursor, len(tensors)))
    name_at = table_end
    for (name, dtype, shape, payload), nb, off in zip(tensors, names, placed):
        shp = tuple(shape) + (0,) * (4 - len(shape))
        out += struct.pack("<IHBBQQ4IQQQQ", name_at, len(nb), dtype, 0, off, len(payload), *shp, 0, 0, 0, 0)
        name_at += len(nb)
    for nb in names:
        out += nb
    out += bytes(index_size - TRAILER_BYTES - len(out))
    out += INDEX_MAGIC + struct.pack("<II", trailer_version, 0) if trailer_version is not None else bytes(TRAILER_BYTES)
    assert len(out) == index_size
    for (_, _, _, payload), off in zip(tensors, placed):
        out += bytes(off - len(out))
        out += bytes(payload)
    return bytes(out)


def llama_tensor_list(cfg, mats, norms, tied=False):
    """A random_weights() set under the names the reference's Llama runner looks up
    (crates/runtime/src/families/llama/mod.rs:49-51,99,371-386; attn.rs:173-197,438; dense.rs:60-62)."""
    from .model import (W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_EMBED, W_LM_HEAD, N_ATTN, N_FFN, N_OUT)
    suffix = {W_Q: "self_attn.q_proj.weight", W_K: "self_attn.k_proj.weight", W_V: "self_attn.v_proj.weight",
              W_O: "self_attn.o_proj.weight", W_GATE: "mlp.gate_proj.weight", W_UP: "mlp.up_proj.weight",
              W_DOWN: "mlp.down_proj.weight"}
    out = []

    def mat(name, key):
        blocks, rows, cols, qt = mats[key]
        out.append((name, DTYPE_OF_QTYPE[qt], (rows, cols, 1, 1), np.ascontiguousarray(blocks, dtype=np.uint8).tobytes()))

    def norm(name, key):
        out.append((name, DTYPE_BF16, (cfg.d_model, 1, 1, 1), np.ascontiguousarray(norms[key], dtype=np.uint16).tobytes()))

    mat("language_model.model.embed_tokens.weight", (-1, W_EMBED))
    for l in range(cfg.n_layers):
        p = "language_model.model.layers.%d." % l
        norm(p + "input_layernorm.weight", (l, N_ATTN))
        for w in (W_Q, W_K, W_V, W_O):
            mat(p + suffix[w], (l, w))
        norm(p + "post_attention_layernorm.weight", (l, N_FFN))
        for w in (W_GATE, W_UP, W_DOWN):
            mat(p + suffix[w], (l, w))
    norm("language_model.model.norm.weight", (-1, N_OUT))
    if not tied:
        mat("language_model.lm_head.weight", (-1, W_LM_HEAD))
    return out
