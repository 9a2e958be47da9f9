"""Model / session bindings and the synthetic configurations the tests and the benchmark use."""
import ctypes as C

import numpy as np

from . import capi
from .capi import lib, Shaping

W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_EMBED, W_LM_HEAD = range(9)
N_ATTN, N_FFN, N_OUT = range(3)


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d_model", "n_q_heads", "n_kv_heads", "head_dim", "ffn", "vocab",
                                         "max_context")] + [("rms_eps", C.c_float), ("rope_theta", C.c_float)]


class RunConfig(C.Structure):
    _fields_ = [("shaping", Shaping), ("max_new_tokens", C.c_int32), ("block", C.c_int32), ("uniform_mode", C.c_int32),
                ("n_stop", C.c_int32), ("stop_tokens", C.c_int32 * 8), ("adaptive", C.c_int32),
                ("tree_nodes", C.c_int32), ("tree_levels", C.c_int32), ("tree_branching", C.c_int32 * 8),
                ("reuse_prefix", C.c_int32), ("tree_best_first", C.c_int32), ("tree_cand", C.c_int32)]


class TreeNode(C.Structure):
    _fields_ = [("depth", C.c_int32), ("cand", C.c_int32), ("parent", C.c_int32)]


class RunResult(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("new_tokens", "reason", "rounds", "accepted_total", "rollbacks", "history_len",
                                         "reused_prefix", "_pad")] + \
               [("kv_position", C.c_int64), ("draws", C.c_uint64), ("prefill_seconds", C.c_double),
                ("decode_seconds", C.c_double)]


def run_config(shaping_cfg, max_new_tokens, block, uniform_mode=0, stop_tokens=(), adaptive=0, tree_nodes=0, tree_branching=(),
               reuse_prefix=False, tree_best_first=False, tree_cand=0, tree_levels=None):
    rc = RunConfig()
    rc.reuse_prefix = 1 if reuse_prefix else 0
    rc.tree_nodes, rc.tree_levels = tree_nodes, (len(tree_branching) if tree_levels is None else tree_levels)
    rc.tree_best_first, rc.tree_cand = (1 if tree_best_first else 0), tree_cand
    for i, b in enumerate(tree_branching):
        rc.tree_branching[i] = b
    rc.shaping = shaping_cfg
    rc.max_new_tokens, rc.block, rc.uniform_mode, rc.adaptive = max_new_tokens, block, uniform_mode, adaptive
    rc.n_stop = len(stop_tokens)
    for i, t in enumerate(stop_tokens):
        rc.stop_tokens[i] = t
    return rc


# Configurations named by the benchmark definition (shapes only; weights are synthetic).
def config_tiny(max_context=1024):
    """4-layer Llama-style decoder: d 512, 8 q x 64, 2 kv, SwiGLU FFN 1408 zero-padded to 1536 (Q4_K needs whole
    256-column superblocks), RMSNorm eps 1e-6, RoPE theta 1e4, vocabulary 8192."""
    return ModelConfig(4, 512, 8, 2, 64, 1536, 8192, max_context, 1e-6, 1e4)


def config_8b_target(max_context=4608):
    return ModelConfig(32, 4096, 32, 8, 128, 14336, 128256, max_context, 1e-5, 5e5)


def config_8b_draft(max_context=4608):
    return ModelConfig(16, 2048, 32, 8, 64, 8192, 128256, max_context, 1e-5, 5e5)


class Model:
    def __init__(self, ctx, cfg):
        self.ctx, self.cfg = ctx, cfg
        h = C.c_void_p()
        ctx.check(lib().tsb_model_create(ctx.h, C.byref(cfg), C.byref(h)))
        self.h = h

    def set_matrix(self, layer, which, qtype, blocks, rows, cols):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        self.ctx.check(lib().tsb_model_set_matrix(self.h, C.c_int32(layer), C.c_int32(which), C.c_int32(qtype),
                                                  blocks.ctypes.data_as(C.c_void_p), C.c_int64(rows), C.c_int64(cols)))

    def set_norm(self, layer, which, bf16):
        bf16 = np.ascontiguousarray(bf16, dtype=np.uint16)
        self.ctx.check(lib().tsb_model_set_norm(self.h, C.c_int32(layer), C.c_int32(which),
                                                bf16.ctypes.data_as(C.c_void_p), C.c_int32(bf16.size)))

    def set_moe(self, n_experts, top_k, moe_ffn):
        """Every layer's feed-forward becomes routed; call before uploading tensors."""
        self.n_experts, self.top_k, self.moe_ffn = n_experts, top_k, moe_ffn
        self.ctx.check(lib().tsb_model_set_moe(self.h, C.c_int32(n_experts), C.c_int32(top_k), C.c_int32(moe_ffn)))

    def set_expert_shard(self, expert_lo, n_local):
        """This model holds experts [expert_lo, expert_lo + n_local) only (after set_moe, before the expert tensors)."""
        self.ctx.check(lib().tsb_model_set_expert_shard(self.h, C.c_int32(expert_lo), C.c_int32(n_local)))

    def set_router(self, layer, q_u8, scale_bf16, bias_bf16):
        q = np.ascontiguousarray(q_u8, dtype=np.uint8)
        sc, bi = np.ascontiguousarray(scale_bf16, dtype=np.uint16), np.ascontiguousarray(bias_bf16, dtype=np.uint16)
        assert q.size == self.n_experts * self.cfg.d_model and sc.size == q.size // 64 == bi.size
        self.ctx.check(lib().tsb_model_set_router(self.h, C.c_int32(layer), q.ctypes.data_as(C.c_void_p),
                                                  sc.ctypes.data_as(C.c_void_p), bi.ctypes.data_as(C.c_void_p)))

    def set_experts(self, layer, qtype, gate_up, down):
        gu, dn = np.ascontiguousarray(gate_up, dtype=np.uint8), np.ascontiguousarray(down, dtype=np.uint8)
        self.ctx.check(lib().tsb_model_set_experts(self.h, C.c_int32(layer), C.c_int32(qtype), gu.ctypes.data_as(C.c_void_p),
                                                   dn.ctypes.data_as(C.c_void_p)))

    def share(self, dst_layer, src, src_layer):
        self.ctx.check(lib().tsb_model_share(self.h, C.c_int32(dst_layer), src.h, C.c_int32(src_layer)))

    def fill_synthetic(self, qtype=capi.Q4_K, lm_head_qtype=None, seed=0):
        self.ctx.check(lib().tsb_model_fill_synthetic(self.h, C.c_int32(qtype),
                                                      C.c_int32(qtype if lm_head_qtype is None else lm_head_qtype),
                                                      C.c_uint64(seed)))

    @property
    def weight_bytes(self):
        lib().tsb_model_weight_bytes.restype = C.c_int64
        return int(lib().tsb_model_weight_bytes(self.h))

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_model_destroy(self.h)
            self.h = None


class Session:
    def __init__(self, ctx, target, draft, n_streams, max_rows, page_tokens=64):
        self.ctx, self.target, self.draft = ctx, target, draft
        self.n_streams, self.max_rows = n_streams, max_rows
        h = C.c_void_p()
        ctx.check(lib().tsb_session_create(ctx.h, target.h, draft.h if draft else None, C.c_int32(n_streams),
                                           C.c_int32(max_rows), C.c_int32(page_tokens), C.byref(h)))
        self.h = h
        self.vocab = target.cfg.vocab

    def _logits(self, n):
        return np.empty((n, self.vocab), dtype=np.uint16)

    def reset(self, stream=0):
        self.ctx.check(lib().tsb_producer_reset(self.h, C.c_int32(stream)))

    def produce(self, token, position, stream=0, want_logits=True):
        out = self._logits(1) if want_logits else None
        self.ctx.check(lib().tsb_producer_produce(self.h, C.c_int32(stream), C.c_int32(token), C.c_int64(position),
                                                  out.ctypes.data_as(C.c_void_p) if want_logits else None))
        return out[0] if want_logits else None

    def produce_prefill(self, token, position, stream=0):
        self.ctx.check(lib().tsb_producer_produce_prefill(self.h, C.c_int32(stream), C.c_int32(token), C.c_int64(position)))

    def prime_drafter(self, nxt, position, stream=0):
        self.ctx.check(lib().tsb_producer_prime_drafter(self.h, C.c_int32(stream), C.c_int32(nxt), C.c_int64(position)))

    def draft_step(self, nxt, position, stream=0):
        out = self._logits(1)
        self.ctx.check(lib().tsb_producer_draft_step(self.h, C.c_int32(stream), C.c_int32(nxt), C.c_int64(position),
                                                     out.ctypes.data_as(C.c_void_p)))
        return out[0]

    def verify(self, feed, base, stream=0):
        feed = np.ascontiguousarray(feed, dtype=np.int32)
        out = self._logits(feed.size)
        self.ctx.check(lib().tsb_producer_verify(self.h, C.c_int32(stream), feed.ctypes.data_as(C.c_void_p),
                                                 C.c_int32(feed.size), C.c_int64(base), out.ctypes.data_as(C.c_void_p)))
        return out

    def verify_tree(self, feed, slot_parent, base, stream=0):
        feed = np.ascontiguousarray(feed, dtype=np.int32)
        par = np.ascontiguousarray(slot_parent, dtype=np.int32)
        out = self._logits(feed.size)
        self.ctx.check(lib().tsb_producer_verify_tree(self.h, C.c_int32(stream), feed.ctypes.data_as(C.c_void_p),
                                                      par.ctypes.data_as(C.c_void_p), C.c_int32(feed.size), C.c_int64(base),
                                                      out.ctypes.data_as(C.c_void_p)))
        return out

    def verify_tree_streams(self, feed, slot_parent, want_logits=True):
        """verify_tree of every stream in one target pass: feed is [n_streams, n] slot tokens over one shared tree."""
        feed = np.ascontiguousarray(feed, dtype=np.int32)
        par = np.ascontiguousarray(slot_parent, dtype=np.int32)
        assert feed.ndim == 2 and feed.shape[1] == par.size
        out = self._logits(feed.size) if want_logits else None
        self.ctx.check(lib().tsb_session_verify_tree(self.h, feed.ctypes.data_as(C.c_void_p), par.ctypes.data_as(C.c_void_p),
                                                     C.c_int32(par.size), out.ctypes.data_as(C.c_void_p) if want_logits else None))
        return out.reshape(feed.shape[0], par.size, -1) if want_logits else None

    def compact_tree(self, base, path, stream=0):
        p = np.ascontiguousarray(path, dtype=np.uint32)
        self.ctx.check(lib().tsb_producer_compact_tree(self.h, C.c_int32(stream), C.c_int64(base),
                                                       p.ctypes.data_as(C.c_void_p), C.c_int32(p.size)))

    def checkpoint(self, stream=0):
        lib().tsb_producer_checkpoint.restype = C.c_int64
        return int(lib().tsb_producer_checkpoint(self.h, C.c_int32(stream)))

    def rollback_retaining(self, point, keep_rows, stream=0):
        self.ctx.check(lib().tsb_producer_rollback_retaining(self.h, C.c_int32(stream), C.c_int64(point), C.c_int32(keep_rows)))

    def rewind_drafter(self, position, stream=0):
        self.ctx.check(lib().tsb_producer_rewind_drafter(self.h, C.c_int32(stream), C.c_int64(position)))

    def set_tree(self, nodes, levels=0, branching=(), best_first=False, cand=0):
        br = (C.c_int32 * 8)(*list(branching)[:8])
        self.ctx.check(lib().tsb_session_set_tree(self.h, C.c_int32(nodes), C.c_int32(levels or len(branching)), br,
                                                  C.c_int32(1 if best_first else 0), C.c_int32(cand)))

    def tree_nodes(self):
        n = int(lib().tsb_producer_tree_nodes(self.h))
        return n or None

    def draft_tree(self, anchor, base, nodes, stream=0):
        """-> (depth, cand, parent) int arrays and the nodes' tokens; parent -1 = under the anchor."""
        tree = (TreeNode * nodes)()
        toks = np.zeros(nodes, dtype=np.int32)
        n = C.c_int32()
        self.ctx.check(lib().tsb_producer_draft_tree(self.h, C.c_int32(stream), C.c_int32(anchor), C.c_int64(base), C.c_int32(nodes),
                                                     tree, toks.ctypes.data_as(C.c_void_p), C.byref(n)))
        k = n.value
        return (np.array([tree[i].depth for i in range(k)], dtype=np.int32), np.array([tree[i].cand for i in range(k)], dtype=np.int32),
                np.array([tree[i].parent for i in range(k)], dtype=np.int32), toks[:k].copy())

    def draft_block(self, anchor, base, block, stream=0):
        out = np.zeros(block, dtype=np.int32)
        self.ctx.check(lib().tsb_producer_draft_block(self.h, C.c_int32(stream), C.c_int32(anchor), C.c_int64(base), C.c_int32(block),
                                                      out.ctypes.data_as(C.c_void_p)))
        return out

    def drafts_block_passes(self):
        return bool(lib().tsb_producer_drafts_block_passes(self.h))

    def commit_pending(self, keep_rows, stream=0):
        self.ctx.check(lib().tsb_producer_commit_pending(self.h, C.c_int32(stream), C.c_int32(keep_rows)))

    def discard_pending(self, stream=0):
        self.ctx.check(lib().tsb_producer_discard_pending(self.h, C.c_int32(stream)))

    def supports_retaining_rollback(self):
        return bool(lib().tsb_producer_supports_retaining_rollback(self.h))

    def supports_headless_prefill(self):
        return bool(lib().tsb_producer_supports_headless_prefill(self.h))

    def try_reuse_prefix(self, prompt, stream=0):
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        lib().tsb_producer_try_reuse_prefix.restype = C.c_int64
        return int(lib().tsb_producer_try_reuse_prefix(self.h, C.c_int32(stream), p.ctypes.data_as(C.c_void_p), C.c_int32(p.size)))

    def record_committed(self, tokens, pos0, stream=0):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        self.ctx.check(lib().tsb_producer_record_committed(self.h, C.c_int32(stream), t.ctypes.data_as(C.c_void_p), C.c_int32(t.size),
                                                           C.c_int64(pos0)))

    def _run(self, fn, prompt, rc, stream):
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        toks = np.zeros(p.size + rc.max_new_tokens + 8, dtype=np.int32)
        emitted = np.zeros(rc.max_new_tokens + 8, dtype=np.int32)
        res = RunResult()
        self.ctx.check(fn(self.h, C.c_int32(stream), p.ctypes.data_as(C.c_void_p), C.c_int32(p.size), C.byref(rc),
                          toks.ctypes.data_as(C.c_void_p), emitted.ctypes.data_as(C.c_void_p), C.byref(res)))
        return toks[:res.history_len].copy(), emitted[:res.new_tokens].copy(), res

    def spec_run(self, prompt, rc, stream=0):
        return self._run(lib().tsb_spec_run, prompt, rc, stream)

    def sequential_run(self, prompt, rc, stream=0):
        return self._run(lib().tsb_sequential_run, prompt, rc, stream)

    def fill_context(self, tokens, seed=0):
        self.ctx.check(lib().tsb_session_fill_context(self.h, C.c_int64(tokens), C.c_uint64(seed)))

    def round(self, rc, next_tokens, draw_steps):
        """One lockstep round; next_tokens (int32[n_streams]) and draw_steps (uint64[n_streams]) are updated in place."""
        accepted = np.zeros(self.n_streams, dtype=np.int32)
        self.ctx.check(lib().tsb_session_round(self.h, C.byref(rc), next_tokens.ctypes.data_as(C.c_void_p),
                                               accepted.ctypes.data_as(C.c_void_p), draw_steps.ctypes.data_as(C.c_void_p)))
        return accepted

    def round_tokens(self, rc, next_tokens, draw_steps):
        """round() that also returns the committed tokens: (accepted[n_streams], tokens[n_streams, 16])."""
        accepted = np.zeros(self.n_streams, dtype=np.int32)
        toks = np.full((self.n_streams, 16), -1, dtype=np.int32)
        self.ctx.check(lib().tsb_session_round_tokens(self.h, C.byref(rc), next_tokens.ctypes.data_as(C.c_void_p),
                                                      accepted.ctypes.data_as(C.c_void_p), toks.ctypes.data_as(C.c_void_p),
                                                      draw_steps.ctypes.data_as(C.c_void_p)))
        return accepted, toks

    def set_comm(self, comm):
        """The passes of this session exchange through `comm` (a turbospark_b200.comm.Comm; None: single GPU)."""
        self.ctx.check(lib().tsb_session_set_comm(self.h, comm.h if comm is not None else None))

    def set_generated(self, generated, stream=0):
        """How many tokens at the end of the stream's history count as generated (the presence / frequency penalties' window)."""
        self.ctx.check(lib().tsb_session_set_generated(self.h, C.c_int32(stream), C.c_int32(generated)))

    def set_graph(self, enabled):
        self.ctx.check(lib().tsb_session_set_graph(self.h, C.c_int32(int(enabled))))

    def round_times(self):
        t = (C.c_float * 4)()
        self.ctx.check(lib().tsb_session_round_times(self.h, t))
        return list(t)

    @property
    def stream_ptr(self):
        lib().tsb_session_stream.restype = C.c_void_p
        return int(lib().tsb_session_stream(self.h))

    def time_matmuls(self, rows, iters):
        """-> (ms per sequence, algorithmic bytes per sequence, launches per sequence)"""
        ms, by, ln = C.c_float(), C.c_int64(), C.c_int32()
        self.ctx.check(lib().tsb_session_time_matmuls(self.h, C.c_int32(rows), C.c_int32(iters), C.byref(ms), C.byref(by),
                                                      C.byref(ln)))
        return ms.value / iters, by.value, ln.value

    def time_pass_rest(self, rows, iters):
        """-> ms per sequence of a pass's launches other than the layer matmuls (embedding, attention, head)"""
        ms = C.c_float()
        self.ctx.check(lib().tsb_session_time_pass_rest(self.h, C.c_int32(rows), C.c_int32(iters), C.byref(ms)))
        return ms.value / iters

    def kv(self, which=0):
        lib().tsb_session_kv.restype = C.c_void_p
        k = capi.KvCache.__new__(capi.KvCache)
        cfg = (self.target if which == 0 else self.draft).cfg
        k.ctx, k.layers, k.kv_heads, k.head_dim = self.ctx, cfg.n_layers, cfg.n_kv_heads, cfg.head_dim
        k.h = C.c_void_p(lib().tsb_session_kv(self.h, C.c_int32(which)))
        return k

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_session_destroy(self.h)
            self.h = None
