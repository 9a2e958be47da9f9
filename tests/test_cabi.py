"""CPU-side checks of the drop-in boundary: the shared library loads and exports every symbol include/tsb.h
declares, refuses to run without a CUDA device, and the Python binding's struct layouts match the header."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tsb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"TSB_API\s+[\w\s\*]+?\b(tsb_\w+)\s*\(", text)))


def test_header_declares_the_operator_and_producer_surface():
    syms = declared_symbols()
    for needed in ("tsb_gemm_quant", "tsb_gemv_q4k", "tsb_gemm_mxfp4", "tsb_attn_decode_rows", "tsb_kv_commit_path",
                   "tsb_accept", "tsb_sample", "tsb_rope_store_kv", "tsb_rmsnorm_rows", "tsb_producer_verify",
                   "tsb_producer_draft_step", "tsb_producer_rollback_retaining", "tsb_producer_compact_tree",
                   "tsb_producer_rewind_drafter", "tsb_spec_run", "tsb_session_round", "tsb_producer_draft_tree",
                   "tsb_producer_tree_nodes", "tsb_producer_draft_block", "tsb_producer_commit_pending",
                   "tsb_producer_discard_pending", "tsb_producer_supports_retaining_rollback",
                   "tsb_producer_supports_headless_prefill", "tsb_best_first_tree", "tsb_tree_accept",
                   "tsb_tree_slot_parents", "tsb_ctx_set_wait_limit_us", "tsb_gemm_workspace_bytes", "tsb_gemm_prepare",
                   "tsb_gemm_quant_prepared"):
        assert needed in syms, needed
    assert len(syms) >= 60


def test_library_exports_every_declared_symbol():
    import turbospark_b200 as tsb
    lib = tsb.lib()
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_every_declaration_cites_the_reference_interface_it_replaces():
    text = open(os.path.join(ROOT, "include", "tsb.h")).read()
    assert text.count("crates/") >= 30


def test_no_cuda_device_fails_loudly_not_silently():
    import turbospark_b200 as tsb
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a CUDA device is present")
    with pytest.raises(tsb.TsbError):
        tsb.Ctx(0)


def test_struct_layouts_match_the_header():
    import turbospark_b200 as tsb
    assert C.sizeof(tsb.RowDesc) == 32
    assert C.sizeof(tsb.Shaping) == 64
    assert C.sizeof(tsb.AcceptOut) == 96
    assert C.sizeof(tsb.ModelConfig) == 40
    # shaping, four ints, stop tokens, adaptive, tree nodes/levels, branching list, reuse_prefix, best-first flag and width
    assert C.sizeof(tsb.RunConfig) == 64 + 4 * 4 + 32 + 4 + 2 * 4 + 32 + 4 + 2 * 4
    assert C.sizeof(tsb.TreeNode) == 12
    assert tsb.lib().tsb_row_bytes(0, 4096) == 2304 and tsb.lib().tsb_row_bytes(1, 4096) == 3360
    assert tsb.lib().tsb_row_bytes(2, 4096) == 2176
    assert tsb.lib().tsb_row_bytes(3, 4096) == 16 * 176 and tsb.lib().tsb_row_bytes(4, 4096) == 128 * 34
    assert tsb.lib().tsb_row_bytes(5, 4096) == -1


def test_uniform_sources_match_the_oracle(oracle):
    import turbospark_b200 as tsb
    for mode in (0, 1):
        for seed, step in ((0, 0), (2, 7), (2**63 + 5, 2**40 + 3), (4, 5000)):
            assert tsb.lib().tsb_uniform_u64(mode, seed, step) == oracle.uniform_u64(mode, seed, step)
    # Philox4x32-10 known answer (Random123 kat_vectors: counter 0, key 0)
    assert oracle.uniform_u64(1, 0, 0) == (0xE169C58D << 32 | 0x6627E8D5)


def test_tree_helpers_match_the_oracle(oracle):
    """dflash_best_first_tree, dflash_tree_accept and dflash_tree_slot_parents are host code of the library
    (crates/runtime/src/dflash_tree.rs:30-124): they run without a GPU and must equal the oracle's restatement."""
    import numpy as np
    import turbospark_b200 as tsb
    lib = tsb.lib()
    rng = np.random.default_rng(0)
    for depth_max, branch, nodes in [(3, 4, 7), (5, 3, 20), (2, 8, 12), (4, 2, 40), (1, 5, 9)]:
        scores = (rng.standard_normal((depth_max, branch)) * 2.0).astype(np.float32)
        if branch >= 3:
            scores[0, 2] = scores[0, 1]  # a tie: the lower candidate goes first
        want_d, want_c, want_p = oracle.best_first_tree(scores, nodes)
        out = (tsb.TreeNode * nodes)()
        n = lib.tsb_best_first_tree(scores.ctypes.data_as(C.c_void_p), C.c_int32(depth_max), C.c_int32(branch), C.c_int32(nodes), out)
        assert n == len(want_d)
        assert [out[i].depth for i in range(n)] == list(want_d)
        assert [out[i].cand for i in range(n)] == list(want_c)
        assert [out[i].parent for i in range(n)] == list(want_p)
        sp = np.zeros(n + 1, dtype=np.int32)
        assert lib.tsb_tree_slot_parents(out, C.c_int32(n), sp.ctypes.data_as(C.c_void_p)) == 0
        assert list(sp) == list(oracle.tree_slot_parents(want_p))
        # the accept walk over random tokens / picks
        toks = rng.integers(0, 4, size=n).astype(np.int32)
        picks = rng.integers(0, 4, size=n + 1).astype(np.int32)
        acc = np.zeros(n + 1, dtype=np.int32)
        k = lib.tsb_tree_accept(out, toks.ctypes.data_as(C.c_void_p), C.c_int32(n), picks.ctypes.data_as(C.c_void_p),
                                acc.ctypes.data_as(C.c_void_p))
        assert list(acc[:k]) == list(oracle.tree_accept(want_p, toks, picks))
    # the reference's own worked example (dflash_tree.rs tests): a prefix of a best-first tree is the best tree of its size
    scores = np.array([[0.0, -1.0, -2.0], [0.5, -0.5, -3.0]], dtype=np.float32)
    big = (tsb.TreeNode * 6)()
    small = (tsb.TreeNode * 3)()
    nb = lib.tsb_best_first_tree(scores.ctypes.data_as(C.c_void_p), 2, 3, 6, big)
    ns = lib.tsb_best_first_tree(scores.ctypes.data_as(C.c_void_p), 2, 3, 3, small)
    assert nb == 6 and ns == 3
    assert [(big[i].depth, big[i].cand, big[i].parent) for i in range(3)] == [(small[i].depth, small[i].cand, small[i].parent) for i in range(3)]
