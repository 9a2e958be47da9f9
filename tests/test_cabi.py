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
                   "tsb_producer_rewind_drafter", "tsb_spec_run", "tsb_session_round"):
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
    # shaping, four ints, stop tokens, adaptive, tree nodes/levels, branching list, padding to 8
    assert C.sizeof(tsb.RunConfig) == 64 + 4 * 4 + 32 + 4 + 2 * 4 + 32 + 4
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
