"""turbospark_b200 — CUDA (sm_100a) backend for TurboSpark's speculative-decoding verify path.

The product is the C-ABI shared library ``libtsb.so`` (declared in include/tsb.h); this package
is the thin Python binding used by the tests and the benchmark.  There is no CPU fallback: if the
library has not been built, or no CUDA device is present, loading or creating a context fails.
"""
from .capi import (row_descs, shaping, Ctx, DeviceBuffer, TsbError, lib, lib_path, Q4_K, Q6_K, MXFP4, Q5_K, Q8_0, RowDesc, Shaping, AcceptOut,
                   KvCache)

__all__ = ["row_descs", "shaping", "Ctx", "DeviceBuffer", "TsbError", "lib", "lib_path", "Q4_K", "Q6_K", "MXFP4", "Q5_K", "Q8_0", "RowDesc", "Shaping",
           "AcceptOut", "KvCache"]
from .model import (Model, Session, ModelConfig, RunConfig, RunResult, TreeNode, run_config, config_tiny, config_8b_target,
                    config_8b_draft)
