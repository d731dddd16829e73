"""The kernel libraries as built: every C function the Python side declares is exported.
Needs the CUDA compiler but no GPU (nvcc cross-compiles; the libraries load without a device)."""

from __future__ import annotations

import ctypes
import shutil

import pytest


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="no CUDA compiler")
def test_every_declared_entry_point_is_exported():
    from inference_engine_b200.kernels.build import build_attention, build_core
    from inference_engine_b200.kernels.cuda_ops import CudaOps

    core = ctypes.CDLL(str(build_core()))
    fake = type("Declared", (), {"lib": core})()
    CudaOps._declare(fake)  # looks every core entry point up by name
    assert hasattr(core, "ie_set_pdl")
    attention = ctypes.CDLL(str(build_attention(64)))
    for name in ("ie_set_pdl", "ie_set_decode_pair", "ie_attention_decode", "ie_attention_decode_balanced", "ie_attention_prefill",
                 "ie_attention_prefill_tc5", "ie_attention_prefill_tc5_ok", "ie_attention_prefill_rows",
                 "ie_attention_decode_scratch_floats", "ie_attention_decode_balanced_scratch_floats",
                 "ie_attention_decode_balanced_max_seqs", "ie_attention_prefill_tc5_scratch_floats",
                 "ie_attention_decode_static", "ie_attention_decode_static_capacity_floats"):
        assert hasattr(attention, name), name
