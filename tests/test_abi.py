"""The C-ABI library loads and exports every symbol include/zinc_cuda.h declares (no compute calls)."""
import ctypes as C
import os
import re

import pytest

import zinc_b200 as zb
from zinc_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "zinc_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    L = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L, n), f"{n} declared in zinc_cuda.h but not exported"
    assert set(names) == set(_lib.EXPORTS)


def test_integration_binding_lists_every_export():
    """The reference-side binding written out in INTEGRATION.md has one extern per exported function."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    bound = set(re.findall(r'pub extern "zinc_b200" fn (zc_[a-z0-9_]+)\(', text))
    assert bound == set(declared_symbols())


def test_layout_helpers_match_reference_constants():
    # src/model/gguf.zig:545-576, src/compute/forward.zig:11409-11423, 11737-11756
    assert (zb.block_size(zb.Q4_K), zb.bytes_per_block(zb.Q4_K)) == (256, 144)
    assert (zb.block_size(zb.Q5_K), zb.bytes_per_block(zb.Q5_K)) == (256, 176)
    assert (zb.block_size(zb.Q6_K), zb.bytes_per_block(zb.Q6_K)) == (256, 210)
    assert (zb.block_size(zb.Q8_0), zb.bytes_per_block(zb.Q8_0)) == (32, 34)
    assert (zb.block_size(zb.MXFP4), zb.bytes_per_block(zb.MXFP4)) == (32, 17)
    assert zb.tensor_size_bytes(zb.Q4_K, 4096 * 4096) == 9_437_184
    assert zb.expert_slice_bytes(zb.Q4_K, 512, 2048) == 589_824
    assert zb.expert_slice_bytes(zb.Q5_K, 2048, 512) == 720_896
    assert zb.expert_slice_bytes(zb.Q6_K, 256, 2048) == 430_080
    assert zb.expert_slice_bytes(zb.Q8_0, 2048, 2048) == 4_456_448
    assert zb.expert_slice_bytes(zb.F16, 512, 2048) == 2_097_152


def test_layout_helpers_agree_with_oracle(oracle):
    for t in (zb.F32, zb.F16, zb.Q5_0, zb.Q5_1, zb.Q8_0, zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.MXFP4):
        assert zb.block_size(t) == oracle.block_size(t)
        assert zb.bytes_per_block(t) == oracle.bytes_per_block(t)
        assert zb.expert_slice_bytes(t, 96, 1024) == oracle.expert_slice_bytes(t, 96, 1024)


def test_type_support_tables():
    # pipelineForType (src/compute/dmmv.zig:678-691)
    L = _lib.lib()
    for t in (zb.Q4_K, zb.MXFP4, zb.Q5_0, zb.Q5_1, zb.Q5_K, zb.Q6_K, zb.Q8_0, zb.F16, zb.F32):
        assert L.zc_dmmv_supported(t) == 1
    for t in (2, 3, 9, 10, 11, 15, 30):  # q4_0 q4_1 q8_1 q2_k q3_k q8_k bf16
        assert L.zc_dmmv_supported(t) == 0


def test_status_strings_and_null_context():
    L = _lib.lib()
    assert L.zc_status_string(0) == b"ok"
    assert b"invalid" in L.zc_status_string(3)
    assert L.zc_barrier(None) == _lib.ERR_INVALID_ARG
    assert L.zc_submit_and_wait(None) == _lib.ERR_INVALID_ARG
    assert L.zc_launch_count(None) == 0


def test_no_cpu_fallback_without_device():
    """Without a CUDA device the context cannot be created: there is no host compute path."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(zb.ZincError):
        zb.Context(0)


def test_product_does_not_import_oracle():
    """Nothing under zinc_b200/ may reference the oracle."""
    pkg = os.path.join(ROOT, "zinc_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath.split(os.sep):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
