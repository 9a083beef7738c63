"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as ct
import os
import re

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qtensor_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:void|int|unsigned long long|const char \*)\s*\*?\s*((?:c|qt_)\w+)\s*\(", text)
    return sorted(set(names))


def test_header_lists_the_sixteen_reference_symbols():
    names = declared_functions()
    legacy = [n for n in names if n.startswith("c")]
    assert len(legacy) == 16
    for op in ("quantize", "dequantize"):
        for kind in ("", "diagreal_"):
            for bits in (8, 4):
                for dt in ("fp32", "bf16"):
                    assert f"c{op}_blockwise_{kind}{bits}bit_{dt}" in legacy


def test_library_exports_every_declared_symbol(native_lib):
    for name in declared_functions():
        assert hasattr(native_lib, name), name


def test_status_codes_without_gpu(native_lib):
    lib = native_lib
    assert lib.qt_version() >= 100
    assert lib.qt_error_string(0) == b"ok"
    # argument validation happens before any CUDA call, so it is testable on a CPU box
    null = ct.c_void_p(0)
    one = ct.c_void_p(16)
    assert lib.qt_quantize_blockwise(one, 0, 0, one, 64, 1, one, 0, null, 0, one, 0, 63, 4, null) == 2
    assert lib.qt_quantize_blockwise(one, 0, 0, one, 64, 1, one, 0, null, 0, one, 0, 64, 5, null) == 3
    assert lib.qt_quantize_blockwise(one, 7, 0, one, 64, 1, one, 0, null, 0, one, 0, 64, 4, null) == 5
    assert lib.qt_quantize_blockwise(null, 0, 0, one, 64, 1, one, 0, null, 0, one, 0, 64, 4, null) == 1
    assert lib.qt_last_error() == 1
    assert lib.qt_dequantize_blockwise(one, 0, one, 64, 1, one, 0, null, 0, one, 0, 0, 100, 4, null) == 2
    assert lib.qt_dequantize_blockwise(one, 0, one, -1, 1, one, 0, null, 0, one, 0, 0, 64, 4, null) == 1
    # empty work is a no-op, not an error
    assert lib.qt_quantize_blockwise(null, 0, 0, null, 0, 0, null, 0, null, 0, null, 0, 64, 4, null) == 0
    # legacy symbols record instead of exiting the process (reference: ops.cuh:20-26)
    lib.cquantize_blockwise_4bit_fp32(null, one, 64, one, one, 64)
    assert lib.qt_last_error() == 1


def test_functional_rejects_cpu_tensors(native_lib):
    import pytest
    import torch
    import qtensor.functional as F
    code = F.create_linear_map(True, 4, 2)
    with pytest.raises(RuntimeError):
        F.quantize_blockwise(torch.zeros(64, 64), code, 64, blocksize=64, bits=4)
    with pytest.raises(RuntimeError):
        F.dequantize_blockwise(torch.zeros(2048, dtype=torch.uint8), code, 64, torch.zeros(64), blocksize=64, bits=4)
