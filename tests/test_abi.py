"""The shared library loads on a machine without a GPU and exports every symbol that
include/b200gptq.h declares (no kernel is launched here)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200gptq.h")).read()
    return sorted(set(re.findall(r"B200GPTQ_API\s+[\w\s\*]+?\b(b200gptq_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for must in ("b200gptq_gemv", "b200gptq_gemm", "b200gptq_dequant", "b200gptq_sort_rows",
                 "b200gptq_workspace_bytes", "b200gptq_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from autogptq.tvm_b200 import build
    path = build.build()  # no-op when the library is newer than its sources
    lib = ctypes.CDLL(path)
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_status_strings_and_host_side_queries():
    from autogptq.tvm_b200 import _lib
    lib = _lib.lib
    assert lib.b200gptq_abi_version() >= 1
    assert lib.b200gptq_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert lib.b200gptq_strerror(code) not in (b"", b"unknown status")
    assert lib.b200gptq_strerror(-99) == b"unknown status"
    # argument validation happens on the host before anything touches the device
    assert lib.b200gptq_gemv(None, None, None, None, None, None, None, None, 1, 4096, 4096, 4, 128, None, 0, None) == -1
    assert lib.b200gptq_dequant(None, None, None, None, 4096, 4096, 4, 128, None, None, None) == -1


def test_quantlinear_refuses_cpu_tensors_and_bad_bits():
    import pytest
    import torch
    from autogptq.tvm_b200 import QuantLinear
    with pytest.raises(NotImplementedError):
        QuantLinear(5, 128, 256, 64, False)
    with pytest.raises(ValueError):
        QuantLinear(4, 128, 100, 64, False)
    layer = QuantLinear(4, 128, 256, 64, True)
    assert layer.qweight.shape == (32, 64) and layer.qzeros.shape == (2, 8) and layer.scales.shape == (2, 64)
    assert layer.g_idx.tolist()[:3] == [0, 0, 0] and int(layer.g_idx[-1]) == 1
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 256))
