"""The C-ABI library loads on a machine without a GPU and exports every symbol the header
declares (no compute calls here)."""
import os
import re

import carat_b200
from carat_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    header = open(os.path.join(ROOT, "include", "carat_b200.h")).read()
    return sorted(set(re.findall(r"\b(carat_b200_[a-z0-9_]+)\s*\(", header)))


def test_every_declared_symbol_is_exported_and_bound():
    library = carat_b200.library()
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(library, name), name
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_library_reports_its_abi_version_and_errors():
    library = carat_b200.library()
    assert library.carat_b200_abi_version() == 1
    # An invalid shape is rejected on the host before any CUDA call.
    assert library.carat_b200_fp8_linear_workspace_bytes(0, 128, 128) == 0
    assert library.carat_b200_fp8_linear_workspace_bytes(120, 8192, 5376) == 3 * 120 * 5376 * 4
    assert library.carat_b200_fp8_linear_workspace_bytes(120, 5376, 18944) == 0
    status = library.carat_b200_fp8_linear(None, None, None, None, None, 4, 128, 128, None, 0, None)
    assert status != 0
    assert b"invalid FP8 linear shape" in library.carat_b200_last_error()


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(capi, "_library", None)
    monkeypatch.setattr(capi, "LIBRARY_PATH", "/nonexistent/libcarat_b200.so")
    try:
        capi.library()
    except carat_b200.CaratError as error:
        assert "no CPU or PyTorch fallback" in str(error)
    else:
        raise AssertionError("loading a missing library must fail")
