"""The C-ABI library loads without a GPU and exports every symbol the public header declares (no compute calls)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "mptorch_b200.h")
LIB = os.path.join(ROOT, "mptorch_b200", "lib", "libmptorch_b200.so")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"MPT_API\s+[\w\s\*]+?\b(mpt_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        from mptorch_b200 import build

        build.build()
    return ctypes.CDLL(LIB)


def test_header_declares_entry_points():
    names = declared_symbols()
    assert len(names) >= 18
    for must in ("mpt_float_quantize_nearest", "mpt_float_mm_nearest", "mpt_float_softmax_forward",
                 "mpt_float_layernorm_backward", "mpt_binary8_quantize", "mpt_last_error"):
        assert must in names


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_exported(lib, name):
    assert getattr(lib, name) is not None


def test_no_undeclared_exports(lib):
    import subprocess

    out = subprocess.run(["nm", "-D", "--defined-only", LIB], capture_output=True, text=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln and ln.split()[-1].startswith("mpt_")}
    assert exported == set(declared_symbols())


def test_calls_without_device_memory_report_errors(lib):
    """Argument validation happens before any CUDA call, so it can be exercised on a machine without a GPU."""
    lib.mpt_last_error.restype = ctypes.c_char_p
    lib.mpt_version.restype = ctypes.c_int
    assert lib.mpt_version() >= 100
    lib.mpt_float_quantize_nearest.restype = ctypes.c_int
    lib.mpt_float_quantize_nearest.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64] + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    assert lib.mpt_float_quantize_nearest(None, None, 0, 2, 5, 1, 0, None) == 0          # empty input: nothing to do
    assert lib.mpt_float_quantize_nearest(None, None, 16, 2, 5, 1, 0, None) == 1         # null pointers
    assert b"null pointer" in lib.mpt_last_error()
    assert lib.mpt_float_quantize_nearest(None, None, 0, 30, 5, 1, 0, None) == 1         # bad format
    assert b"unsupported format" in lib.mpt_last_error()
    lib.mpt_mm_workspace_bytes.restype = ctypes.c_size_t
    lib.mpt_mm_workspace_bytes.argtypes = [ctypes.c_int64]
    assert lib.mpt_mm_workspace_bytes(1) == 256 and lib.mpt_mm_workspace_bytes(96) == 1536
