"""pytest configuration: the ``gpu`` marker, and shared helpers for the oracle and fixtures."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import loader

    loader.lib()
    return loader


@pytest.fixture(scope="session")
def ref_cpu():
    """The compiled, unmodified reference CPU extension, when it has been built (oracle/_ref)."""
    from oracle.build_ref import load_ref

    mod = load_ref("quant_cpu")
    if mod is None:
        pytest.skip("oracle/_ref/quant_cpu not built")
    return mod


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def same_bits(a, b):
    """Bitwise equality of two float32 arrays, all NaN payloads counted as equal."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if a.shape != b.shape:
        return False
    ab, bb = a.view(np.uint32), b.view(np.uint32)
    return bool(np.all((ab == bb) | (np.isnan(a) & np.isnan(b))))


def mismatch_report(a, b, limit=5):
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    b = np.ascontiguousarray(b, dtype=np.float32).ravel()
    bad = np.nonzero((a.view(np.uint32) != b.view(np.uint32)) & ~(np.isnan(a) & np.isnan(b)))[0]
    head = ", ".join(f"[{i}] {a[i]!r}({a.view(np.uint32)[i]:#010x}) != {b[i]!r}({b.view(np.uint32)[i]:#010x})" for i in bad[:limit])
    return f"{bad.size} of {a.size} differ: {head}"
