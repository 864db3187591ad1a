"""Builds and loads ``quant_b200``: a PyTorch C++ extension with the reference's ``quant_cuda`` interface that
forwards to the C ABI (``quant_b200.cpp``).  The extension is built in-tree with ``torch.utils.cpp_extension``
and links against ``mptorch_b200/lib/libmptorch_b200.so``.

    from mptorch_b200.torch_ext import load
    quant_b200 = load()            # builds on first use (about a minute), then imports the cached .so
"""
from __future__ import annotations

import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
_BUILD = os.path.join(_PKG, "lib", "quant_b200")
_SO = os.path.join(_BUILD, "quant_b200.so")


def _preload_kernels() -> None:
    """The extension resolves the mpt_* symbols from libmptorch_b200.so; load it first, globally."""
    import ctypes

    from .._cabi import LIB_PATH

    ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)


def build(verbose: bool = False) -> str:
    from torch.utils.cpp_extension import load as _load

    from .. import build as libbuild

    libbuild.build()
    _preload_kernels()
    os.makedirs(_BUILD, exist_ok=True)
    libdir = os.path.join(_PKG, "lib")
    _load(name="quant_b200", sources=[os.path.join(_HERE, "quant_b200.cpp")],
          extra_include_paths=[os.path.join(_PKG, "..", "include")],
          extra_ldflags=["-L" + libdir, "-lmptorch_b200"],
          build_directory=_BUILD, with_cuda=True, is_python_module=False, verbose=verbose)
    return _SO


def available() -> bool:
    """True when the extension has been built and is not older than its source."""
    src = os.path.join(_HERE, "quant_b200.cpp")
    return os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(src)


def load(build_if_missing: bool = True):
    src = os.path.join(_HERE, "quant_b200.cpp")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        if not build_if_missing:
            raise RuntimeError("quant_b200 is not built; call mptorch_b200.torch_ext.build()")
        build()
    import torch  # noqa: F401

    _preload_kernels()
    spec = importlib.util.spec_from_file_location("quant_b200", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
