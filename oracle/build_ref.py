"""Build the UNMODIFIED reference extensions into ``oracle/_ref/``.

Test infrastructure only.  The reference (mptorch) JIT-compiles two pybind11
extensions from its own source tree with ``torch.utils.cpp_extension.load``
(reference ``mptorch/quant/quant_function.py:57-92``).  This recipe runs the
same call on the same source files, where they lie in the mounted reference
tree, and only redirects the build directory so the resulting shared objects
land in ``oracle/_ref/``:

* ``quant_cpu.so``  -- the reference CPU path; the checker the C restatement
  in ``oracle/mpt_oracle.c`` is pinned against, and the timed CPU baseline.
* ``quant_cuda.so`` -- the reference CUDA path compiled for sm_100a
  (optional, ``--cuda``); can only be *run* where a GPU is present.

No reference source is copied.  If the reference tree is absent (as on a GPU
machine) nothing is built and already-built objects are used as they are.

Usage:  python oracle/build_ref.py [--cuda] [--ref /path/to/reference]
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

CPU_SOURCES = ["pybind_cpu.cpp", "binary8.cpp", "quant.cpp", "sim_helper.cpp", "bit_helper.cpp"]
CUDA_SOURCES = [
    "pybind_cuda.cpp", "bit_helper.cu", "sim_helper.cu", "block_kernel.cu", "fp_kernel.cu",
    "fxp_kernel.cu", "superfp_kernel.cu", "quant.cu", "binary8_kernel.cu", "cublas_helper.cpp",
]


def _so_path(name: str) -> str:
    return os.path.join(OUT, name, name + ".so")


def build_cpu(ref_root: str, verbose: bool = False) -> str:
    from torch.utils.cpp_extension import load

    src = os.path.join(ref_root, "mptorch", "quant", "quant_cpu")
    bdir = os.path.join(OUT, "quant_cpu")
    os.makedirs(bdir, exist_ok=True)
    load(
        name="quant_cpu",
        sources=[os.path.join(src, s) for s in CPU_SOURCES],
        extra_cflags=["-fopenmp"],
        build_directory=bdir,
        verbose=verbose,
        is_python_module=False,
    )
    return _so_path("quant_cpu")


def build_cuda(ref_root: str, verbose: bool = False) -> str:
    from torch.utils.cpp_extension import load

    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    src = os.path.join(ref_root, "mptorch", "quant", "quant_cuda")
    bdir = os.path.join(OUT, "quant_cuda")
    os.makedirs(bdir, exist_ok=True)
    load(
        name="quant_cuda",
        sources=[os.path.join(src, s) for s in CUDA_SOURCES],
        extra_cuda_cflags=["--extended-lambda"],
        build_directory=bdir,
        verbose=verbose,
        is_python_module=False,
        with_cuda=True,
    )
    return _so_path("quant_cuda")


def load_ref(name: str = "quant_cpu"):
    """Import an already-built reference extension from ``oracle/_ref``; None if absent."""
    path = _so_path(name)
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--ref", default=os.environ.get("MPT_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(here)), "reference"),
                    help="root of the reference checkout (default: $MPT_REFERENCE_ROOT, else a sibling directory `reference`)")
    ap.add_argument("--cuda", action="store_true", help="also build quant_cuda for sm_100a")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args(argv)
    if not os.path.isdir(os.path.join(args.ref, "mptorch", "quant", "quant_cpu")):
        print("reference tree not found at %s; nothing built" % args.ref)
        return 0
    print("built", build_cpu(args.ref, args.verbose))
    if args.cuda:
        print("built", build_cuda(args.ref, args.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
