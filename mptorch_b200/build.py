"""Builds the sm_100a CUDA library (``mptorch_b200/lib/libmptorch_b200.so``) in-tree with nvcc.

    python -m mptorch_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is installed.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libmptorch_b200.so")
OBJDIR = os.path.join(PKG, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Wno-deprecated-gpu-targets", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]
# Every fp32 multiply/add of the algorithms is written with an explicit rounding intrinsic, which the
# compiler never contracts.  -fmad=false additionally keeps it from contracting the few plain
# expressions that remain.  reduce.cu is the exception: it calls expf/logf, and those must compile
# exactly as they do in the reference's CUDA build (nvcc defaults) to give the same bits.
EXTRA_FLAGS = {"reduce.cu": [], "rows_softmax_fwd.cu": [], "rows_softmax_bwd.cu": [], "rows_softmax_lse.cu": [], "rows_layernorm_fwd.cu": [],
               "rows_layernorm_bwd.cu": []}
DEFAULT_EXTRA = ["-fmad=false"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _includes(path: str, seen: set[str]) -> set[str]:
    """Local headers a source file pulls in, transitively (`#include "..."` relative to csrc/ or include/)."""
    import re

    for name in re.findall(r'^\s*#include\s+"([^"]+)"', open(path).read(), flags=re.M):
        for base in (CSRC, os.path.join(PKG, "..", "include")):
            cand = os.path.normpath(os.path.join(base, name))
            if os.path.exists(cand) and cand not in seen:
                seen.add(cand)
                _includes(cand, seen)
    return seen


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + sorted(_includes(src, set()))):
            extra = EXTRA_FLAGS.get(os.path.basename(src), DEFAULT_EXTRA)
            cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out)
        if pr.returncode:
            raise RuntimeError("nvcc failed on %s" % src)
    if force or procs or _stale(LIB, objs):
        # the CUDA runtime is linked statically (nvcc's default), so the library does not depend on
        # which libcudart the host process happens to have loaded
        cmd = [_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-Xlinker", "-soname=libmptorch_b200.so", "-o", LIB] + objs
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
