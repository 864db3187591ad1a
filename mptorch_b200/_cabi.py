"""ctypes binding of the C ABI declared in ``include/mptorch_b200.h``.

This is the only place the Python package touches the native library.  There is no fallback:
if the library has not been built (``python -m mptorch_b200.build``) or a call fails, an
exception is raised.  Tensors are torch CUDA tensors; torch is used for device memory and the
current stream only.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmptorch_b200.so")

_lib = None


class MptError(RuntimeError):
    pass


class Format(C.Structure):
    """``mpt_format`` of include/mptorch_b200.h: one descriptor for float, supernormal-float and binary8 rounding."""
    _fields_ = [("kind", C.c_int), ("man", C.c_int), ("exp", C.c_int), ("subnormals", C.c_int), ("saturate", C.c_int),
                ("binades_l", C.c_int), ("binades_u", C.c_int), ("P", C.c_int), ("is_signed", C.c_int),
                ("overflow_policy", C.c_int)]

    @staticmethod
    def float(man, exp, subnormals=True, saturate=False):
        return Format(0, man, exp, int(subnormals), int(saturate), 1, 1, 1, 1, 0)

    @staticmethod
    def superfp(man, exp, binades_l=1, binades_u=1, saturate=False):
        return Format(1, man, exp, 1, int(saturate), binades_l, binades_u, 1, 1, 0)

    @staticmethod
    def binary8(P, is_signed=True, overflow_policy=1, subnormals=True):
        return Format(2, 0, 0, int(subnormals), 0, 1, 1, P, int(is_signed), int(overflow_policy))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MptError(
                "the CUDA library %s is missing; build it with `python -m mptorch_b200.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        p, i32, i64, u64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_size_t
        L.mpt_last_error.restype = C.c_char_p
        L.mpt_version.restype = i32
        L.mpt_mm_workspace_bytes.restype = sz
        L.mpt_mm_workspace_bytes.argtypes = [i64]
        L.mpt_scale_quantize_workspace_bytes.restype = sz
        L.mpt_scale_quantize_workspace_bytes.argtypes = [i64]
        sig = {
            "mpt_float_quantize_nearest": [p, p, i64, i32, i32, i32, i32, p],
            "mpt_float_quantize_truncate": [p, p, i64, i32, i32, i32, i32, p],
            "mpt_float_quantize_stochastic": [p, p, p, i64, i32, i32, i32, i32, i32, p],
            "mpt_float_quantize_stochastic_philox": [p, p, i64, i32, i32, i32, i32, i32, u64, p],
            "mpt_float_quantize_multi": [p, p, p, i32, i32, i32, i32, i32, i32, i32, u64, p],
            "mpt_binary8_quantize": [p, p, p, i64, i32, i32, i32, i32, i32, i32, p],
            "mpt_superfp_quantize_nearest": [p, p, i64, i32, i32, i32, i32, i32, p],
            "mpt_float_mm_nearest": [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, p, sz, p],
            "mpt_float_conv2d_nearest": [p, p, p] + [i32] * 22 + [p, sz, p],
            "mpt_float_conv2d_wgrad_nearest": [p, p, p] + [i32] * 22 + [p, sz, p],
            "mpt_float_mm_nearest_static": [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, p],
            "mpt_float_mm_nearest_piece": [p, p, p, i64] + [i32] * 12 + [p, sz, p],
            "mpt_copy_columns_async": [p, sz, p, sz, sz, sz, p],
            "mpt_transpose_last2": [p, p, i64, i64, i64, p],
            "mpt_float_mm_nearest_fma": [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, p, sz, p],
            "mpt_float_mm_stochastic": [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, u64, p, sz, p],
            "mpt_float_softmax_forward": [p, p, i64, i32, i64] + [i32] * 9 + [p],
            "mpt_float_softmax_lse_forward": [p, p, i64, i32, i64] + [i32] * 7 + [p],
            "mpt_float_softmax_backward": [p, p, p, i64, i32, i64] + [i32] * 7 + [p],
            "mpt_float_layernorm_forward": [p] * 6 + [C.c_float, i64, i32, i64] + [i32] * 11 + [p],
            "mpt_float_layernorm_backward": [p] * 8 + [i64, i32, i64] + [i32] * 9 + [p],
            "mpt_qsum_rows": [p, p, i64, i64, i32, i32, i32, i32, p],
            "mpt_mm_nearest_fmt": [p, p, p, i64, i32, i32, i32, p, p, i32, i32, p, sz, p],
            "mpt_softmax_forward_fmt": [p, p, i64, i32, i64, p, p, p, i32, p],
            "mpt_softmax_lse_forward_fmt": [p, p, i64, i32, i64, p, p, i32, p],
            "mpt_softmax_backward_fmt": [p, p, p, i64, i32, i64, p, p, i32, p],
            "mpt_layernorm_forward_fmt": [p] * 6 + [C.c_float, i64, i32, i64, p, p, p, p, i32, p],
            "mpt_layernorm_backward_fmt": [p] * 8 + [i64, i32, i64, p, p, p, i32, p],
            "mpt_stream_priority_range": [p, p],
            "mpt_qsgd_step": [p, i32, C.c_float, C.c_float, C.c_float, C.c_float] + [i32] * 10 + [p],
            "mpt_qadamw_step": [p, i32] + [C.c_float] * 7 + [i32] * 10 + [p],
            "mpt_scale_quantize": [p, p, i64, i64, C.c_double, i32, i32, i32, i32, i32, i32, p, p, sz, p],
            "mpt_mx_quantize": [p, p, p, p, i64, i64, i32, i32, p],
            "mpt_nvfp4_quantize": [p, p, p, p, p, i64, i64, C.c_float, p, p, p],
        }
        for name, args in sig.items():
            fn = getattr(L, name, None)
            if fn is None:
                continue
            fn.restype = i32
            fn.argtypes = args
        _lib = L
    return _lib


def call(name: str, *args) -> None:
    fn = getattr(lib(), name)
    rc = fn(*args)
    if rc != 0:
        raise MptError("%s failed (code %d): %s" % (name, rc, lib().mpt_last_error().decode()))


def check_cuda_f32(t: torch.Tensor, what: str) -> None:
    """Mirrors the reference's CHECK_INPUT (quant_cuda/pybind_cuda.cpp:8-13) plus a dtype check."""
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % what)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % what)
    if t.dtype != torch.float32:
        raise RuntimeError("%s must be float32" % what)


def ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device: torch.device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def mm_workspace(device: torch.device, batch: int = 1) -> torch.Tensor:
    """A small per-(device, stream) scratch buffer for the GEMM's operand statistics (grown on demand)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    need = int(lib().mpt_mm_workspace_bytes(max(int(batch), 1)))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws
