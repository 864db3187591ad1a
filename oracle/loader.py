"""ctypes front end of the CPU oracle (``oracle/mpt_oracle.c``).

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The
shipped package never imports this module.

All array arguments are C-contiguous numpy arrays (float32 unless stated);
results are new numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libmpt_oracle.so")

_lib = None

POLICY = {"saturate_infty": 0, "saturate_maxfloat": 1, "saturate_maxfloat2": 2}
MODE = {"nearest": 0, "stochastic": 1, "truncate": 2}
ORDER = {"seq": 0, "tile8": 1, "tree64": 1}


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (a second or two) if it is not built yet."""
    src = os.path.join(HERE, "mpt_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", HERE], stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        f32, i32, i64, u32, u64, p = C.c_float, C.c_int, C.c_int64, C.c_uint32, C.c_uint64, C.c_void_p
        L.orc_cast_fp_nearest.restype = f32
        L.orc_cast_fp_nearest.argtypes = [f32, i32, i32, i32, i32]
        L.orc_cast_fp_truncate.restype = f32
        L.orc_cast_fp_truncate.argtypes = [f32, i32, i32, i32, i32]
        L.orc_cast_fp_stochastic.restype = f32
        L.orc_cast_fp_stochastic.argtypes = [f32, u32, i32, i32, i32, i32, i32]
        L.orc_cast_binary8.restype = f32
        L.orc_cast_binary8.argtypes = [f32, i32, i32, i32, i32, i32, u32, i32]
        L.orc_cast_superfp.restype = f32
        L.orc_cast_superfp.argtypes = [f32, i32, i32, i32, i32, i32]
        L.orc_float_quantize.argtypes = [p, p, i64, i32, i32, i32, i32, i32, p, i32]
        L.orc_binary8_quantize.argtypes = [p, p, i64, i32, i32, i32, i32, i32, p, i32]
        L.orc_superfp_quantize.argtypes = [p, p, i64, i32, i32, i32, i32, i32]
        L.orc_philox.argtypes = [u32, u32, u32, u32, u32, u32, p]
        L.orc_mm.argtypes = [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32]
        L.orc_mm_sr.argtypes = [p, p, p, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, u64]
        L.orc_softmax_forward.argtypes = [p, p, i64, i32, i64] + [i32] * 9
        L.orc_softmax_lse_forward.argtypes = [p, p, i64, i32, i64] + [i32] * 7
        L.orc_softmax_backward.argtypes = [p, p, p, i64, i32, i64] + [i32] * 7
        L.orc_layernorm_forward.argtypes = [p, p, p, p, p, p, f32, i64, i32, i64] + [i32] * 11
        L.orc_layernorm_backward.argtypes = [p] * 8 + [i64, i32, i64] + [i32] * 9
        L.orc_mm_fmt.argtypes = [p, p, p, i64, i32, i32, i32, p, p, i32, i32]
        L.orc_softmax_forward_fmt.argtypes = [p, p, i64, i32, i64, p, p, p, i32]
        L.orc_softmax_lse_forward_fmt.argtypes = [p, p, i64, i32, i64, p, p, i32]
        L.orc_softmax_backward_fmt.argtypes = [p, p, p, i64, i32, i64, p, p, i32]
        L.orc_layernorm_forward_fmt.argtypes = [p, p, p, p, p, p, f32, i64, i32, i64, p, p, p, p, i32]
        L.orc_layernorm_backward_fmt.argtypes = [p] * 8 + [i64, i32, i64, p, p, p, i32]
        L.orc_mx_quantize.argtypes = [p, p, p, i64, i64, i32, i32]
        L.orc_nvfp4_quantize.restype = f32
        L.orc_nvfp4_quantize.argtypes = [p, p, p, i64, i64, f32]
        L.orc_qsum_rows.argtypes = [p, p, i64, i64, i32, i32, i32, i32]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def float_quantize(a, man, exp, rounding="nearest", subnormals=True, saturate=True, rand=None, rbits=0):
    a = _f32(a)
    o = np.empty_like(a)
    r = None if rand is None else np.ascontiguousarray(rand, dtype=np.int32)
    lib().orc_float_quantize(_ptr(a), _ptr(o), a.size, man, exp, int(subnormals), int(saturate),
                             MODE[rounding], _ptr(r), rbits)
    return o


def binary8_quantize(a, P, rounding="nearest", overflow_policy="saturate_maxfloat", is_signed=True,
                     subnormals=True, rand=None, prng_bits=0):
    a = _f32(a)
    o = np.empty_like(a)
    r = None if rand is None else np.ascontiguousarray(rand, dtype=np.int32)
    lib().orc_binary8_quantize(_ptr(a), _ptr(o), a.size, P, int(is_signed), POLICY[overflow_policy],
                               int(subnormals), MODE[rounding], _ptr(r), prng_bits)
    return o


def superfp_quantize(a, man, exp, binades_l=1, binades_u=1, saturate=False):
    a = _f32(a)
    o = np.empty_like(a)
    lib().orc_superfp_quantize(_ptr(a), _ptr(o), a.size, man, exp, binades_l, binades_u, int(saturate))
    return o


def philox(c0, c1, c2, c3, k0, k1):
    out = np.zeros(4, dtype=np.uint32)
    lib().orc_philox(c0, c1, c2, c3, k0, k1, _ptr(out))
    return out


def mm(a, b, man_add, exp_add, man_mul, exp_mul, subnormals=True, saturate=False, fma=False,
       order="seq", compensated=False):
    """a: [M,K] or [B,M,K]; b: [K,N] or [B,K,N]."""
    a, b = _f32(a), _f32(b)
    batched = a.ndim == 3
    B = a.shape[0] if batched else 1
    M, K = a.shape[-2:]
    N = b.shape[-1]
    c = np.zeros((B, M, N) if batched else (M, N), dtype=np.float32)
    lib().orc_mm(_ptr(a), _ptr(b), _ptr(c), B, M, K, N, man_add, exp_add, man_mul, exp_mul,
                 int(subnormals), int(saturate), int(fma), ORDER[order], int(compensated))
    return c


def mm_sr(a, b, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals=True, saturate=False,
          fma=False, seed=0):
    a, b = _f32(a), _f32(b)
    batched = a.ndim == 3
    B = a.shape[0] if batched else 1
    M, K = a.shape[-2:]
    N = b.shape[-1]
    c = np.zeros((B, M, N) if batched else (M, N), dtype=np.float32)
    lib().orc_mm_sr(_ptr(a), _ptr(b), _ptr(c), B, M, K, N, man_add, exp_add, rbits_add, man_mul, exp_mul,
                    rbits_mul, int(subnormals), int(saturate), int(fma), seed)
    return c


def partition(shape, dim):
    """(outer, channel, inner) for a reduction over `dim` (an int) or contiguous `dims` (a list).
    reference: quant_cpu/sim_helper.cpp:28-67."""
    nd = len(shape)
    dims = [dim] if isinstance(dim, int) else list(dim)
    real = [(nd + (d % nd)) % nd for d in dims]
    channel = 1
    for d in real:
        channel *= shape[d]
    lo, hi = (real[0], real[0]) if isinstance(dim, int) else (real[-1], real[0])
    outer = int(np.prod(shape[:lo], dtype=np.int64))
    inner = int(np.prod(shape[hi + 1:], dtype=np.int64))
    if outer * channel * inner != int(np.prod(shape, dtype=np.int64)):
        raise ValueError("dims %r must be adjacent dimensions listed last-first of shape %r" % (dim, tuple(shape)))
    return outer, channel, inner


def softmax_forward(a, dim, man_exp, exp_exp, man_off, exp_off, man_acc, exp_acc, subnormals=True,
                    saturate=False, order="seq"):
    a = _f32(a)
    o = np.zeros_like(a)
    outer, ch, inner = partition(a.shape, dim)
    lib().orc_softmax_forward(_ptr(a), _ptr(o), outer, ch, inner, man_exp, exp_exp, man_off, exp_off,
                              man_acc, exp_acc, int(subnormals), int(saturate), ORDER[order])
    return o


def softmax_lse_forward(a, dim, man_off, exp_off, man_lse, exp_lse, subnormals=True, saturate=False,
                        order="seq"):
    a = _f32(a)
    o = np.zeros_like(a)
    outer, ch, inner = partition(a.shape, dim)
    lib().orc_softmax_lse_forward(_ptr(a), _ptr(o), outer, ch, inner, man_off, exp_off, man_lse, exp_lse,
                                  int(subnormals), int(saturate), ORDER[order])
    return o


def softmax_backward(y, g, dim, man_add, exp_add, man_mul, exp_mul, subnormals=True, saturate=False,
                     order="seq"):
    y, g = _f32(y), _f32(g)
    o = np.zeros_like(y)
    outer, ch, inner = partition(y.shape, dim)
    lib().orc_softmax_backward(_ptr(y), _ptr(g), _ptr(o), outer, ch, inner, man_add, exp_add, man_mul,
                               exp_mul, int(subnormals), int(saturate), ORDER[order])
    return o


def layernorm_forward(x, w, b, eps, dims, man_acc, exp_acc, man_mul, exp_mul, man_div, exp_div,
                      man_sqrt, exp_sqrt, subnormals=True, saturate=False, order="seq"):
    x, w, b = _f32(x), _f32(w), _f32(b)
    outer, ch, inner = partition(x.shape, dims)
    y = np.zeros_like(x)
    mean = np.zeros(outer * inner, dtype=np.float32)
    rstd = np.zeros(outer * inner, dtype=np.float32)
    lib().orc_layernorm_forward(_ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), eps,
                                outer, ch, inner, man_acc, exp_acc, man_mul, exp_mul, man_div, exp_div,
                                man_sqrt, exp_sqrt, int(subnormals), int(saturate), ORDER[order])
    return y, mean, rstd


def layernorm_backward(x, g, w, mean, rstd, dims, man_acc, exp_acc, man_mul, exp_mul, man_div, exp_div,
                       subnormals=True, saturate=False, order="seq"):
    x, g, w, mean, rstd = _f32(x), _f32(g), _f32(w), _f32(mean), _f32(rstd)
    outer, ch, inner = partition(x.shape, dims)
    gin = np.zeros_like(x)
    gg = np.zeros(ch, dtype=np.float32)
    gb = np.zeros(ch, dtype=np.float32)
    lib().orc_layernorm_backward(_ptr(x), _ptr(g), _ptr(w), _ptr(mean), _ptr(rstd), _ptr(gin), _ptr(gg),
                                 _ptr(gb), outer, ch, inner, man_acc, exp_acc, man_mul, exp_mul, man_div,
                                 exp_div, int(subnormals), int(saturate), ORDER[order])
    return gin, gg, gb


def mx_quantize(x, elem="e4m3", block=32, return_codes=False):
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    cols = x.shape[-1]
    o = np.empty_like(x)
    sc = np.zeros((rows, (cols + block - 1) // block), dtype=np.uint8)
    kind = {"e4m3": 0, "e2m1": 1}[elem]
    if not return_codes:
        lib().orc_mx_quantize(_ptr(x), _ptr(o), _ptr(sc), rows, cols, block, kind)
        return o, sc.reshape(x.shape[:-1] + (sc.shape[1],))
    width = cols if kind == 0 else (cols + 1) // 2
    codes = np.zeros((rows, width), dtype=np.uint8)
    L = lib()
    L.orc_mx_quantize_codes.restype = None
    L.orc_mx_quantize_codes.argtypes = [C.c_void_p] * 4 + [C.c_int64, C.c_int64, C.c_int, C.c_int]
    L.orc_mx_quantize_codes(_ptr(x), _ptr(o), _ptr(sc), _ptr(codes), rows, cols, block, kind)
    return o, sc.reshape(x.shape[:-1] + (sc.shape[1],)), codes.reshape(x.shape[:-1] + (width,))


def nvfp4_quantize(x, global_scale=0.0, return_codes=False):
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    cols = x.shape[-1]
    o = np.empty_like(x)
    sc = np.zeros((rows, (cols + 15) // 16), dtype=np.float32)
    if not return_codes:
        sg = lib().orc_nvfp4_quantize(_ptr(x), _ptr(o), _ptr(sc), rows, cols, float(global_scale))
        return o, sc.reshape(x.shape[:-1] + (sc.shape[1],)), sg
    codes = np.zeros((rows, (cols + 1) // 2), dtype=np.uint8)
    scodes = np.zeros_like(sc, dtype=np.uint8)
    L = lib()
    L.orc_nvfp4_quantize_codes.restype = C.c_float
    L.orc_nvfp4_quantize_codes.argtypes = [C.c_void_p] * 5 + [C.c_int64, C.c_int64, C.c_float]
    sg = L.orc_nvfp4_quantize_codes(_ptr(x), _ptr(o), _ptr(sc), _ptr(codes), _ptr(scodes), rows, cols, float(global_scale))
    lead = x.shape[:-1]
    return o, sc.reshape(lead + (sc.shape[1],)), sg, codes.reshape(lead + (codes.shape[1],)), scodes.reshape(lead + (sc.shape[1],))


def qsum_rows(x, man, exp, subnormals=True, saturate=False):
    x = _f32(x)
    o = np.zeros(x.shape[1], dtype=np.float32)
    lib().orc_qsum_rows(_ptr(x), _ptr(o), x.shape[0], x.shape[1], man, exp, int(subnormals), int(saturate))
    return o


# ---------------------------------------------------------------------------------- generic formats
# A format descriptor is an int32[8]: {kind, man, exp, subnormals, saturate, a, b, c}.
def fmt_float(man, exp, subnormals=True, saturate=False):
    return np.array([0, man, exp, int(subnormals), int(saturate), 0, 0, 0], dtype=np.int32)


def fmt_superfp(man, exp, binades_l=1, binades_u=1, saturate=False):
    return np.array([1, man, exp, 0, int(saturate), binades_l, binades_u, 0], dtype=np.int32)


def fmt_binary8(P, is_signed=True, overflow_policy="saturate_maxfloat", subnormals=True):
    pol = POLICY[overflow_policy] if isinstance(overflow_policy, str) else int(overflow_policy)
    return np.array([2, 0, 0, int(subnormals), 0, P, int(is_signed), pol], dtype=np.int32)


def mm_fmt(a, b, fadd, fmul, fma=False, order="seq"):
    a, b = _f32(a), _f32(b)
    batched = a.ndim == 3
    B = a.shape[0] if batched else 1
    M, K = a.shape[-2:]
    N = b.shape[-1]
    c = np.zeros((B, M, N) if batched else (M, N), dtype=np.float32)
    lib().orc_mm_fmt(_ptr(a), _ptr(b), _ptr(c), B, M, K, N, _ptr(fadd), _ptr(fmul), int(fma), ORDER[order])
    return c


def softmax_forward_fmt(a, dim, fexp, foff, facc, order="seq"):
    a = _f32(a)
    o = np.zeros_like(a)
    outer, ch, inner = partition(a.shape, dim)
    lib().orc_softmax_forward_fmt(_ptr(a), _ptr(o), outer, ch, inner, _ptr(fexp), _ptr(foff), _ptr(facc), ORDER[order])
    return o


def softmax_lse_forward_fmt(a, dim, foff, flse, order="seq"):
    a = _f32(a)
    o = np.zeros_like(a)
    outer, ch, inner = partition(a.shape, dim)
    lib().orc_softmax_lse_forward_fmt(_ptr(a), _ptr(o), outer, ch, inner, _ptr(foff), _ptr(flse), ORDER[order])
    return o


def softmax_backward_fmt(y, g, dim, fadd, fmul, order="seq"):
    y, g = _f32(y), _f32(g)
    o = np.zeros_like(y)
    outer, ch, inner = partition(y.shape, dim)
    lib().orc_softmax_backward_fmt(_ptr(y), _ptr(g), _ptr(o), outer, ch, inner, _ptr(fadd), _ptr(fmul), ORDER[order])
    return o


def layernorm_forward_fmt(x, w, b, eps, dims, facc, fmul, fdiv, fsqrt, order="seq"):
    x, w, b = _f32(x), _f32(w), _f32(b)
    outer, ch, inner = partition(x.shape, dims)
    y = np.zeros_like(x)
    mean = np.zeros(outer * inner, dtype=np.float32)
    rstd = np.zeros(outer * inner, dtype=np.float32)
    lib().orc_layernorm_forward_fmt(_ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), eps, outer, ch, inner,
                                    _ptr(facc), _ptr(fmul), _ptr(fdiv), _ptr(fsqrt), ORDER[order])
    return y, mean, rstd


def layernorm_backward_fmt(x, g, w, mean, rstd, dims, facc, fmul, fdiv, order="seq"):
    x, g, w, mean, rstd = _f32(x), _f32(g), _f32(w), _f32(mean), _f32(rstd)
    outer, ch, inner = partition(x.shape, dims)
    gin = np.zeros_like(x)
    gg = np.zeros(ch, dtype=np.float32)
    gb = np.zeros(ch, dtype=np.float32)
    lib().orc_layernorm_backward_fmt(_ptr(x), _ptr(g), _ptr(w), _ptr(mean), _ptr(rstd), _ptr(gin), _ptr(gg), _ptr(gb), outer, ch,
                                     inner, _ptr(facc), _ptr(fmul), _ptr(fdiv), ORDER[order])
    return gin, gg, gb
