"""Host-side mirror of the reference's ``quant_cuda`` extension module.

Function names, argument order and argument meaning follow the pybind registrations in the
reference's ``mptorch/quant/quant_cuda/pybind_cuda.cpp`` (line numbers cited per function), so
``mptorch_b200.quant.quant_function`` can call this module exactly where the reference calls
``quant_cuda``.  Each function checks its tensors the way the reference's ``CHECK_INPUT`` does,
allocates outputs, and forwards to the C ABI on the current CUDA stream.

Two knobs exist that the reference does not have, because its CPU and CUDA back ends disagree:

``accum_order``  "cuda" (default) reproduces the CUDA kernels' 8-wide tiled K accumulation,
                 "seq" the CPU path's strictly sequential accumulation;
``reduce_order`` same choice for the softmax / layernorm row reductions.
"""
from __future__ import annotations

import contextlib
import enum

import torch

from . import _cabi
from ._cabi import call, check_cuda_f32, ptr, stream_ptr

INT_MAX = 2147483647


class OverflowPolicy(enum.IntEnum):
    """reference: quant_cuda/binary8_kernel.h:20-25, pybind_cuda.cpp:784-787."""
    SATURATE_INFTY = 0
    SATURATE_MAXFLOAT = 1
    SATURATE_MAXFLOAT2 = 2


_ORDER = {"seq": 0, "cuda": 1, "tile8": 1, "tree64": 1}
_state = {"accum_order": "cuda", "reduce_order": "cuda"}

# Two routes lead from here to the C ABI: the PyTorch C++ extension `quant_b200` (mptorch_b200/torch_ext, the reference's
# quant_cuda interface over the C ABI, a few microseconds less host time per call) when it has been built, and ctypes
# otherwise.  Both call the same entry points of the same library.  MPT_BACKEND=ctypes (or =ext) forces one.
_ext = None


def _load_ext():
    import os

    global _ext
    want = os.environ.get("MPT_BACKEND", "")
    if want == "ctypes":
        return
    try:
        from . import torch_ext

        if want == "ext" or torch_ext.available():
            _ext = torch_ext.load(build_if_missing=(want == "ext"))
    except Exception:
        if want == "ext":
            raise
        _ext = None


_load_ext()


def route() -> str:
    """Which host layer the hot entry points go through: "ext" (the C++ extension) or "ctypes"."""
    return "ext" if _ext is not None else "ctypes"


def set_accum_order(order: str) -> None:
    if order not in _ORDER:
        raise ValueError("accum_order must be 'cuda' or 'seq'")
    _state["accum_order"] = order
    if _ext is not None:
        _ext.set_accum_order("seq" if _ORDER[order] == 0 else "cuda")


def set_reduce_order(order: str) -> None:
    if order not in _ORDER:
        raise ValueError("reduce_order must be 'cuda' or 'seq'")
    _state["reduce_order"] = order
    if _ext is not None:
        _ext.set_reduce_order("seq" if _ORDER[order] == 0 else "cuda")


def get_accum_order() -> str:
    return _state["accum_order"]


def get_reduce_order() -> str:
    return _state["reduce_order"]


@contextlib.contextmanager
def orders(accum: str | None = None, reduce: str | None = None):
    """Temporarily select accumulation / reduction orders."""
    old = dict(_state)
    try:
        if accum is not None:
            set_accum_order(accum)
        if reduce is not None:
            set_reduce_order(reduce)
        yield
    finally:
        set_accum_order(old["accum_order"])
        set_reduce_order(old["reduce_order"])


def _order_code(order: str | None, kind: str) -> int:
    return _ORDER[_state[kind] if order is None else order]


# ---------------------------------------------------------------------------------- quantizers
def float_quantize_nearest(a, man_bits, exp_bits, subnormals, saturate):
    """pybind_cuda.cpp:44."""
    if _ext is not None:
        return _ext.float_quantize_nearest(a, man_bits, exp_bits, subnormals, saturate)
    check_cuda_f32(a, "a")
    o = torch.empty_like(a)
    with torch.cuda.device(a.device):
        call("mpt_float_quantize_nearest", ptr(a), ptr(o), a.numel(), man_bits, exp_bits, int(subnormals),
             int(saturate), stream_ptr(a.device))
    return o


def float_quantize_truncate(a, man_bits, exp_bits, subnormals, saturate):
    """New: no counterpart in the reference."""
    check_cuda_f32(a, "a")
    o = torch.empty_like(a)
    with torch.cuda.device(a.device):
        call("mpt_float_quantize_truncate", ptr(a), ptr(o), a.numel(), man_bits, exp_bits, int(subnormals),
             int(saturate), stream_ptr(a.device))
    return o


def float_quantize_stochastic(a, man_bits, exp_bits, prng_bits, subnormals, saturate, rand=None, seed=None):
    """pybind_cuda.cpp:98.  By default the random words are drawn exactly as the reference draws them
    (``randint_like(a, INT_MAX)`` from the torch CUDA generator, quant_cuda/quant.cu:132), so results
    match the reference under the same ``torch.manual_seed``.  ``rand`` supplies the words explicitly;
    ``seed`` switches to the in-kernel Philox generator (no random-word tensor at all)."""
    check_cuda_f32(a, "a")
    o = torch.empty_like(a)
    with torch.cuda.device(a.device):
        if seed is not None:
            call("mpt_float_quantize_stochastic_philox", ptr(a), ptr(o), a.numel(), man_bits, exp_bits, prng_bits,
                 int(subnormals), int(saturate), int(seed) & (2**64 - 1), stream_ptr(a.device))
        else:
            if rand is None:
                rand = torch.randint_like(a, INT_MAX, dtype=torch.int32)
            if not (rand.is_cuda and rand.is_contiguous() and rand.dtype == torch.int32 and rand.numel() == a.numel()):
                raise RuntimeError("rand must be a contiguous CUDA int32 tensor with one word per element")
            call("mpt_float_quantize_stochastic", ptr(a), ptr(rand), ptr(o), a.numel(), man_bits, exp_bits, prng_bits,
                 int(subnormals), int(saturate), stream_ptr(a.device))
    return o


def _binary8(a, P, is_signed, overflow_policy, subnormals, rounding, prng_bits=0, rand=None):
    check_cuda_f32(a, "a")
    o = torch.empty_like(a)
    with torch.cuda.device(a.device):
        if rounding == 1:
            if rand is None:
                rand = torch.randint_like(a, INT_MAX, dtype=torch.int32)
            if not (rand.is_cuda and rand.is_contiguous() and rand.dtype == torch.int32 and rand.numel() == a.numel()):
                raise RuntimeError("rand must be a contiguous CUDA int32 tensor with one word per element")
        call("mpt_binary8_quantize", ptr(a), ptr(rand), ptr(o), a.numel(), P, int(is_signed), int(overflow_policy),
             int(subnormals), rounding, prng_bits, stream_ptr(a.device))
    return o


def binary8_quantize_nearest(a, P, is_signed, overflow_policy, subnormals):
    """pybind_cuda.cpp:61."""
    return _binary8(a, P, is_signed, overflow_policy, subnormals, 0)


def binary8_quantize_stochastic(a, P, prng_bits, is_signed, overflow_policy, subnormals, rand=None):
    """pybind_cuda.cpp:107 (random words drawn as quant_cuda/quant.cu:202 does unless given)."""
    return _binary8(a, P, is_signed, overflow_policy, subnormals, 1, prng_bits, rand)


def binary8_quantize_truncate(a, P, is_signed, overflow_policy, subnormals):
    """pybind_cuda.cpp:115."""
    return _binary8(a, P, is_signed, overflow_policy, subnormals, 2)


def float_quantize_multi(ins, outs, man_bits, exp_bits, subnormals, saturate, rounding=0, prng_bits=0, seed=0):
    """Quantize a list of tensors with one launch per 48 tensors (no reference counterpart; `rounding`: 0 nearest,
    1 stochastic with in-kernel Philox words, 2 truncate).  `outs[i]` may be `ins[i]`."""
    import ctypes as C

    assert len(ins) == len(outs)
    if not ins:
        return
    dev = ins[0].device
    for a, o in zip(ins, outs):
        check_cuda_f32(a, "input"); check_cuda_f32(o, "output")
        if a.device != dev or o.device != dev or a.numel() != o.numel():
            raise RuntimeError("float_quantize_multi: tensors must live on one device and outputs must match inputs in size")
    n = len(ins)
    pin = (C.c_void_p * n)(*[a.data_ptr() for a in ins])
    pout = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    cnt = (C.c_int64 * n)(*[a.numel() for a in ins])
    with torch.cuda.device(dev):
        call("mpt_float_quantize_multi", pin, pout, cnt, n, man_bits, exp_bits, int(subnormals), int(saturate), int(rounding),
             int(prng_bits), int(seed) & 0xFFFFFFFFFFFFFFFF, stream_ptr(dev))


def superfp_quantize_nearest(a, man_bits, exp_bits, binades_l, binades_u, saturate):
    """pybind_cuda.cpp:53."""
    check_cuda_f32(a, "a")
    o = torch.empty_like(a)
    with torch.cuda.device(a.device):
        call("mpt_superfp_quantize_nearest", ptr(a), ptr(o), a.numel(), man_bits, exp_bits, binades_l, binades_u,
             int(saturate), stream_ptr(a.device))
    return o


# ---------------------------------------------------------------------------------- GEMM
def _mm_checks(a, b, c):
    check_cuda_f32(a, "a")
    check_cuda_f32(b, "b")
    check_cuda_f32(c, "c")


def _batch_of(a) -> int:
    # the reference reads the batch count from a.sizes()[0] for the bmm entry points (quant.cu:370-379)
    return a.shape[0] if a.dim() > 2 else 1


def _mm_nearest(a, b, c, batch, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, compensated, order):
    if _ext is not None and order is None and batch == _batch_of(a):
        _ext.float_quantize_nearest_bmm(a, b, c, M, N, K, man_add, exp_add, man_mul, exp_mul, bool(subnormals), bool(saturate), bool(compensated))
        return
    _mm_checks(a, b, c)
    with torch.cuda.device(a.device):
        ws = _cabi.mm_workspace(a.device, batch)
        call("mpt_float_mm_nearest", ptr(a), ptr(b), ptr(c), batch, M, N, K, man_add, exp_add, man_mul, exp_mul,
             int(subnormals), int(saturate), int(bool(compensated)), _order_code(order, "accum_order"), ptr(ws), ws.numel(),
             stream_ptr(a.device))


def _mm_nearest_fma(a, b, c, batch, M, N, K, man_fma, exp_fma, subnormals, saturate, compensated, order):
    if _ext is not None and order is None and batch == _batch_of(a):
        _ext.float_quantize_nearest_bmm_fma(a, b, c, M, N, K, man_fma, exp_fma, bool(subnormals), bool(saturate), bool(compensated))
        return
    _mm_checks(a, b, c)
    with torch.cuda.device(a.device):
        ws = _cabi.mm_workspace(a.device, batch)
        call("mpt_float_mm_nearest_fma", ptr(a), ptr(b), ptr(c), batch, M, N, K, man_fma, exp_fma, int(subnormals),
             int(saturate), int(bool(compensated)), _order_code(order, "accum_order"), ptr(ws), ws.numel(),
             stream_ptr(a.device))


MM_PIECE_FROM_C, MM_PIECE_MORE = 1, 2


def float_mm_nearest_piece(a, b, c, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, fma, flags, order=None):
    """The steps of a product that one K panel contributes (no reference counterpart; `mpt_float_mm_nearest_piece`):
    a [M, K] and b [K, N] are the panel's columns of A and rows of B, c [M, N] carries the running sums from piece to
    piece (MM_PIECE_FROM_C: start from what c holds; MM_PIECE_MORE: another piece follows, K a multiple of 8)."""
    _mm_checks(a, b, c)
    (M, K), N = a.shape, b.shape[1]
    assert b.shape[0] == K and tuple(c.shape) == (M, N)
    with torch.cuda.device(a.device):
        ws = _cabi.mm_workspace(a.device, 1)
        call("mpt_float_mm_nearest_piece", ptr(a), ptr(b), ptr(c), 1, M, N, K, man_add, exp_add, man_mul, exp_mul,
             int(subnormals), int(saturate), int(bool(fma)), _order_code(order, "accum_order"), int(flags), ptr(ws), ws.numel(),
             stream_ptr(a.device))


def transpose_last2(x):
    """A dense copy of ``x.transpose(-2, -1)`` for a contiguous float32 CUDA tensor with at least two dimensions, or None
    when the kernel's grid limits do not admit the shape (the caller then lets torch copy)."""
    rows, cols = x.shape[-2], x.shape[-1]
    batch = x.numel() // (rows * cols) if rows * cols else 0
    if batch > 65535 or (rows + 63) // 64 > 65535:
        return None
    out = torch.empty(*x.shape[:-2], cols, rows, device=x.device, dtype=torch.float32)
    if x.numel():
        with torch.cuda.device(x.device):
            call("mpt_transpose_last2", ptr(x), ptr(out), batch, rows, cols, stream_ptr(x.device))
    return out


def copy_columns_async(dst, src, col0: int, col1: int):
    """dst[:, :] = src[:, col0:col1] for row-major float32 matrices on either side of the bus, as one pitched copy on
    the current stream of dst's (or src's) device; dst is dense with col1 - col0 columns."""
    assert dst.dim() == 2 and src.dim() == 2 and dst.is_contiguous() and src.is_contiguous()
    assert dst.dtype == torch.float32 and src.dtype == torch.float32
    rows, width = src.shape[0], col1 - col0
    assert dst.shape == (rows, width) and 0 <= col0 <= col1 <= src.shape[1]
    dev = dst.device if dst.is_cuda else src.device
    with torch.cuda.device(dev):
        call("mpt_copy_columns_async", dst.data_ptr(), 4 * width, src.data_ptr() + 4 * col0, 4 * src.shape[1], 4 * width, rows,
             stream_ptr(dev))


def float_quantize_nearest_mm(a, b, c, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate,
                              compensated, order=None):
    """pybind_cuda.cpp:123.  Note the (M, N, K) argument order of the reference."""
    _mm_nearest(a, b, c, 1, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, compensated, order)


def float_quantize_nearest_bmm(a, b, c, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate,
                               compensated, order=None):
    """pybind_cuda.cpp:140."""
    _mm_nearest(a, b, c, _batch_of(a), M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate,
                compensated, order)


def float_quantize_nearest_mm_fma(a, b, c, M, N, K, man_fma, exp_fma, subnormals, saturate, compensated, order=None):
    """pybind_cuda.cpp:157."""
    _mm_nearest_fma(a, b, c, 1, M, N, K, man_fma, exp_fma, subnormals, saturate, compensated, order)


def float_quantize_nearest_bmm_fma(a, b, c, M, N, K, man_fma, exp_fma, subnormals, saturate, compensated, order=None):
    """pybind_cuda.cpp:173."""
    _mm_nearest_fma(a, b, c, _batch_of(a), M, N, K, man_fma, exp_fma, subnormals, saturate, compensated, order)


def float_conv2d_nearest(x, wt, y, groups, kernel_size, stride, padding, dilation, man_add, exp_add, man_mul, exp_mul,
                         subnormals, saturate, fma=False, order=None):
    """2-D convolution as an implicit GEMM (new; no pybind counterpart: the reference unfolds the input and calls
    float_quantize_nearest_mm).  ``x`` [N, C, H, W], ``y`` [N, C_out, OH, OW], ``wt`` the per-group transposed
    weight matrices [groups, C / groups * KH * KW, C_out / groups], all contiguous float32 on one device."""
    check_cuda_f32(x, "x"); check_cuda_f32(wt, "wt"); check_cuda_f32(y, "y")
    n, c, h, w = x.shape
    c_out = y.shape[1]
    with torch.cuda.device(x.device):
        ws = _cabi.mm_workspace(x.device, 1)
        call("mpt_float_conv2d_nearest", ptr(x), ptr(wt), ptr(y), n, c, h, w, c_out, groups, kernel_size[0], kernel_size[1],
             stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1], man_add, exp_add, man_mul, exp_mul,
             int(subnormals), int(saturate), int(bool(fma)), _order_code(order, "accum_order"), ptr(ws), ws.numel(),
             stream_ptr(x.device))


def float_conv2d_wgrad_nearest(grad_out, x, grad_w, groups, kernel_size, stride, padding, dilation, man_add, exp_add, man_mul,
                               exp_mul, subnormals, saturate, fma=False, order=None):
    """Weight gradient of the 2-D convolution as an implicit GEMM (new; the reference unfolds the saved input and calls
    float_quantize_nearest_mm on it).  ``grad_out`` [N, C_out, OH, OW], ``x`` [N, C, H, W], ``grad_w`` [C_out, C / groups *
    KH * KW], all contiguous float32 on one device."""
    check_cuda_f32(grad_out, "grad_out"); check_cuda_f32(x, "x"); check_cuda_f32(grad_w, "grad_w")
    n, c, h, w = x.shape
    c_out = grad_out.shape[1]
    with torch.cuda.device(x.device):
        ws = _cabi.mm_workspace(x.device, 1)
        call("mpt_float_conv2d_wgrad_nearest", ptr(grad_out), ptr(x), ptr(grad_w), n, c, h, w, c_out, groups, kernel_size[0],
             kernel_size[1], stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1], man_add, exp_add, man_mul,
             exp_mul, int(subnormals), int(saturate), int(bool(fma)), _order_code(order, "accum_order"), ptr(ws), ws.numel(),
             stream_ptr(x.device))


def _mm_sr(a, b, c, batch, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals, saturate,
           fma, seed):
    _mm_checks(a, b, c)
    if seed is None:
        # one draw from the torch generator keeps runs reproducible under torch.manual_seed
        seed = int(torch.randint(0, 2**62, (1,), dtype=torch.int64).item())
    with torch.cuda.device(a.device):
        ws = _cabi.mm_workspace(a.device, batch)
        call("mpt_float_mm_stochastic", ptr(a), ptr(b), ptr(c), batch, M, N, K, man_add, exp_add, rbits_add, man_mul,
             exp_mul, rbits_mul, int(subnormals), int(saturate), int(fma), int(seed) & (2**64 - 1), ptr(ws), ws.numel(),
             stream_ptr(a.device))


def float_quantize_stochastic_mm(a, b, c, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul,
                                 subnormals, saturate, seed=None):
    """pybind_cuda.cpp:254."""
    _mm_sr(a, b, c, 1, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals, saturate, False, seed)


def float_quantize_stochastic_bmm(a, b, c, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul,
                                  subnormals, saturate, seed=None):
    """pybind_cuda.cpp:270."""
    _mm_sr(a, b, c, _batch_of(a), M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals,
           saturate, False, seed)


def float_quantize_stochastic_mm_fma(a, b, c, M, N, K, man_fma, exp_fma, rbits_fma, subnormals, saturate, seed=None):
    """pybind_cuda.cpp:286."""
    _mm_sr(a, b, c, 1, M, N, K, man_fma, exp_fma, rbits_fma, man_fma, exp_fma, rbits_fma, subnormals, saturate, True, seed)


def float_quantize_stochastic_bmm_fma(a, b, c, M, N, K, man_fma, exp_fma, rbits_fma, subnormals, saturate, seed=None):
    """pybind_cuda.cpp:300."""
    _mm_sr(a, b, c, _batch_of(a), M, N, K, man_fma, exp_fma, rbits_fma, man_fma, exp_fma, rbits_fma, subnormals,
           saturate, True, seed)


# ---------------------------------------------------------------------------------- row reductions
def partition_tensor(shape, dim):
    """(outer, channel, inner) of a reduction over ``dim`` (int) or over the trailing ``dims`` (list, given
    last dimension first as the layers do).  reference: quant_cuda/quant.cu:678-726."""
    nd = len(shape)
    if isinstance(dim, int):
        real = [(nd + (dim % nd)) % nd]
        lo = hi = real[0]
    else:
        real = [(nd + (d % nd)) % nd for d in dim]
        lo, hi = real[-1], real[0]
    channel = 1
    for d in real:
        channel *= shape[d]
    outer = 1
    for i in range(lo):
        outer *= shape[i]
    inner = 1
    for i in range(hi + 1, nd):
        inner *= shape[i]
    total = 1
    for n in shape:
        total *= n
    if outer * channel * inner != total:
        # the reference computes sizes that overrun the tensor here; refuse instead
        raise ValueError("dims %r must be adjacent dimensions listed last-first (e.g. [-1, -2]) of a tensor of shape %r"
                         % (dim, tuple(shape)))
    return outer, channel, inner


def float_quantize_nearest_softmax_forward(a, o, dim, man_exp, exp_exp, man_off, exp_off, man_acc, exp_acc, subnormals,
                                           saturate, order=None):
    """pybind_cuda.cpp:599."""
    if _ext is not None and order is None and isinstance(dim, int):
        _ext.float_quantize_nearest_softmax_forward(a, o, dim, man_exp, exp_exp, man_off, exp_off, man_acc, exp_acc, bool(subnormals), bool(saturate))
        return
    check_cuda_f32(a, "a"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_float_softmax_forward", ptr(a), ptr(o), outer, ch, inner, man_exp, exp_exp, man_off, exp_off, man_acc,
             exp_acc, int(subnormals), int(saturate), _order_code(order, "reduce_order"), stream_ptr(a.device))


def float_quantize_nearest_softmax_lse_forward(a, o, dim, man_off, exp_off, man_lse, exp_lse, subnormals, saturate,
                                               order=None):
    """pybind_cuda.cpp:615."""
    check_cuda_f32(a, "a"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_float_softmax_lse_forward", ptr(a), ptr(o), outer, ch, inner, man_off, exp_off, man_lse, exp_lse,
             int(subnormals), int(saturate), _order_code(order, "reduce_order"), stream_ptr(a.device))


def float_quantize_nearest_softmax_backward(a, g, o, dim, man_add, exp_add, man_mul, exp_mul, subnormals, saturate,
                                            order=None):
    """pybind_cuda.cpp:629.  ``a`` is the softmax output, ``g`` the incoming gradient."""
    if _ext is not None and order is None and isinstance(dim, int):
        _ext.float_quantize_nearest_softmax_backward(a, g, o, dim, man_add, exp_add, man_mul, exp_mul, bool(subnormals), bool(saturate))
        return
    check_cuda_f32(a, "a"); check_cuda_f32(g, "g"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_float_softmax_backward", ptr(a), ptr(g), ptr(o), outer, ch, inner, man_add, exp_add, man_mul, exp_mul,
             int(subnormals), int(saturate), _order_code(order, "reduce_order"), stream_ptr(a.device))


def float_quantize_layernorm_forward(input, weight, bias, output, mean, rstd, eps, dims, man_acc, exp_acc, man_mul,
                                     exp_mul, man_div, exp_div, man_sqrt, exp_sqrt, subnormals, saturate, order=None):
    """pybind_cuda.cpp:434."""
    outer, ch, inner = partition_tensor(input.shape, list(dims))      # also refuses dimension lists the reference mishandles
    if _ext is not None and order is None:
        _ext.float_quantize_layernorm_forward(input, weight, bias, output, mean, rstd, float(eps), [int(d) for d in dims], man_acc, exp_acc,
                                              man_mul, exp_mul, man_div, exp_div, man_sqrt, exp_sqrt, bool(subnormals), bool(saturate))
        return
    for t, n in ((input, "input"), (weight, "weight"), (bias, "bias"), (output, "output"), (mean, "mean"), (rstd, "rstd")):
        check_cuda_f32(t, n)
    with torch.cuda.device(input.device):
        call("mpt_float_layernorm_forward", ptr(input), ptr(weight), ptr(bias), ptr(output), ptr(mean), ptr(rstd),
             float(eps), outer, ch, inner, man_acc, exp_acc, man_mul, exp_mul, man_div, exp_div, man_sqrt, exp_sqrt,
             int(subnormals), int(saturate), _order_code(order, "reduce_order"), stream_ptr(input.device))


def float_quantize_layernorm_backward(input, grad_output, weight, bias, mean, rstd, grad_input, grad_gamma, grad_beta,
                                      dims, man_acc, exp_acc, man_mul, exp_mul, man_div, exp_div, subnormals, saturate,
                                      order=None):
    """pybind_cuda.cpp:459 (``bias`` is accepted and unused, as in the reference)."""
    outer, ch, inner = partition_tensor(input.shape, list(dims))
    if _ext is not None and order is None:
        _ext.float_quantize_layernorm_backward(input, grad_output, weight, bias if bias is not None else weight, mean, rstd, grad_input,
                                               grad_gamma, grad_beta, [int(d) for d in dims], man_acc, exp_acc, man_mul, exp_mul, man_div,
                                               exp_div, bool(subnormals), bool(saturate))
        return
    for t, n in ((input, "input"), (grad_output, "grad_output"), (weight, "weight"), (mean, "mean"), (rstd, "rstd"),
                 (grad_input, "grad_input"), (grad_gamma, "grad_gamma"), (grad_beta, "grad_beta")):
        check_cuda_f32(t, n)
    with torch.cuda.device(input.device):
        call("mpt_float_layernorm_backward", ptr(input), ptr(grad_output), ptr(weight), ptr(mean), ptr(rstd),
             ptr(grad_input), ptr(grad_gamma), ptr(grad_beta), outer, ch, inner, man_acc, exp_acc, man_mul, exp_mul,
             man_div, exp_div, int(subnormals), int(saturate), _order_code(order, "reduce_order"),
             stream_ptr(input.device))


def qsum_rows(a, man_bits, exp_bits, subnormals, saturate):
    """New: sequential rounded sum over dim 0 of a 2-D tensor in one launch."""
    if _ext is not None:
        return _ext.qsum_rows(a, man_bits, exp_bits, bool(subnormals), bool(saturate))
    check_cuda_f32(a, "a")
    if a.dim() != 2:
        raise RuntimeError("qsum_rows expects a 2-D tensor")
    o = torch.empty(a.shape[1], device=a.device)
    with torch.cuda.device(a.device):
        call("mpt_qsum_rows", ptr(a), ptr(o), a.shape[0], a.shape[1], man_bits, exp_bits, int(subnormals), int(saturate),
             stream_ptr(a.device))
    return o


def scale_quantize(a, normal_max, margin, fmt=None):
    """New: the layers' tensor scaling in two kernels.  For every matrix (the last two dimensions) of ``a``:
    s = floor(log2(normal_max / amax)) - margin and out = Q(a * 2^s), with Q the nearest rounding to ``fmt`` =
    (man, exp, subnormals, saturate), or no rounding when ``fmt`` is None.  Returns (out, s) with s shaped
    [..., 1, 1] like the reference's compute_bias (functional.py:39-46)."""
    check_cuda_f32(a, "a")
    if a.dim() < 2:
        raise RuntimeError("scale_quantize expects at least two dimensions")
    per = a.shape[-1] * a.shape[-2]
    mats = a.numel() // per if per else 0
    o = torch.empty_like(a)
    sc = torch.empty(tuple(a.shape[:-2]) + (1, 1), device=a.device)
    man, exp, sub, sat = fmt if fmt is not None else (23, 8, True, False)
    with torch.cuda.device(a.device):
        ws = torch.empty(max(4 * mats, 4), dtype=torch.uint8, device=a.device)
        call("mpt_scale_quantize", ptr(a), ptr(o), mats, per, float(normal_max), int(margin), int(fmt is not None), man, exp,
             int(sub), int(sat), ptr(sc), ptr(ws), ws.numel(), stream_ptr(a.device))
    return o, sc


# ---------------------------------------------------------------------------------- other format families
# The reference registers the same GEMM / softmax / layernorm entry points once more for supernormal floats and, for
# the reductions, for binary8 (pybind_cuda.cpp:815-824, :887-924).  They all forward to the generic-format C ABI.
Format = _cabi.Format
def _fp(f):
    import ctypes

    return ctypes.byref(f)


def mm_fmt(a, b, c, batch, M, N, K, fadd: Format, fmul: Format, fma: bool, order=None):
    _mm_checks(a, b, c)
    with torch.cuda.device(a.device):
        ws = _cabi.mm_workspace(a.device, batch)
        call("mpt_mm_nearest_fmt", ptr(a), ptr(b), ptr(c), batch, M, N, K, _fp(fadd), _fp(fmul), int(fma),
             _order_code(order, "accum_order"), ptr(ws), ws.numel(), stream_ptr(a.device))


def superfp_quantize_nearest_mm(a, b, c, M, N, K, man_add, exp_add, man_mul, exp_mul, binades_add_l, binades_add_u,
                                binades_mul_l, binades_mul_u, saturate, order=None):
    """pybind_cuda.cpp:815."""
    mm_fmt(a, b, c, 1, M, N, K, Format.superfp(man_add, exp_add, binades_add_l, binades_add_u, saturate),
           Format.superfp(man_mul, exp_mul, binades_mul_l, binades_mul_u, saturate), False, order)


def superfp_quantize_nearest_bmm(a, b, c, M, N, K, man_add, exp_add, man_mul, exp_mul, binades_add_l, binades_add_u,
                                 binades_mul_l, binades_mul_u, saturate, order=None):
    """pybind_cuda.cpp:818."""
    mm_fmt(a, b, c, _batch_of(a), M, N, K, Format.superfp(man_add, exp_add, binades_add_l, binades_add_u, saturate),
           Format.superfp(man_mul, exp_mul, binades_mul_l, binades_mul_u, saturate), False, order)


def superfp_quantize_nearest_mm_fma(a, b, c, M, N, K, man_fma, exp_fma, binades_fma_l, binades_fma_u, saturate, order=None):
    """pybind_cuda.cpp:821."""
    f = Format.superfp(man_fma, exp_fma, binades_fma_l, binades_fma_u, saturate)
    mm_fmt(a, b, c, 1, M, N, K, f, f, True, order)


def superfp_quantize_nearest_bmm_fma(a, b, c, M, N, K, man_fma, exp_fma, binades_fma_l, binades_fma_u, saturate, order=None):
    """pybind_cuda.cpp:824."""
    f = Format.superfp(man_fma, exp_fma, binades_fma_l, binades_fma_u, saturate)
    mm_fmt(a, b, c, _batch_of(a), M, N, K, f, f, True, order)


def softmax_forward_fmt(a, o, dim, fexp: Format, foff: Format, facc: Format, order=None):
    check_cuda_f32(a, "a"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_softmax_forward_fmt", ptr(a), ptr(o), outer, ch, inner, _fp(fexp), _fp(foff), _fp(facc),
             _order_code(order, "reduce_order"), stream_ptr(a.device))


def softmax_lse_forward_fmt(a, o, dim, foff: Format, flse: Format, order=None):
    check_cuda_f32(a, "a"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_softmax_lse_forward_fmt", ptr(a), ptr(o), outer, ch, inner, _fp(foff), _fp(flse),
             _order_code(order, "reduce_order"), stream_ptr(a.device))


def softmax_backward_fmt(a, g, o, dim, fadd: Format, fmul: Format, order=None):
    check_cuda_f32(a, "a"); check_cuda_f32(g, "g"); check_cuda_f32(o, "o")
    outer, ch, inner = partition_tensor(a.shape, dim)
    with torch.cuda.device(a.device):
        call("mpt_softmax_backward_fmt", ptr(a), ptr(g), ptr(o), outer, ch, inner, _fp(fadd), _fp(fmul),
             _order_code(order, "reduce_order"), stream_ptr(a.device))


def layernorm_forward_fmt(input, weight, bias, output, mean, rstd, eps, dims, facc, fmul, fdiv, fsqrt, order=None):
    for t, n in ((input, "input"), (weight, "weight"), (bias, "bias"), (output, "output"), (mean, "mean"), (rstd, "rstd")):
        check_cuda_f32(t, n)
    outer, ch, inner = partition_tensor(input.shape, list(dims))
    with torch.cuda.device(input.device):
        call("mpt_layernorm_forward_fmt", ptr(input), ptr(weight), ptr(bias), ptr(output), ptr(mean), ptr(rstd), float(eps),
             outer, ch, inner, _fp(facc), _fp(fmul), _fp(fdiv), _fp(fsqrt), _order_code(order, "reduce_order"),
             stream_ptr(input.device))


def layernorm_backward_fmt(input, grad_output, weight, mean, rstd, grad_input, grad_gamma, grad_beta, dims, facc, fmul, fdiv,
                           order=None):
    for t, n in ((input, "input"), (grad_output, "grad_output"), (weight, "weight"), (mean, "mean"), (rstd, "rstd"),
                 (grad_input, "grad_input"), (grad_gamma, "grad_gamma"), (grad_beta, "grad_beta")):
        check_cuda_f32(t, n)
    outer, ch, inner = partition_tensor(input.shape, list(dims))
    with torch.cuda.device(input.device):
        call("mpt_layernorm_backward_fmt", ptr(input), ptr(grad_output), ptr(weight), ptr(mean), ptr(rstd), ptr(grad_input),
             ptr(grad_gamma), ptr(grad_beta), outer, ch, inner, _fp(facc), _fp(fmul), _fp(fdiv),
             _order_code(order, "reduce_order"), stream_ptr(input.device))


def superfp_quantize_nearest_softmax_forward(a, o, dim, man_exp, exp_exp, bel, beu, man_off, exp_off, bol, bou, man_acc, exp_acc,
                                             bal, bau, saturate, order=None):
    """pybind_cuda.cpp:887."""
    softmax_forward_fmt(a, o, dim, Format.superfp(man_exp, exp_exp, bel, beu, saturate), Format.superfp(man_off, exp_off, bol, bou, saturate),
                        Format.superfp(man_acc, exp_acc, bal, bau, saturate), order)


def superfp_quantize_nearest_softmax_lse_forward(a, o, dim, man_off, exp_off, bol, bou, man_lse, exp_lse, bll, blu, saturate, order=None):
    """pybind_cuda.cpp:890."""
    softmax_lse_forward_fmt(a, o, dim, Format.superfp(man_off, exp_off, bol, bou, saturate), Format.superfp(man_lse, exp_lse, bll, blu, saturate), order)


def superfp_quantize_nearest_softmax_backward(a, g, o, dim, man_add, exp_add, bal, bau, man_mul, exp_mul, bml, bmu, saturate, order=None):
    """pybind_cuda.cpp:893."""
    softmax_backward_fmt(a, g, o, dim, Format.superfp(man_add, exp_add, bal, bau, saturate), Format.superfp(man_mul, exp_mul, bml, bmu, saturate), order)


def binary8_quantize_nearest_softmax_forward(a, o, dim, P_exp, op_exp, signed_exp, P_off, op_off, signed_off, P_acc, op_acc,
                                             signed_acc, subnormals, order=None):
    """pybind_cuda.cpp:897."""
    softmax_forward_fmt(a, o, dim, Format.binary8(P_exp, signed_exp, op_exp, subnormals), Format.binary8(P_off, signed_off, op_off, subnormals),
                        Format.binary8(P_acc, signed_acc, op_acc, subnormals), order)


def binary8_quantize_nearest_softmax_lse_forward(a, o, dim, P_off, op_off, signed_off, P_lse, op_lse, signed_lse, subnormals, order=None):
    """pybind_cuda.cpp:900."""
    softmax_lse_forward_fmt(a, o, dim, Format.binary8(P_off, signed_off, op_off, subnormals), Format.binary8(P_lse, signed_lse, op_lse, subnormals), order)


def binary8_quantize_nearest_softmax_backward(a, g, o, dim, P_add, op_add, signed_add, P_mul, op_mul, signed_mul, subnormals, order=None):
    """pybind_cuda.cpp:903."""
    softmax_backward_fmt(a, g, o, dim, Format.binary8(P_add, signed_add, op_add, subnormals), Format.binary8(P_mul, signed_mul, op_mul, subnormals), order)


def superfp_quantize_layernorm_forward(input, weight, bias, output, mean, rstd, eps, dims, man_acc, exp_acc, bal, bau, man_mul, exp_mul,
                                       bml, bmu, man_div, exp_div, bdl, bdu, man_sqrt, exp_sqrt, bsl, bsu, saturate, order=None):
    """pybind_cuda.cpp:914."""
    layernorm_forward_fmt(input, weight, bias, output, mean, rstd, eps, dims, Format.superfp(man_acc, exp_acc, bal, bau, saturate),
                          Format.superfp(man_mul, exp_mul, bml, bmu, saturate), Format.superfp(man_div, exp_div, bdl, bdu, saturate),
                          Format.superfp(man_sqrt, exp_sqrt, bsl, bsu, saturate), order)


def superfp_quantize_layernorm_backward(input, grad_output, weight, bias, mean, rstd, grad_input, grad_gamma, grad_beta, dims, man_acc,
                                        exp_acc, bal, bau, man_mul, exp_mul, bml, bmu, man_div, exp_div, bdl, bdu, saturate, order=None):
    """pybind_cuda.cpp:917."""
    layernorm_backward_fmt(input, grad_output, weight, mean, rstd, grad_input, grad_gamma, grad_beta, dims,
                           Format.superfp(man_acc, exp_acc, bal, bau, saturate), Format.superfp(man_mul, exp_mul, bml, bmu, saturate),
                           Format.superfp(man_div, exp_div, bdl, bdu, saturate), order)


def binary8_quantize_layernorm_forward(input, weight, bias, output, mean, rstd, eps, dims, P_acc, op_acc, signed_acc, P_mul, op_mul,
                                       signed_mul, P_div, op_div, signed_div, P_sqrt, op_sqrt, signed_sqrt, subnormals, order=None):
    """pybind_cuda.cpp:921."""
    layernorm_forward_fmt(input, weight, bias, output, mean, rstd, eps, dims, Format.binary8(P_acc, signed_acc, op_acc, subnormals),
                          Format.binary8(P_mul, signed_mul, op_mul, subnormals), Format.binary8(P_div, signed_div, op_div, subnormals),
                          Format.binary8(P_sqrt, signed_sqrt, op_sqrt, subnormals), order)


def binary8_quantize_layernorm_backward(input, grad_output, weight, bias, mean, rstd, grad_input, grad_gamma, grad_beta, dims, P_acc,
                                        op_acc, signed_acc, P_mul, op_mul, signed_mul, P_div, op_div, signed_div, subnormals, order=None):
    """pybind_cuda.cpp:924."""
    layernorm_backward_fmt(input, grad_output, weight, mean, rstd, grad_input, grad_gamma, grad_beta, dims,
                           Format.binary8(P_acc, signed_acc, op_acc, subnormals), Format.binary8(P_mul, signed_mul, op_mul, subnormals),
                           Format.binary8(P_div, signed_div, op_div, subnormals), order)


# ---------------------------------------------------------------------------------- block-scaled quantizers (new)
_ELEM = {"e4m3": 0, "e2m1": 1}


def mx_quantize(a, elem_format="e4m3", block=32, return_scales=False, return_codes=False):
    """OCP MX block quantization along the last dimension; returns the dequantized tensor, then (on request) the E8M0
    scale codes and the packed element codes (uint8: one byte per E4M3 element, two E2M1 elements per byte)."""
    check_cuda_f32(a, "a")
    if elem_format not in _ELEM:
        raise ValueError("elem_format must be 'e4m3' or 'e2m1'")
    cols = a.shape[-1] if a.dim() else 1
    rows = a.numel() // cols if cols else 0
    o = torch.empty_like(a)
    lead = tuple(a.shape[:-1])
    sc = torch.empty(lead + ((cols + block - 1) // block,), dtype=torch.uint8, device=a.device) if return_scales else None
    width = cols if elem_format == "e4m3" else (cols + 1) // 2
    codes = torch.zeros(lead + (width,), dtype=torch.uint8, device=a.device) if return_codes else None
    with torch.cuda.device(a.device):
        call("mpt_mx_quantize", ptr(a), ptr(o), ptr(sc), ptr(codes), rows, cols, block, _ELEM[elem_format], stream_ptr(a.device))
    res = (o,) + ((sc,) if return_scales else ()) + ((codes,) if return_codes else ())
    return res if len(res) > 1 else o


def nvfp4_quantize(a, global_scale=None, return_scales=False, return_codes=False):
    """NVFP4 quantization along the last dimension; returns the dequantized tensor, then (``return_scales``) the block
    scales as fp32 and the tensor scale, then (``return_codes``) the packed E2M1 codes and the E4M3 scale bytes."""
    check_cuda_f32(a, "a")
    cols = a.shape[-1] if a.dim() else 1
    rows = a.numel() // cols if cols else 0
    o = torch.empty_like(a)
    lead = tuple(a.shape[:-1])
    nblk = (cols + 15) // 16
    sc = torch.empty(lead + (nblk,), device=a.device) if return_scales else None
    gs_out = torch.empty(1, device=a.device) if return_scales else None
    codes = torch.zeros(lead + ((cols + 1) // 2,), dtype=torch.uint8, device=a.device) if return_codes else None
    scodes = torch.empty(lead + (nblk,), dtype=torch.uint8, device=a.device) if return_codes else None
    ws = None
    gs = float(global_scale) if global_scale is not None else 0.0
    if not gs > 0.0:
        ws = torch.empty(1, dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        call("mpt_nvfp4_quantize", ptr(a), ptr(o), ptr(sc), ptr(codes), ptr(scodes), rows, cols, gs, ptr(ws), ptr(gs_out),
             stream_ptr(a.device))
    res = (o,) + ((sc, gs_out) if return_scales else ()) + ((codes, scodes) if return_codes else ())
    return res if len(res) > 1 else o
