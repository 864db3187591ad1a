"""Public quantization API: the Python layer of the reference's ``mptorch.quant.quant_function`` on
top of the B200 kernels.

Names, argument order, defaults and assertion behaviour follow the reference (file:line cited per
function, paths within the reference project).  Tensors must live on a CUDA device: this library has no
CPU arithmetic path.  Functions of the reference that are outside the accelerated hot path
(fixed point, block floating point, cuBLAS passthrough) are present but raise ``NotImplementedError``.
"""
from __future__ import annotations

from typing import Literal

import torch

from .. import backend as _be
from ..number import Binary8, BlockFloatingPoint, FixedPoint, FloatingPoint, Number, SuperNormalFloat

__all__ = [
    "fixed_point_quantize", "block_quantize", "float_quantize", "float_quantize_multi", "binary8_quantize", "superfp_quantize", "quantizer",
    "mx_quantize", "nvfp4_quantize",
    "mp_mm", "mp_bmm", "float_mm", "float_mm_streamed", "float_bmm", "fxp_mm", "fxp_bmm", "superfp_mm", "superfp_bmm",
    "superfp_softmax_forward", "superfp_softmax_lse_forward", "superfp_softmax_backward", "binary8_softmax_forward",
    "binary8_softmax_lse_forward", "binary8_softmax_backward", "superfp_layernorm_forward", "superfp_layernorm_backward",
    "binary8_layernorm_forward", "binary8_layernorm_backward",
    "mp_softmax_forward", "mp_softmax_backward", "float_softmax_forward", "float_softmax_lse_forward",
    "float_softmax_backward", "mp_layernorm_forward", "mp_layernorm_backward", "float_layernorm_forward",
    "float_layernorm_backward", "qsum_rows",
    "cublas_mm", "cublas_bmm", "cublas_acceleration",
    "set_accum_order", "set_reduce_order", "orders",
]

set_accum_order = _be.set_accum_order
set_reduce_order = _be.set_reduce_order
orders = _be.orders


def _require_cuda(x: torch.Tensor, who: str) -> None:
    if not isinstance(x, torch.Tensor):
        raise AssertionError("x is not a single precision Floating Point Tensor")
    if not x.is_cuda:
        raise RuntimeError(
            "%s: CPU tensors are not supported; this library runs on CUDA devices only (no CPU fallback)" % who)


def _f32c(x: torch.Tensor) -> torch.Tensor:
    """``x`` as a dense float32 tensor.  A transposed view of a dense CUDA tensor (W^T, dY^T, X^T, K^T: what the layers
    hand the GEMM) is copied by the tiled transpose kernel instead of torch's strided elementwise copy."""
    if x.dtype == torch.float32 and x.is_cuda and x.dim() >= 2 and not x.is_contiguous() and x.shape[-1] > 1 and x.shape[-2] > 1:
        t = x.transpose(-2, -1)
        if t.is_contiguous():
            y = _be.transpose_last2(t)
            if y is not None:
                return y
    return x.contiguous() if x.dtype == torch.float32 else x.float().contiguous()


def translate_overflow_policy(policy: str) -> _be.OverflowPolicy:
    """reference: quant_function.py:108-124."""
    table = {"saturate_infty": _be.OverflowPolicy.SATURATE_INFTY, "saturate_maxfloat": _be.OverflowPolicy.SATURATE_MAXFLOAT,
             "saturate_maxfloat2": _be.OverflowPolicy.SATURATE_MAXFLOAT2}
    if policy not in table:
        raise ValueError("invalid overflow policy, {}".format(policy))
    return table[policy]


def normalize_binades(binades) -> tuple[int, int]:
    if isinstance(binades, int):
        return binades, binades
    if len(binades) == 1:
        return binades[0], binades[0]
    return binades[0], binades[1]


# ------------------------------------------------------------------------------------------ quantizers
def float_quantize(x: torch.Tensor, exp: int, man: int,
                   rounding: Literal["nearest", "stochastic", "truncate"] = "stochastic",
                   subnormals: bool = True, saturate: bool = True, prng: int = 0) -> torch.Tensor:
    """Quantize an fp32 tensor to an IEEE-like (exp, man) format; the result stays fp32.

    reference: quant_function.py:2982-3023.  ``rounding="truncate"`` is new (the reference has it only
    for binary8).  Stochastic rounding draws its random words from the torch CUDA generator exactly as
    the reference does, so the two agree bit for bit under the same ``torch.manual_seed``.
    """
    assert isinstance(x, torch.Tensor), "x is not a single precision Floating Point Tensor"
    assert rounding in ["stochastic", "nearest", "truncate"], "invalid rounding mode, {}".format(rounding)
    _require_cuda(x, "float_quantize")
    xc = _f32c(x)
    if rounding == "nearest":
        return _be.float_quantize_nearest(xc, man, exp, subnormals, saturate)
    if rounding == "truncate":
        return _be.float_quantize_truncate(xc, man, exp, subnormals, saturate)
    if prng == 0:
        prng = 23 - man
    return _be.float_quantize_stochastic(xc, man, exp, prng, subnormals, saturate)


def float_quantize_multi(tensors, exp: int, man: int, rounding: Literal["nearest", "stochastic", "truncate"] = "nearest",
                         subnormals: bool = True, saturate: bool = True, prng: int = 0, inplace: bool = False,
                         seed: int | None = None):
    """``float_quantize`` over a list of tensors with one kernel launch per 48 tensors (new; the optimizer wrapper's
    per-tensor loops, reference optim_low.py:65-113, are its use).  Nearest and truncate give the bits of
    ``float_quantize`` per tensor; stochastic draws Philox words inside the kernel from ``seed`` (default: one draw
    from the torch CPU generator), so it is reproducible under ``torch.manual_seed`` but does not repeat the
    per-tensor ``randint_like`` streams of ``float_quantize``.  Returns the list of results (the inputs themselves
    when ``inplace``)."""
    assert rounding in ["stochastic", "nearest", "truncate"], "invalid rounding mode, {}".format(rounding)
    tensors = list(tensors)
    for t in tensors:
        _require_cuda(t, "float_quantize_multi")
    if inplace:
        for t in tensors:
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise RuntimeError("float_quantize_multi(inplace=True) needs contiguous float32 tensors")
        ins = outs = tensors
    else:
        ins = [_f32c(t) for t in tensors]
        outs = [torch.empty_like(t) for t in ins]
    mode = {"nearest": 0, "stochastic": 1, "truncate": 2}[rounding]
    if mode == 1:
        if prng == 0:
            prng = 23 - man
        if seed is None:
            seed = int(torch.randint(0, 2**62, (1,)).item())
    _be.float_quantize_multi(ins, outs, man, exp, subnormals, saturate, mode, prng, seed or 0)
    return outs


def binary8_quantize(x: torch.Tensor, P: int, rounding: Literal["nearest", "stochastic", "truncate"] = "nearest",
                     overflow_policy: str = "saturate_maxfloat", is_signed: bool = True, subnormals: bool = True,
                     prng_bits: int = 0) -> torch.Tensor:
    """Quantize to an IEEE P3109 binary8 format.  reference: quant_function.py:3026-3083."""
    assert isinstance(x, torch.Tensor), "x is not a single precision Floating Point Tensor"
    assert rounding in ["stochastic", "nearest", "truncate"], "invalid rounding mode, {}".format(rounding)
    assert 0 <= prng_bits <= 23 - (P - 1), "prng_bits should be between 0 and 23 minus the number of mantissa bits"
    _require_cuda(x, "binary8_quantize")
    pol = translate_overflow_policy(overflow_policy)
    xc = _f32c(x)
    if rounding == "nearest":
        return _be.binary8_quantize_nearest(xc, P, is_signed, pol, subnormals)
    if rounding == "stochastic":
        return _be.binary8_quantize_stochastic(xc, P, prng_bits, is_signed, pol, subnormals)
    return _be.binary8_quantize_truncate(xc, P, is_signed, pol, subnormals)


def superfp_quantize(x: torch.Tensor, exp: int, man: int, binades, rounding: Literal["stochastic", "nearest"] = "nearest",
                     saturate: bool = False) -> torch.Tensor:
    """Quantize to a supernormal float format.  reference: quant_function.py:3086-3125."""
    assert isinstance(x, torch.Tensor), "x is not a single precision Floating Point Tensor"
    assert rounding in ["stochastic", "nearest"], "invalid rounding mode, {}".format(rounding)
    _require_cuda(x, "superfp_quantize")
    if rounding == "stochastic":
        raise NotImplementedError("SR SuperNormalFloat not yet implemented")
    bl, bu = normalize_binades(binades)
    return _be.superfp_quantize_nearest(_f32c(x), man, exp, bl, bu, saturate)


def mx_quantize(x: torch.Tensor, elem_format: Literal["e4m3", "e2m1"] = "e4m3", block: int = 32,
                return_scales: bool = False, return_codes: bool = False):
    """OCP Microscaling block quantization along the last dimension (new; the reference has none).

    Every ``block`` consecutive elements share one power-of-two scale 2^(floor(log2 amax) - emax) stored as
    E8M0; elements are rounded to nearest even into OCP E4M3 (MXFP8, max 448) or E2M1 (MXFP4, max 6) with
    saturation.  Returns the dequantized fp32 tensor, plus the uint8 scale codes with ``return_scales`` and the
    packed element codes with ``return_codes`` (uint8: a byte per E4M3 element; two E2M1 elements per byte, the
    even one in the low nibble).  Note these OCP element formats differ from ``float_quantize(exp=4, man=3)``,
    which reserves the top exponent and tops out at 240."""
    _require_cuda(x, "mx_quantize")
    return _be.mx_quantize(_f32c(x), elem_format, block, return_scales, return_codes)


def nvfp4_quantize(x: torch.Tensor, global_scale: float | None = None, return_scales: bool = False,
                   return_codes: bool = False):
    """NVFP4 quantization along the last dimension (new): E2M1 elements in blocks of 16, an E4M3 scale per
    block and one fp32 scale per tensor (``amax / (448 * 6)`` over the finite entries unless given).  Returns the
    dequantized tensor, plus (block scales, tensor scale) with ``return_scales`` and (packed E2M1 codes, E4M3 scale
    bytes) with ``return_codes``."""
    _require_cuda(x, "nvfp4_quantize")
    return _be.nvfp4_quantize(_f32c(x), global_scale, return_scales, return_codes)


def fixed_point_quantize(*args, **kwargs):
    """reference: quant_function.py:2913.  Fixed point is outside this library's hot path."""
    raise NotImplementedError("fixed_point_quantize is not part of the B200 hot path")


def block_quantize(*args, **kwargs):
    """reference: quant_function.py:2950 (legacy block floating point).  See mx_quantize / nvfp4_quantize."""
    raise NotImplementedError("block_quantize (legacy block floating point) is not part of the B200 hot path")


def quantizer(forward_number: Number | None = None, backward_number: Number | None = None,
              forward_rounding: str = "stochastic", backward_rounding: str = "stochastic",
              clamping_grad_zero: bool = False, backward_hooks=[]):
    """A differentiable quantization function: quantizes activations on the way forward and gradients on
    the way back.  reference: quant_function.py:2661-2910 (float-like formats only here)."""
    for rnd in (forward_rounding, backward_rounding):
        assert rnd in ["stochastic", "nearest"], "invalid rounding type {:s}".format(rnd)
    for num in (forward_number, backward_number):
        if num is not None:
            assert isinstance(num, Number)
    if clamping_grad_zero:
        raise NotImplementedError("clamping_grad_zero applies to fixed point, which is outside the hot path")

    def make(num, rounding):
        if num is None:
            return lambda x: x
        if isinstance(num, FloatingPoint):
            return lambda x: float_quantize(x, num.exp, num.man, rounding, num.subnormals, num.saturate)
        if isinstance(num, Binary8):
            return lambda x: binary8_quantize(x, num.P, rounding, num.overflow_policy, num.signed, num.subnormals)
        if isinstance(num, SuperNormalFloat):
            return lambda x: superfp_quantize(x, num.exp, num.man, num.binades, rounding, num.saturate)
        raise NotImplementedError("quantizer: %r is outside the B200 hot path" % (num,))

    fwd, bwd = make(forward_number, forward_rounding), make(backward_number, backward_rounding)

    class Rounding(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x if forward_number is None else fwd(x.contiguous())

        @staticmethod
        def backward(ctx, grad_output):
            if not ctx.needs_input_grad[0]:
                return None
            g = grad_output if backward_number is None else bwd(grad_output.contiguous())
            for hook in backward_hooks:
                g = hook(g)
            return g

    def apply(x):
        return Rounding.apply(x)

    # what the function does, for callers that can fuse it (the optimizer wrapper quantizes whole parameter lists)
    apply.forward_number, apply.forward_rounding = forward_number, forward_rounding
    apply.backward_number, apply.backward_rounding = backward_number, backward_rounding
    return apply


# ------------------------------------------------------------------------------------------ GEMM
def _mm_dispatch(a2, b2, batched, man_add, exp_add, man_mul, exp_mul, rounding, fma, subnormals, saturate,
                 compensated, rbits_add, rbits_mul):
    """One (possibly batched) GEMM on contiguous fp32 operands; allocates and returns C."""
    # The kernel's CTA tile is 128 rows by 64 columns: a product with at most 64 rows and many columns would leave half of
    # every tile idle.  C^T = B^T A^T has the same products (multiplication commutes exactly) accumulated in the same
    # K order, so the transposed problem gives the same bits with full tiles; the result comes back as a transposed view.
    # (Not for stochastic rounding: its random words are keyed by the position of the output in C.)
    if rounding == "nearest" and a2.shape[-2] <= 64 and b2.shape[-1] >= 256 and a2.shape[-1] >= 128:
        ct = _mm_dispatch(b2.transpose(-2, -1).contiguous(), a2.transpose(-2, -1).contiguous(), batched, man_add, exp_add, man_mul,
                          exp_mul, rounding, fma, subnormals, saturate, compensated, rbits_add, rbits_mul)
        return ct.transpose(-2, -1)
    if batched:
        Bn, M, K = a2.shape
        N = b2.shape[2]
        c = torch.empty(Bn, M, N, device=a2.device)
    else:
        M, K = a2.shape
        N = b2.shape[1]
        c = torch.empty(M, N, device=a2.device)
    if rounding == "nearest":
        if not fma:
            fn = _be.float_quantize_nearest_bmm if batched else _be.float_quantize_nearest_mm
            fn(a2, b2, c, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, compensated)
        else:
            fn = _be.float_quantize_nearest_bmm_fma if batched else _be.float_quantize_nearest_mm_fma
            fn(a2, b2, c, M, N, K, man_add, exp_add, subnormals, saturate, compensated)
    else:
        # reference quant_function.py:1616-1619: rbits_add defaults to 23 - man_add; the matching line for
        # rbits_mul is a comparison, so rbits_mul keeps the caller's value (0 unless set)
        if rbits_add <= 0:
            rbits_add = 23 - man_add
        if not fma:
            fn = _be.float_quantize_stochastic_bmm if batched else _be.float_quantize_stochastic_mm
            fn(a2, b2, c, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals, saturate)
        else:
            fn = _be.float_quantize_stochastic_bmm_fma if batched else _be.float_quantize_stochastic_mm_fma
            fn(a2, b2, c, M, N, K, man_add, exp_add, rbits_add, subnormals, saturate)
    return c


def float_mm(a: torch.Tensor, b: torch.Tensor, man_add: int = 23, exp_add: int = 8, man_mul: int = 23, exp_mul: int = 8,
             rounding: Literal["nearest", "stochastic"] = "nearest", fma: bool = True, subnormals: bool = True,
             saturate: bool = True, compensated: bool = False, rbits_add: int = 0, rbits_mul: int = 0) -> torch.Tensor:
    """GEMM (M,K) x (K,N) in which every multiply and every add is rounded to its format.

    reference: quant_function.py:1527-1651.  With ``fma=True`` each step is one fused multiply-add rounded
    to (man_add, exp_add).  The K-accumulation order is the one selected by ``set_accum_order`` /
    ``orders`` ("cuda": the reference CUDA kernels' 8-wide tiles; "seq": the reference CPU loop).
    """
    assert len(a.shape) == 2
    assert len(b.shape) == 2
    assert a.shape[1] == b.shape[0]
    assert a.device == b.device
    _require_cuda(a, "float_mm")
    return _mm_dispatch(_f32c(a), _f32c(b), False, man_add, exp_add, man_mul, exp_mul, rounding, fma, subnormals,
                        saturate, compensated, rbits_add, rbits_mul)


def float_mm_streamed(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, device=None, block_rows: int = 1024,
                      man_add: int = 23, exp_add: int = 8, man_mul: int = 23, exp_mul: int = 8,
                      rounding: Literal["nearest", "stochastic"] = "nearest", fma: bool = True, subnormals: bool = True,
                      saturate: bool = True, compensated: bool = False, rbits_add: int = 0, rbits_mul: int = 0,
                      b_ready: "torch.cuda.Event | None" = None) -> torch.Tensor:
    """``float_mm`` for operands that live in HOST memory (new; the reference would run them on the CPU).

    B is copied to the GPU once; A travels in blocks of ``block_rows`` rows on a copy stream while the previous block
    is in the kernel and the one before that returns to the host on a third stream, so the copies of A and C overlap
    the arithmetic.  Rows of C are independent, so the bits equal one ``float_mm`` call on the whole matrices
    (nearest rounding; the stochastic kernel's words are keyed by output position within a call, so its blocks draw
    as separate calls do).  ``a``, ``b`` and ``out`` must be pinned float32 CPU tensors for the copies to overlap;
    pageable tensors work but serialise.  Returns ``out`` (allocated pinned when not given); the call returns after
    the last block has arrived.

    ``b`` may instead already be resident on the device (a caller that assembles it there, e.g. from slices the ranks
    of a job exchange); ``b_ready`` is then an event after which its contents are valid: the first kernel waits for
    it, the copies of A do not."""
    assert len(a.shape) == 2 and len(b.shape) == 2 and a.shape[1] == b.shape[0]
    for t in (a, b):
        if (t.is_cuda and t is not b) or t.dtype != torch.float32 or not t.is_contiguous():
            raise RuntimeError("float_mm_streamed takes contiguous float32 CPU tensors (use float_mm for CUDA tensors)")
    if not torch.cuda.is_available():
        raise RuntimeError("float_mm_streamed: no CUDA device (there is no CPU fallback)")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32).pin_memory()
    assert out.shape == (M, N) and out.dtype == torch.float32 and not out.is_cuda and out.is_contiguous()
    block_rows = max(1, min(int(block_rows), M)) if M else 1
    kw = (man_add, exp_add, man_mul, exp_mul, rounding, fma, subnormals, saturate, compensated, rbits_add, rbits_mul)
    panels = _k_panels(K) if (rounding == "nearest" and not compensated and not b.is_cuda and M > 0 and N > 0) else None
    if panels is not None:
        fmt = (man_add, exp_add, man_add, exp_add) if fma else (man_add, exp_add, man_mul, exp_mul)
        return _mm_streamed_by_panels(a, N, out, dev, block_rows, panels, fmt, subnormals, saturate, fma,
                                      lambda k0, k1, bd: bd.copy_(b[k0:k1], non_blocking=True))
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        abuf = [torch.empty(block_rows, K, device=dev) for _ in range(2)]
        a_free = [None, None]          # event: the kernel that read abuf[i] has finished
        c_done = []                    # C blocks in flight to the host (kept alive until the final synchronisation)
        s_in.wait_stream(main)
        if b.is_cuda:
            bd = b
            if b_ready is not None:
                main.wait_event(b_ready)
        else:
            bd = b.to(dev, non_blocking=True)
        for i, r0 in enumerate(range(0, M, block_rows)):
            r1 = min(M, r0 + block_rows)
            slot = i & 1
            with torch.cuda.stream(s_in):
                if a_free[slot] is not None:
                    s_in.wait_event(a_free[slot])
                ad = abuf[slot][: r1 - r0]
                ad.copy_(a[r0:r1], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            main.wait_event(arrived)
            cd = _mm_dispatch(ad, bd, False, *kw)
            a_free[slot] = torch.cuda.Event()
            a_free[slot].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(a_free[slot])
                out[r0:r1].copy_(cd, non_blocking=True)
            cd.record_stream(s_out)
            c_done.append(cd)
        s_out.synchronize()
        main.synchronize()
        for t in abuf:
            t.record_stream(s_in)
    return out


_PANEL, _FIRST_PANEL, _LAST_PANEL = 2048, 256, 512


def _k_panels(K: int):
    """Column panels [(k0, k1), ...] of the K-panel pipeline, or None when K is too short to be worth it: a short first
    panel (the first kernel starts after one small copy), then panels that double up to 2048 steps (a panel's copy
    takes a small fraction of the kernel before it, and every kernel ends with a partly filled wave, so few long ones
    are better than many), and a last panel just long enough for its kernels to cover the copy of C back to the host.
    Every boundary but the end is a multiple of 8."""
    if K < _FIRST_PANEL + 1024 + _LAST_PANEL:
        return None
    last0 = (K - _LAST_PANEL) // 8 * 8
    cuts, width = [0, _FIRST_PANEL], 2 * _FIRST_PANEL
    while last0 - cuts[-1] > width + width // 2:
        cuts.append(cuts[-1] + width)
        width = min(2 * width, _PANEL)
    if last0 > cuts[-1]:
        cuts.append(last0)
    cuts.append(K)
    return list(zip(cuts[:-1], cuts[1:]))


def _mm_streamed_by_panels(a, N, out, dev, block_rows, panels, fmt, subnormals, saturate, fma, load_b):
    """``float_mm_streamed`` for host operands, nearest rounding: the product advances along K.  Panel c of A (columns)
    and of B (rows) travels to the GPU while panel c - 1 is in the kernel; a kernel continues the running sums that C
    holds (`mpt_float_mm_nearest_piece`), which performs exactly the operations of the single call, so the bits are
    those of ``float_mm``.  The last panel is multiplied in blocks of ``block_rows`` rows, each finished block of C
    returning to the host under the next block's kernel.  Against copying B whole before the first kernel this hides
    all of the inbound traffic but one short panel.  ``load_b(k0, k1, bd)`` fills the device buffer ``bd`` with rows
    k0 .. k1 - 1 of B on the current (copy) stream: a host copy, or whatever assembles the panel."""
    M, K = a.shape
    block_rows = min(block_rows, max(128, -(-M // 4)))       # at least four blocks of C on their way home
    widest = max(k1 - k0 for k0, k1 in panels)
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        abuf = [torch.empty(M * widest, device=dev) for _ in range(2)]
        bbuf = [torch.empty(widest * N, device=dev) for _ in range(2)]
        c = torch.empty(M, N, device=dev)
        free = [None, None]            # event: the kernels that read slot i have finished
        s_in.wait_stream(main)
        last = len(panels) - 1
        for ci, (k0, k1) in enumerate(panels):
            slot, kc = ci & 1, k1 - k0
            ad, bd = abuf[slot][: M * kc].view(M, kc), bbuf[slot][: kc * N].view(kc, N)
            with torch.cuda.stream(s_in):
                if free[slot] is not None:
                    s_in.wait_event(free[slot])
                _be.copy_columns_async(ad, a, k0, k1)
                load_b(k0, k1, bd)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            main.wait_event(arrived)
            flags = (_be.MM_PIECE_FROM_C if ci else 0) | (_be.MM_PIECE_MORE if ci < last else 0)
            if ci < last:
                _be.float_mm_nearest_piece(ad, bd, c, *fmt, subnormals, saturate, fma, flags)
            else:
                for r0 in range(0, M, block_rows):
                    r1 = min(M, r0 + block_rows)
                    _be.float_mm_nearest_piece(ad[r0:r1], bd, c[r0:r1], *fmt, subnormals, saturate, fma, flags)
                    done = torch.cuda.Event()
                    done.record(main)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(done)
                        out[r0:r1].copy_(c[r0:r1], non_blocking=True)
            free[slot] = torch.cuda.Event()
            free[slot].record(main)
        s_out.synchronize()
        main.synchronize()
        for t in (*abuf, *bbuf):
            t.record_stream(s_in)
        c.record_stream(s_out)
    return out


def float_bmm(a: torch.Tensor, b: torch.Tensor, man_add: int = 23, exp_add: int = 8, man_mul: int = 23, exp_mul: int = 8,
              rounding: Literal["nearest", "stochastic"] = "nearest", fma: bool = True, subnormals: bool = True,
              saturate: bool = True, compensated: bool = False, rbits_add: int = 0, rbits_mul: int = 0) -> torch.Tensor:
    """Batched variant; accepts the reference's four shape cases (quant_function.py:1853-1933):
    3-D x 3-D (equal batch), 3-D x 2-D (one GEMM over the flattened rows), 4-D x 4-D (leading dims
    flattened) and 2-D x 2-D."""
    assert a.shape[-1] == b.shape[-2]
    assert a.device == b.device
    _require_cuda(a, "float_bmm")
    kw = (man_add, exp_add, man_mul, exp_mul, rounding, fma, subnormals, saturate, compensated, rbits_add, rbits_mul)
    a, b = _f32c(a), _f32c(b)
    if a.dim() == 3 and b.dim() == 3:
        return _mm_dispatch(a, b, True, *kw)
    if a.dim() == 3 and b.dim() == 2:
        c = _mm_dispatch(a.reshape(a.shape[0] * a.shape[1], a.shape[2]), b, False, *kw)
        return c.reshape(a.shape[0], a.shape[1], b.shape[1])
    if a.dim() == 4 and b.dim() == 4:
        a_r = a.reshape(a.shape[0] * a.shape[1], a.shape[2], a.shape[3])
        b_r = b.reshape(b.shape[0] * b.shape[1], b.shape[2], b.shape[3])
        c = _mm_dispatch(a_r, b_r, True, *kw)
        return c.reshape(a.shape[0], a.shape[1], a.shape[2], b.shape[3])
    if a.dim() == 2 and b.dim() == 2:
        return _mm_dispatch(a, b, False, *kw)
    raise Exception("Wrong tensor sizes")


def _sfp(man, exp, binades, saturate):
    bl, bu = normalize_binades(binades)
    return _be.Format.superfp(man, exp, bl, bu, saturate)


def _b8(P, policy, signed, subnormals):
    return _be.Format.binary8(P, signed, translate_overflow_policy(policy), subnormals)


def _mm_fmt(a, b, fadd, fmul, fma):
    """GEMM for the shape cases of float_bmm with generic rounding formats."""
    assert a.shape[-1] == b.shape[-2]
    assert a.device == b.device
    _require_cuda(a, "matrix product")
    a, b = _f32c(a), _f32c(b)

    def run(a2, b2, batched):
        if batched:
            Bn, M, K = a2.shape
            N = b2.shape[2]
            c = torch.empty(Bn, M, N, device=a2.device)
        else:
            (M, K), N = a2.shape, b2.shape[1]
            Bn, c = 1, torch.empty(M, N, device=a2.device)
        _be.mm_fmt(a2, b2, c, Bn, M, N, K, fadd, fmul, fma)
        return c

    if a.dim() == 3 and b.dim() == 3:
        return run(a, b, True)
    if a.dim() == 3 and b.dim() == 2:
        return run(a.reshape(-1, a.shape[2]), b, False).reshape(a.shape[0], a.shape[1], b.shape[1])
    if a.dim() == 4 and b.dim() == 4:
        c = run(a.reshape(-1, a.shape[2], a.shape[3]), b.reshape(-1, b.shape[2], b.shape[3]), True)
        return c.reshape(a.shape[0], a.shape[1], a.shape[2], b.shape[3])
    if a.dim() == 2 and b.dim() == 2:
        return run(a, b, False)
    raise Exception("Wrong tensor sizes")


def superfp_mm(a: torch.Tensor, b: torch.Tensor, man_add: int = 7, exp_add: int = 8, binades_add=1, man_mul: int = 7,
               exp_mul: int = 8, binades_mul=1, rounding: Literal["nearest", "stochastic"] = "nearest", fma: bool = True,
               saturate: bool = False) -> torch.Tensor:
    """GEMM with multiplies and adds rounded to supernormal-float formats.  reference: quant_function.py:1654-1732."""
    assert len(a.shape) == 2 and len(b.shape) == 2
    if rounding != "nearest":
        raise NotImplementedError("SR SuperNormalFloat MM is not yet implemented")
    return _mm_fmt(a, b, _sfp(man_add, exp_add, binades_add, saturate), _sfp(man_mul, exp_mul, binades_mul, saturate), fma)


def superfp_bmm(a: torch.Tensor, b: torch.Tensor, man_add: int = 7, exp_add: int = 8, binades_add=1, man_mul: int = 7,
                exp_mul: int = 8, binades_mul=1, rounding: Literal["nearest", "stochastic"] = "nearest", fma: bool = True,
                saturate: bool = False) -> torch.Tensor:
    """Batched variant for the shape cases of ``float_bmm``.  reference: quant_function.py:2176-2365."""
    if rounding != "nearest":
        raise NotImplementedError("SR SuperNormalFloat BMM is not yet implemented")
    return _mm_fmt(a, b, _sfp(man_add, exp_add, binades_add, saturate), _sfp(man_mul, exp_mul, binades_mul, saturate), fma)


_FP32 = FloatingPoint(exp=8, man=23, subnormals=True, saturate=False)


def _mac_config(formats, use_forward: bool):
    """reference: quant_function.py:1358-1387."""
    if use_forward:
        if formats.fwd_use_default_prec:
            return _FP32, _FP32, True, "nearest"
        return formats.fwd_add, formats.fwd_mul, formats.fwd_fma, formats.fwd_rnd
    if formats.bwd_use_default_prec:
        return _FP32, _FP32, True, "nearest"
    return formats.bwd_add, formats.bwd_mul, formats.bwd_fma, formats.bwd_rnd


def _mp_matmul(fn, a, b, formats, use_forward):
    add_cfg, mul_cfg, fma, rnd = _mac_config(formats, use_forward)
    assert type(add_cfg) == type(mul_cfg), "Only the same types are currently support for add and mul operations"
    if type(add_cfg) == FloatingPoint:
        # subnormals / saturate of the whole MAC come from the add format (quant_function.py:1402-1403)
        return fn(a, b, man_add=add_cfg.man, exp_add=add_cfg.exp, man_mul=mul_cfg.man, exp_mul=mul_cfg.exp, rounding=rnd,
                  fma=fma, subnormals=add_cfg.subnormals, saturate=add_cfg.saturate, compensated=formats.compensated,
                  rbits_add=formats.rbits_add, rbits_mul=formats.rbits_mul)
    if type(add_cfg) == SuperNormalFloat:
        sfn = superfp_mm if fn is float_mm else superfp_bmm
        return sfn(a, b, man_add=add_cfg.man, exp_add=add_cfg.exp, binades_add=add_cfg.binades, man_mul=mul_cfg.man,
                   exp_mul=mul_cfg.exp, binades_mul=mul_cfg.binades, rounding=rnd, fma=fma, saturate=add_cfg.saturate)
    raise NotImplementedError("matrix products in %s are outside the B200 hot path" % type(add_cfg).__name__)


def mp_mm(a: torch.Tensor, b: torch.Tensor, formats, use_forward: bool = True) -> torch.Tensor:
    """reference: quant_function.py:1354-1433."""
    return _mp_matmul(float_mm, a, b, formats, use_forward)


def mp_bmm(a: torch.Tensor, b: torch.Tensor, formats, use_forward: bool = True) -> torch.Tensor:
    """reference: quant_function.py:1735-1814."""
    return _mp_matmul(float_bmm, a, b, formats, use_forward)


# ------------------------------------------------------------------------------------------ softmax
def float_softmax_forward(input: torch.Tensor, dim: int, man_exp: int = 23, exp_exp: int = 8, man_off: int = 23,
                          exp_off: int = 8, man_acc: int = 23, exp_acc: int = 8,
                          rounding: Literal["nearest", "stochastic"] = "nearest", subnormals: bool = True,
                          saturate: bool = False) -> torch.Tensor:
    """Softmax along ``dim``: y = Qexp(exp(Qoff(x - max))) / sum, the sum accumulated in (man_acc, exp_acc).
    The final division is left unrounded.  reference: quant_function.py:546-575."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    _require_cuda(input, "float_softmax_forward")
    x = _f32c(input)
    out = torch.empty_like(x)
    _be.float_quantize_nearest_softmax_forward(x, out, dim, man_exp, exp_exp, man_off, exp_off, man_acc, exp_acc,
                                               subnormals, saturate)
    return out


def float_softmax_lse_forward(input: torch.Tensor, dim: int, man_off: int = 23, exp_off: int = 8, man_lse: int = 23,
                              exp_lse: int = 8, rounding: Literal["nearest", "stochastic"] = "nearest",
                              subnormals: bool = True, saturate: bool = False) -> torch.Tensor:
    """Division-free softmax through a rounded log-sum-exp recurrence.  reference: quant_function.py:578-603."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    _require_cuda(input, "float_softmax_lse_forward")
    x = _f32c(input)
    out = torch.empty_like(x)
    _be.float_quantize_nearest_softmax_lse_forward(x, out, dim, man_off, exp_off, man_lse, exp_lse, subnormals, saturate)
    return out


def float_softmax_backward(input: torch.Tensor, grad_output: torch.Tensor, dim: int, man_add: int = 23, exp_add: int = 8,
                           man_mul: int = 23, exp_mul: int = 8, rounding: Literal["nearest", "stochastic"] = "nearest",
                           subnormals: bool = True, saturate: bool = False) -> torch.Tensor:
    """``input`` is the softmax output.  reference: quant_function.py:606-634."""
    assert input.device == grad_output.device
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    _require_cuda(input, "float_softmax_backward")
    y = _f32c(input)
    out = torch.empty_like(y)
    _be.float_quantize_nearest_softmax_backward(y, _f32c(grad_output), out, dim, man_add, exp_add, man_mul, exp_mul,
                                                subnormals, saturate)
    return out


def _softmax_fwd(input, dim, fexp, foff, facc):
    _require_cuda(input, "softmax_forward")
    x = _f32c(input)
    out = torch.empty_like(x)
    _be.softmax_forward_fmt(x, out, dim, fexp, foff, facc)
    return out


def _softmax_lse(input, dim, foff, flse):
    _require_cuda(input, "softmax_lse_forward")
    x = _f32c(input)
    out = torch.empty_like(x)
    _be.softmax_lse_forward_fmt(x, out, dim, foff, flse)
    return out


def _softmax_bwd(input, grad_output, dim, fadd, fmul):
    assert input.device == grad_output.device
    _require_cuda(input, "softmax_backward")
    y = _f32c(input)
    out = torch.empty_like(y)
    _be.softmax_backward_fmt(y, _f32c(grad_output), out, dim, fadd, fmul)
    return out


def superfp_softmax_forward(input, dim, man_exp=23, exp_exp=8, binades_exp=1, man_off=23, exp_off=8, binades_off=1, man_acc=23,
                            exp_acc=8, binades_acc=1, rounding="nearest", saturate=False):
    """reference: quant_function.py:637-678."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_fwd(input, dim, _sfp(man_exp, exp_exp, binades_exp, saturate), _sfp(man_off, exp_off, binades_off, saturate),
                        _sfp(man_acc, exp_acc, binades_acc, saturate))


def superfp_softmax_lse_forward(input, dim, man_off=23, exp_off=8, binades_off=1, man_lse=23, exp_lse=8, binades_lse=1,
                                rounding="nearest", saturate=False):
    """reference: quant_function.py:681-714."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_lse(input, dim, _sfp(man_off, exp_off, binades_off, saturate), _sfp(man_lse, exp_lse, binades_lse, saturate))


def superfp_softmax_backward(input, grad_output, dim, man_add=23, exp_add=8, binades_add=1, man_mul=23, exp_mul=8, binades_mul=1,
                             rounding="nearest", saturate=False):
    """reference: quant_function.py:717-753."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_bwd(input, grad_output, dim, _sfp(man_add, exp_add, binades_add, saturate), _sfp(man_mul, exp_mul, binades_mul, saturate))


def binary8_softmax_forward(input, dim, P_exp, op_exp, signed_exp, P_off, op_off, signed_off, P_acc, op_acc, signed_acc, rounding,
                            subnormals):
    """reference: quant_function.py:756-789."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_fwd(input, dim, _b8(P_exp, op_exp, signed_exp, subnormals), _b8(P_off, op_off, signed_off, subnormals),
                        _b8(P_acc, op_acc, signed_acc, subnormals))


def binary8_softmax_lse_forward(input, dim, P_off, op_off, signed_off, P_lse, op_lse, signed_lse, rounding, subnormals):
    """reference: quant_function.py:792-819."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_lse(input, dim, _b8(P_off, op_off, signed_off, subnormals), _b8(P_lse, op_lse, signed_lse, subnormals))


def binary8_softmax_backward(input, grad_output, dim, P_add, op_add, signed_add, P_mul, op_mul, signed_mul, rounding, subnormals):
    """reference: quant_function.py:822-852."""
    assert rounding == "nearest", "Only nearest rounding softmax is implemented."
    return _softmax_bwd(input, grad_output, dim, _b8(P_add, op_add, signed_add, subnormals), _b8(P_mul, op_mul, signed_mul, subnormals))


def _layernorm_fwd(inp, weight, bias, eps, dims, facc, fmul, fdiv, fsqrt):
    _require_cuda(inp, "layernorm_forward")
    x = _f32c(inp)
    lead = list(x.shape[: x.dim() - len(dims)])
    mean = torch.empty(lead, device=x.device)
    rstd = torch.empty(lead, device=x.device)
    out = torch.empty_like(x)
    _be.layernorm_forward_fmt(x, _f32c(weight), _f32c(bias), out, mean, rstd, eps, dims, facc, fmul, fdiv, fsqrt)
    return out, mean, rstd


def _layernorm_bwd(inp, grad_output, weight, bias, mean, rstd, dims, facc, fmul, fdiv):
    assert inp.device == grad_output.device
    _require_cuda(inp, "layernorm_backward")
    x = _f32c(inp)
    gi = torch.empty_like(x)
    gw = torch.empty_like(weight, dtype=torch.float32).contiguous()
    gb = torch.empty_like(bias, dtype=torch.float32).contiguous()
    _be.layernorm_backward_fmt(x, _f32c(grad_output), _f32c(weight), _f32c(mean), _f32c(rstd), gi, gw, gb, dims, facc, fmul, fdiv)
    return gi, gw, gb


def superfp_layernorm_forward(inp, weight, bias, eps, dims, man_acc=23, exp_acc=8, binades_acc=1, man_mul=23, exp_mul=8,
                              binades_mul=1, man_div=23, exp_div=8, binades_div=1, man_sqrt=23, exp_sqrt=8, binades_sqrt=1,
                              rounding="nearest", saturate=False):
    """reference: quant_function.py:1061-1125."""
    assert rounding == "nearest", "Only nearest roudning layernorm is implemented."
    return _layernorm_fwd(inp, weight, bias, eps, dims, _sfp(man_acc, exp_acc, binades_acc, saturate), _sfp(man_mul, exp_mul, binades_mul, saturate),
                          _sfp(man_div, exp_div, binades_div, saturate), _sfp(man_sqrt, exp_sqrt, binades_sqrt, saturate))


def superfp_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, man_acc=23, exp_acc=8, binades_acc=1, man_mul=23,
                               exp_mul=8, binades_mul=1, man_div=23, exp_div=8, binades_div=1, rounding="nearest", saturate=False):
    """reference: quant_function.py:1237-1296."""
    assert rounding == "nearest", "Only nearest rounding layernorm is implemented."
    return _layernorm_bwd(inp, grad_output, weight, bias, mean, rstd, dims, _sfp(man_acc, exp_acc, binades_acc, saturate),
                          _sfp(man_mul, exp_mul, binades_mul, saturate), _sfp(man_div, exp_div, binades_div, saturate))


def binary8_layernorm_forward(inp, weight, bias, eps, dims, P_acc, op_acc, signed_acc, P_mul, op_mul, signed_mul, P_div, op_div,
                              signed_div, P_sqrt, op_sqrt, signed_sqrt, rounding, subnormals):
    """reference: quant_function.py:1128-1183 (policy names are translated here; the reference passes them through
    untranslated, which its extension rejects)."""
    assert rounding == "nearest", "Only nearest roudning layernorm is implemented."
    return _layernorm_fwd(inp, weight, bias, eps, dims, _b8(P_acc, op_acc, signed_acc, subnormals), _b8(P_mul, op_mul, signed_mul, subnormals),
                          _b8(P_div, op_div, signed_div, subnormals), _b8(P_sqrt, op_sqrt, signed_sqrt, subnormals))


def binary8_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, P_acc, op_acc, signed_acc, P_mul, op_mul, signed_mul,
                               P_div, op_div, signed_div, rounding, subnormals):
    """reference: quant_function.py:1299-1351."""
    assert rounding == "nearest", "Only nearest rounding layernorm is implemented."
    return _layernorm_bwd(inp, grad_output, weight, bias, mean, rstd, dims, _b8(P_acc, op_acc, signed_acc, subnormals),
                          _b8(P_mul, op_mul, signed_mul, subnormals), _b8(P_div, op_div, signed_div, subnormals))


def mp_softmax_forward(a: torch.Tensor, dim: int, formats) -> torch.Tensor:
    """reference: quant_function.py:382-491."""
    off_cfg = formats.fwd_off
    if type(off_cfg) == SuperNormalFloat:
        if not formats.use_lse:
            e, acc = formats.fwd_exp, formats.fwd_acc
            assert e.saturate == off_cfg.saturate and acc.saturate == off_cfg.saturate
            return superfp_softmax_forward(a, dim, e.man, e.exp, e.binades, off_cfg.man, off_cfg.exp, off_cfg.binades, acc.man,
                                           acc.exp, acc.binades, formats.fwd_rnd, off_cfg.saturate)
        l = formats.fwd_lse
        assert l.saturate == off_cfg.saturate
        return superfp_softmax_lse_forward(a, dim, off_cfg.man, off_cfg.exp, off_cfg.binades, l.man, l.exp, l.binades,
                                           formats.fwd_rnd, off_cfg.saturate)
    if type(off_cfg) == Binary8:
        if not formats.use_lse:
            e, acc = formats.fwd_exp, formats.fwd_acc
            assert e.subnormals == off_cfg.subnormals and acc.subnormals == off_cfg.subnormals
            return binary8_softmax_forward(a, dim, e.P, e.overflow_policy, e.signed, off_cfg.P, off_cfg.overflow_policy, off_cfg.signed,
                                           acc.P, acc.overflow_policy, acc.signed, formats.fwd_rnd, off_cfg.subnormals)
        l = formats.fwd_lse
        assert l.subnormals == off_cfg.subnormals
        return binary8_softmax_lse_forward(a, dim, off_cfg.P, off_cfg.overflow_policy, off_cfg.signed, l.P, l.overflow_policy, l.signed,
                                           formats.fwd_rnd, off_cfg.subnormals)
    if type(off_cfg) != FloatingPoint:
        raise NotImplementedError("Unsupported number format.")
    if not formats.use_lse:
        assert formats.fwd_exp.subnormals == off_cfg.subnormals and formats.fwd_acc.subnormals == off_cfg.subnormals
        assert formats.fwd_exp.saturate == off_cfg.saturate and formats.fwd_acc.saturate == off_cfg.saturate
        return float_softmax_forward(a, dim, formats.fwd_exp.man, formats.fwd_exp.exp, off_cfg.man, off_cfg.exp,
                                     formats.fwd_acc.man, formats.fwd_acc.exp, formats.fwd_rnd, off_cfg.subnormals,
                                     off_cfg.saturate)
    assert formats.fwd_lse.subnormals == off_cfg.subnormals
    assert formats.fwd_lse.saturate == off_cfg.saturate
    return float_softmax_lse_forward(a, dim, off_cfg.man, off_cfg.exp, formats.fwd_lse.man, formats.fwd_lse.exp,
                                     formats.fwd_rnd, off_cfg.subnormals, off_cfg.saturate)


def mp_softmax_backward(input: torch.Tensor, grad_output: torch.Tensor, dim: int, formats) -> torch.Tensor:
    """reference: quant_function.py:494-543."""
    add_cfg = formats.bwd_add
    mul_cfg = formats.bwd_mul
    if type(add_cfg) == SuperNormalFloat:
        assert mul_cfg.saturate == add_cfg.saturate
        return superfp_softmax_backward(input, grad_output, dim, add_cfg.man, add_cfg.exp, add_cfg.binades, mul_cfg.man, mul_cfg.exp,
                                        mul_cfg.binades, formats.bwd_rnd, add_cfg.saturate)
    if type(add_cfg) == Binary8:
        assert mul_cfg.subnormals == add_cfg.subnormals
        return binary8_softmax_backward(input, grad_output, dim, add_cfg.P, add_cfg.overflow_policy, add_cfg.signed, mul_cfg.P,
                                        mul_cfg.overflow_policy, mul_cfg.signed, formats.bwd_rnd, add_cfg.subnormals)
    if type(add_cfg) != FloatingPoint:
        raise NotImplementedError("Unsupported number format.")
    assert formats.bwd_mul.subnormals == add_cfg.subnormals
    assert formats.bwd_mul.saturate == add_cfg.saturate
    return float_softmax_backward(input, grad_output, dim, add_cfg.man, add_cfg.exp, formats.bwd_mul.man,
                                  formats.bwd_mul.exp, formats.bwd_rnd, add_cfg.subnormals, add_cfg.saturate)


# ------------------------------------------------------------------------------------------ layernorm
def float_layernorm_forward(inp: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, dims: list[int],
                            man_acc: int = 23, exp_acc: int = 8, man_mul: int = 23, exp_mul: int = 8, man_div: int = 23,
                            exp_div: int = 8, man_sqrt: int = 23, exp_sqrt: int = 8,
                            rounding: Literal["nearest"] = "nearest", subnormals: bool = True, saturate: bool = False):
    """Layer normalisation over the trailing ``dims``; returns (output, mean, rstd) with mean and rstd shaped
    like the leading dimensions.  reference: quant_function.py:1009-1058."""
    assert rounding == "nearest", "Only nearest roudning layernorm is implemented."
    _require_cuda(inp, "float_layernorm_forward")
    x = _f32c(inp)
    lead = list(x.shape[: x.dim() - len(dims)])
    mean = torch.empty(lead, device=x.device)
    rstd = torch.empty(lead, device=x.device)
    out = torch.empty_like(x)
    _be.float_quantize_layernorm_forward(x, _f32c(weight), _f32c(bias), out, mean, rstd, eps, dims, man_acc, exp_acc,
                                         man_mul, exp_mul, man_div, exp_div, man_sqrt, exp_sqrt, subnormals, saturate)
    return out, mean, rstd


def float_layernorm_backward(inp: torch.Tensor, grad_output: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                             mean: torch.Tensor, rstd: torch.Tensor, dims: list[int], man_acc: int = 23, exp_acc: int = 8,
                             man_mul: int = 23, exp_mul: int = 8, man_div: int = 23, exp_div: int = 8,
                             rounding: Literal["nearest"] = "nearest", subnormals: bool = True, saturate: bool = False):
    """Returns (grad_input, grad_weight, grad_bias).  reference: quant_function.py:1186-1234."""
    assert rounding == "nearest", "Only nearest rounding layernorm is implemented."
    assert inp.device == grad_output.device
    _require_cuda(inp, "float_layernorm_backward")
    x = _f32c(inp)
    grad_input = torch.empty_like(x)
    grad_weight = torch.empty_like(weight, dtype=torch.float32).contiguous()
    grad_bias = torch.empty_like(bias, dtype=torch.float32).contiguous()
    _be.float_quantize_layernorm_backward(x, _f32c(grad_output), _f32c(weight), _f32c(bias), _f32c(mean), _f32c(rstd),
                                          grad_input, grad_weight, grad_bias, dims, man_acc, exp_acc, man_mul, exp_mul,
                                          man_div, exp_div, subnormals, saturate)
    return grad_input, grad_weight, grad_bias


def mp_layernorm_forward(inp, weight, bias, eps, dims, formats):
    """reference: quant_function.py:855-930."""
    acc = formats.fwd_acc
    m, d, q = formats.fwd_mul, formats.fwd_div, formats.fwd_sqrt
    if type(acc) == SuperNormalFloat:
        return superfp_layernorm_forward(inp, weight, bias, eps, dims, acc.man, acc.exp, acc.binades, m.man, m.exp, m.binades, d.man, d.exp,
                                         d.binades, q.man, q.exp, q.binades, formats.fwd_rnd, acc.saturate)
    if type(acc) == Binary8:
        return binary8_layernorm_forward(inp, weight, bias, eps, dims, acc.P, acc.overflow_policy, acc.signed, m.P, m.overflow_policy,
                                         m.signed, d.P, d.overflow_policy, d.signed, q.P, q.overflow_policy, q.signed, formats.fwd_rnd,
                                         acc.subnormals)
    if type(acc) != FloatingPoint:
        raise NotImplementedError("Unsupported float type.")
    return float_layernorm_forward(inp, weight, bias, eps, dims, acc.man, acc.exp, formats.fwd_mul.man, formats.fwd_mul.exp,
                                   formats.fwd_div.man, formats.fwd_div.exp, formats.fwd_sqrt.man, formats.fwd_sqrt.exp,
                                   formats.fwd_rnd, acc.subnormals, acc.saturate)


def mp_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, formats):
    """reference: quant_function.py:933-1006."""
    acc = formats.bwd_acc
    m, d = formats.bwd_mul, formats.bwd_div
    if type(acc) == SuperNormalFloat:
        return superfp_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, acc.man, acc.exp, acc.binades, m.man, m.exp,
                                          m.binades, d.man, d.exp, d.binades, formats.bwd_rnd, acc.saturate)
    if type(acc) == Binary8:
        return binary8_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, acc.P, acc.overflow_policy, acc.signed, m.P,
                                          m.overflow_policy, m.signed, d.P, d.overflow_policy, d.signed, formats.bwd_rnd, acc.subnormals)
    if type(acc) != FloatingPoint:
        raise NotImplementedError("Unsupported float type.")
    return float_layernorm_backward(inp, grad_output, weight, bias, mean, rstd, dims, acc.man, acc.exp,
                                    formats.bwd_mul.man, formats.bwd_mul.exp, formats.bwd_div.man, formats.bwd_div.exp,
                                    formats.bwd_rnd, acc.subnormals, acc.saturate)


def qsum_rows(x: torch.Tensor, exp: int, man: int, subnormals: bool = True, saturate: bool = False) -> torch.Tensor:
    """Sequential rounded sum over dim 0 of a 2-D tensor (one rounding per added row), in one kernel launch.
    Equals the reference's ``qsum(x, 0, quant)`` with a nearest ``float_quantize`` (functional.py:736-748)."""
    _require_cuda(x, "qsum_rows")
    return _be.qsum_rows(_f32c(x), man, exp, subnormals, saturate)


def _outside(name):
    def fn(*args, **kwargs):
        raise NotImplementedError("%s is outside the B200 hot path" % name)

    fn.__name__ = name
    fn.__doc__ = "Present for API compatibility with the reference; not implemented on this back end."
    return fn


fxp_mm, fxp_bmm = _outside("fxp_mm"), _outside("fxp_bmm")
cublas_mm, cublas_bmm = _outside("cublas_mm"), _outside("cublas_bmm")


class cublas_acceleration:
    """reference: mptorch/quant/cublas.py:45-61.  Kept as an inert switch: tensor-core GEMMs do not round
    per MAC, so this back end never dispatches to them."""
    enabled = False
    fast_mode = None

    def __init__(self, enabled: bool, fast_mode=None):
        self.enabled_new, self.fast_new = enabled, fast_mode

    def __enter__(self):
        self.prev = (cublas_acceleration.enabled, cublas_acceleration.fast_mode)
        cublas_acceleration.enabled, cublas_acceleration.fast_mode = False, self.fast_new

    def __exit__(self, *exc):
        cublas_acceleration.enabled, cublas_acceleration.fast_mode = self.prev

    @staticmethod
    def enable(enabled: bool, fast_mode=None):
        cublas_acceleration.enabled, cublas_acceleration.fast_mode = False, fast_mode
