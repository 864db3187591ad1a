"""Autograd functions that route linear algebra, softmax and layer normalisation through the simulated
arithmetic kernels.  Semantics follow the reference's ``mptorch/quant/functional.py`` (lines cited per class),
including the order in which signals are scaled, quantized and un-scaled.
"""
from __future__ import annotations

from typing import Callable

import torch

from ..number import FloatingPoint, FloatType
from .quant_format import QAffineFormats, QLayerNormFormats, QSoftmaxFormats, id_quant, make_quant_function
from .quant_function import (mp_bmm, mp_layernorm_backward, mp_layernorm_forward, mp_mm, mp_softmax_backward,
                             mp_softmax_forward, qsum_rows)

__all__ = ["qlinear", "qconv2d", "qmm", "qmatmul", "qsoftmax", "qlayernorm", "qsum", "compute_bias", "scale", "unscale"]


# ------------------------------------------------------------------------------------------ two gradients at once
# The two GEMMs of a layer's backward pass (gradient of the input, gradient of the weight or of the other operand) do
# not depend on one another, and neither fills the GPU evenly: a [8192, 768] result is 2.59 waves of CTAs, a weight
# gradient a fraction of one wave with a long K.  Launched on two streams, the CTAs of one fill the SMs the other
# leaves idle.  The results do not change: each kernel computes what it would compute alone.
overlap_backward_gemms = True
_side_streams: dict[int, "torch.cuda.Stream"] = {}


class _second_gradient:
    """Context for the second gradient of a backward pass: on a CUDA device (and with the switch above on) its body
    runs on a side stream that starts after everything the current stream held when the object was made (so the first
    gradient, launched in between, does not hold it back); ``join`` makes the current stream wait for it and hands the
    tensors made there over to the current stream.  The host-side order of the calls, and with it the order in which
    stochastic quantizers draw their seeds, stays that of the reference."""

    def __init__(self, like: torch.Tensor, enabled: bool = True):
        self.main = self.side = None
        if enabled and overlap_backward_gemms and like.is_cuda and not torch.cuda.is_current_stream_capturing():
            dev = like.device.index if like.device.index is not None else torch.cuda.current_device()
            if dev not in _side_streams:
                _side_streams[dev] = torch.cuda.Stream(device=dev)
            self.main, self.side = torch.cuda.current_stream(like.device), _side_streams[dev]
            self.fork = self.main.record_event()

    def __enter__(self):
        if self.side is not None:
            self.side.wait_event(self.fork)
            self._ctx = torch.cuda.stream(self.side)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.side is not None:
            self._ctx.__exit__(*exc)
        return False

    def join(self, *tensors):
        if self.side is not None:
            self.main.wait_stream(self.side)
            for t in tensors:
                if t is not None:
                    t.record_stream(self.main)


# ------------------------------------------------------------------------------------------ tensor scaling
def compute_bias(x: torch.Tensor, cast_to: FloatType, margin: int) -> torch.Tensor:
    """Power-of-two exponent that maps the largest magnitude of each matrix onto ``cast_to``'s largest normal value
    (reference functional.py:39-46; log2 in float64)."""
    with torch.no_grad():
        amax = x.abs().amax(dim=-1, keepdim=True).amax(dim=-2, keepdim=True)
    return torch.floor(torch.log2(cast_to.normal_max / amax.double())).float() - margin


def scale(x: torch.Tensor, x_scale) -> torch.Tensor:
    """x * 2^x_scale (reference functional.py:49-53)."""
    if isinstance(x_scale, torch.Tensor):
        return x * torch.pow(2.0 * torch.ones_like(x), x_scale)
    return x * 2 ** x_scale


def unscale(x: torch.Tensor, x_scale) -> torch.Tensor:
    """x * 2^-x_scale (reference functional.py:56-60)."""
    if isinstance(x_scale, torch.Tensor):
        return x * torch.pow(2.0 * torch.ones_like(x), -x_scale)
    return x * 2 ** (-x_scale)


def _unscale(x, x_scale):
    """``unscale`` inside the layers: a scale of exactly 0 (no tensor scaling) multiplies by one, which leaves every
    value as it is, so the elementwise kernel is skipped."""
    return x if (isinstance(x_scale, int) and x_scale == 0) else unscale(x, x_scale)


def _float_nearest_spec(quant):
    """What ``quant`` does, when a kernel can do it too: "identity", (man, exp, subnormals, saturate) for a float format
    rounded to nearest, or None for anything else (stochastic rounding, other format families, user callables)."""
    if quant is id_quant:
        return "identity"
    num, rnd = getattr(quant, "forward_number", 0), getattr(quant, "forward_rounding", None)
    if num is None:
        return "identity"
    if isinstance(num, FloatingPoint) and rnd == "nearest":
        return (num.man, num.exp, num.subnormals, num.saturate)
    return None


def _scaled_quant(x, scaled_format, margin, quant):
    """(quant(scale(x, s)), s) with s = compute_bias(x, scaled_format, margin): two kernels (row maxima, then scale and
    round) instead of the reference's two reductions, five elementwise kernels and the quantizer launch, same bits."""
    spec = _float_nearest_spec(quant)
    if spec is not None and x.is_cuda and x.dim() >= 2 and x.dtype == torch.float32:
        from .. import backend as _be

        return _be.scale_quantize(x.contiguous(), scaled_format.normal_max, margin, None if spec == "identity" else spec)
    s = compute_bias(x, scaled_format, margin)
    return quant(scale(x, s)), s


def _quantize_operands(ctx, formats, a, b):
    """The scaled and quantized operands of a layer's forward GEMM; records the scales on ``ctx``."""
    if formats.weight_scaled_format and formats.input_scaled_format and formats.use_scaling:
        qb, ctx.weight_scale = _scaled_quant(b, formats.weight_scaled_format, formats.scale_margin, formats.weight_quant)
        qa, ctx.input_scale = _scaled_quant(a, formats.input_scaled_format, formats.scale_margin, formats.input_quant)
        return qa, qb
    ctx.input_scale, ctx.weight_scale = 0, 0
    return formats.input_quant(a), formats.weight_quant(b)


def _quantize_grad(formats, grad_output):
    """(quantized, possibly scaled, output gradient; its scale)."""
    if formats.grad_scaled_format and formats.use_scaling:
        return _scaled_quant(grad_output, formats.grad_scaled_format, formats.scale_margin, formats.grad_quant)
    return formats.grad_quant(grad_output), 0


# ------------------------------------------------------------------------------------------ quantized sums
def qsum_1d(x: torch.Tensor, dim: int, quant: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """Sequential sum along ``dim`` with ``quant`` applied after every addition, starting from zero
    (reference functional.py:736-748: one quantize call per slice)."""
    acc = torch.zeros_like(x.select(dim, 0)).unsqueeze(dim)
    for k in range(x.shape[dim]):
        acc = quant(acc + x.narrow(dim, k, 1))
    return acc


def _qsum_dims_fast(x: torch.Tensor, dims, fmt: FloatingPoint) -> torch.Tensor:
    """The same left-to-right rounded sums over leading dimensions, one kernel launch per reduced dimension
    instead of one quantize launch per slice."""
    out = x
    for d in dims:   # leading dims, reduced in the given order; each reduction keeps the dim (size 1)
        moved = out.movedim(d, 0).contiguous()
        rows = moved.shape[0]
        flat = qsum_rows(moved.reshape(rows, -1), fmt.exp, fmt.man, fmt.subnormals, fmt.saturate)
        out = flat.reshape((1,) + tuple(moved.shape[1:])).movedim(0, d)
    return out


class qsum_kernel(torch.autograd.Function):
    """reference functional.py:751-783."""

    @staticmethod
    def forward(ctx, x, quant, dim=0, keepdim=False):
        ctx.save_for_backward(x)
        if dim is None:
            dim = tuple(range(x.dim()))
        elif not isinstance(dim, tuple):
            dim = (dim,)
        ctx.dim = dim
        sums = x
        for d in dim:
            sums = qsum_1d(sums, d, quant)
        if keepdim is False:
            for _ in dim:
                idx = 0
                while sums.shape[idx] != 1:
                    idx += 1
                sums = torch.squeeze(sums, dim=idx)
        return sums

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        for d in ctx.dim:
            grad_output = torch.unsqueeze(grad_output, d)
        return grad_output * torch.ones_like(x), None, None, None


def qsum(x: torch.Tensor, dim=None, quant: Callable[[torch.Tensor], torch.Tensor] = lambda x: x, keepdim: bool = False):
    """Sum with a quantization after every addition (reference functional.py:786-804)."""
    return qsum_kernel.apply(x, quant, dim, keepdim)


# ------------------------------------------------------------------------------------------ linear
class qlinear_kernel(torch.autograd.Function):
    """y = x W^T + b with per-MAC rounded GEMMs forward and backward (reference functional.py:66-173)."""

    @staticmethod
    def forward(ctx, input, weight, bias, formats):
        ctx.formats = formats
        qinput, qweight = _quantize_operands(ctx, formats, input, weight)
        qbias = formats.bias_quant(bias) if bias is not None else None
        if formats.fwd_use_default_prec:
            with torch.no_grad():
                output = torch.nn.functional.linear(qinput, qweight)
        else:
            output = mp_bmm(qinput, qweight.t(), formats, use_forward=True)
        output = _unscale(output, ctx.input_scale + ctx.weight_scale)
        if qbias is not None:
            output += qbias.view(-1, qbias.shape[-1])     # plain fp32 add; rounding is left to output_quant
        ctx.save_for_backward(qinput, qweight, qbias)
        return formats.output_quant(output)

    @staticmethod
    def backward(ctx, grad_output):
        qinput, qweight, qbias = ctx.saved_tensors
        f = ctx.formats
        qgrad_input = qgrad_weight = qgrad_bias = None
        qgrad_output, grad_scale = _quantize_grad(f, grad_output)
        second = _second_gradient(qgrad_output, ctx.needs_input_grad[0] and ctx.needs_input_grad[1])
        if ctx.needs_input_grad[0]:
            if f.bwd_use_default_prec:
                qgrad_input = torch.matmul(qgrad_output, qweight)
            else:
                qgrad_input = mp_bmm(qgrad_output, qweight, formats=f, use_forward=False)
            qgrad_input = f.grad_quant(_unscale(qgrad_input, grad_scale + ctx.weight_scale))
        if ctx.needs_input_grad[1]:
            with second:
                if f.bwd_use_default_prec:
                    qgrad_weight = torch.matmul(qgrad_output.transpose(-2, -1), qinput)
                else:
                    # for >2-D inputs this is a batched GEMM; autograd sums the [batch, out, in] result over the batch
                    # in plain fp32 when it reduces the gradient to the weight's shape, exactly as in the reference
                    qgrad_weight = mp_bmm(qgrad_output.transpose(-2, -1), qinput, formats=f, use_forward=False)
                qgrad_weight = f.grad_quant(_unscale(qgrad_weight, grad_scale + ctx.input_scale))
        second.join(qgrad_weight)
        if qbias is not None and ctx.needs_input_grad[2]:
            lead = tuple(range(qgrad_output.dim() - 1))
            if f.bwd_use_default_prec:
                qgrad_bias = qgrad_output.sum(dim=lead).reshape(qbias.shape)
            else:
                with torch.no_grad():
                    if isinstance(f.bwd_add, FloatingPoint) and f.bwd_rnd == "nearest" and qgrad_output.is_cuda:
                        qgrad_bias = _qsum_dims_fast(qgrad_output, lead, f.bwd_add).reshape(qbias.shape)
                    else:
                        qgrad_bias = qsum(qgrad_output, dim=lead,
                                          quant=make_quant_function(f.bwd_add, f.bwd_rnd, f.rbits_add)).reshape(qbias.shape)
            qgrad_bias = f.grad_quant(_unscale(qgrad_bias, grad_scale))
        return qgrad_input, qgrad_weight, qgrad_bias, None, None


def qlinear(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
            formats: QAffineFormats = QAffineFormats()) -> torch.Tensor:
    """Functional form of ``QLinear`` (reference functional.py:176-208)."""
    return qlinear_kernel.apply(input, weight, bias, formats)


# ------------------------------------------------------------------------------------------ convolution
def _conv_cols(x, kernel_size, dilation, padding, stride):
    """[N, C, H, W] -> [N * L, C * kh * kw], K ordered channel, kernel row, kernel column (reference conv.py:591-617)."""
    cols = torch.nn.functional.unfold(x, kernel_size, dilation=dilation, padding=padding, stride=stride)
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


def implicit_conv_eligible(formats, input) -> bool:
    """The implicit-GEMM path gives the bits of the unfold + GEMM composition when the forward MACs are float formats
    with nearest rounding (plain or compensated sums excluded), no tensor scaling is in play, and the input quantizer
    rounds deterministically (a stochastic one would draw once per input element instead of once per unfolded copy)."""
    if not input.is_cuda or formats.fwd_use_default_prec or formats.use_scaling or formats.compensated:
        return False
    if formats.fwd_rnd != "nearest" or not isinstance(formats.fwd_add, FloatingPoint) or not isinstance(formats.fwd_mul, FloatingPoint):
        return False
    iq = formats.input_quant
    return iq is id_quant or getattr(iq, "forward_number", 0) is None or getattr(iq, "forward_rounding", None) == "nearest"


def implicit_wgrad_eligible(formats) -> bool:
    """The weight gradient can be taken by the implicit GEMM (no unfolded input) when the backward MACs are float
    formats rounded to nearest without compensation and the gradient quantizer is deterministic (a stochastic one would
    draw once per gradient element here and once per (group, element) in the per-group composition)."""
    if formats.bwd_use_default_prec or formats.compensated or formats.bwd_rnd != "nearest":
        return False
    if not isinstance(formats.bwd_add, FloatingPoint) or not isinstance(formats.bwd_mul, FloatingPoint):
        return False
    return _float_nearest_spec(formats.grad_quant) is not None


class qconv2d_kernel(torch.autograd.Function):
    """Zero-padded 2-D convolution whose forward pass is one implicit GEMM per group on the NCHW input
    (``mpt_float_conv2d_nearest``): the unfolded input, nine times the input for a 3x3 kernel, is neither built nor
    kept for the backward pass.  The weight gradient is an implicit GEMM as well (``mpt_float_conv2d_wgrad_nearest``: the
    NCHW output gradient against the input gathered on the fly) whenever ``implicit_wgrad_eligible``; otherwise, and for
    the input gradient, the backward pass unfolds the saved (already quantized) input and runs the GEMMs of
    ``qlinear_kernel.backward`` per group.  Either way the gradients equal those of the unfold + ``qlinear`` composition
    bit for bit (reference: modules/conv.py:537-640 with functional.py:66-173)."""

    @staticmethod
    def forward(ctx, input, weight, bias, formats, stride, padding, dilation, groups):
        from .. import backend as _be

        ctx.formats, ctx.geom = formats, (stride, padding, dilation, groups)
        qinput = formats.input_quant(input).contiguous()
        qweight = formats.weight_quant(weight)
        qbias = formats.bias_quant(bias) if bias is not None else None
        n, c, h, w = qinput.shape
        c_out, cg, kh, kw = qweight.shape
        oh = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
        ow = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
        wt = qweight.reshape(groups, c_out // groups, cg * kh * kw).transpose(1, 2).contiguous()
        out = torch.empty(n, c_out, oh, ow, device=input.device)
        add, mul = formats.fwd_add, formats.fwd_mul
        _be.float_conv2d_nearest(qinput.float(), wt.float(), out, groups, (kh, kw), stride, padding, dilation, add.man, add.exp,
                                 mul.man, mul.exp, add.subnormals, add.saturate, fma=formats.fwd_fma)
        if qbias is not None:
            out += qbias.view(1, -1, 1, 1)               # plain fp32 add; rounding is left to output_quant, as in qlinear
        ctx.save_for_backward(qinput, qweight, qbias)
        return formats.output_quant(out)

    @staticmethod
    def backward(ctx, grad_output):
        qinput, qweight, qbias = ctx.saved_tensors
        f = ctx.formats
        stride, padding, dilation, groups = ctx.geom
        n, c, h, w = qinput.shape
        c_out, cg, kh, kw = qweight.shape
        og = c_out // groups
        grad_scale = 0                # the implicit path is taken only without tensor scaling (implicit_conv_eligible)
        gin, gws, gbs = [], [], []
        implicit_w = ctx.needs_input_grad[1] and implicit_wgrad_eligible(f)
        # the implicit weight gradient runs beside the per-group input gradients (its quantizer is deterministic, so
        # the order of the calls does not matter to any random stream)
        second = _second_gradient(grad_output, bool(implicit_w and ctx.needs_input_grad[0]))
        if implicit_w:
            from .. import backend as _be

            with second:
                qgo_all = f.grad_quant(grad_output).contiguous().float()     # elementwise: the values the per-group path sees
                gw_all = torch.empty(c_out, cg * kh * kw, device=grad_output.device)
                _be.float_conv2d_wgrad_nearest(qgo_all, qinput.float(), gw_all, groups, (kh, kw), stride, padding, dilation,
                                               f.bwd_add.man, f.bwd_add.exp, f.bwd_mul.man, f.bwd_mul.exp, f.bwd_add.subnormals,
                                               f.bwd_add.saturate, fma=f.bwd_fma)
                gws.append(f.grad_quant(gw_all).view(c_out, cg, kh, kw))
        for g in range(groups):
            go = grad_output[:, g * og:(g + 1) * og]
            go2 = go.reshape(n, og, -1).transpose(1, 2).reshape(-1, og)              # [N * L, og], as qlinear sees it
            qgo = f.grad_quant(go2)
            w2 = qweight[g * og:(g + 1) * og].reshape(og, -1)
            if ctx.needs_input_grad[0]:
                gc = torch.matmul(qgo, w2) if f.bwd_use_default_prec else mp_bmm(qgo, w2, formats=f, use_forward=False)
                gc = f.grad_quant(gc)
                gc = gc.view(n, -1, gc.shape[-1]).transpose(1, 2)                    # [N, K, L]
                gin.append(torch.nn.functional.fold(gc, (h, w), (kh, kw), dilation=dilation, padding=padding, stride=stride))
            if ctx.needs_input_grad[1] and not implicit_w:
                cols = _conv_cols(qinput[:, g * cg:(g + 1) * cg], (kh, kw), dilation, padding, stride)
                gw = (torch.matmul(qgo.transpose(-2, -1), cols) if f.bwd_use_default_prec
                      else mp_bmm(qgo.transpose(-2, -1), cols, formats=f, use_forward=False))
                gws.append(f.grad_quant(gw).view(og, cg, kh, kw))
            if qbias is not None and ctx.needs_input_grad[2]:
                if f.bwd_use_default_prec:
                    gb = qgo.sum(dim=0)
                else:
                    with torch.no_grad():
                        if isinstance(f.bwd_add, FloatingPoint) and f.bwd_rnd == "nearest":
                            gb = _qsum_dims_fast(qgo, (0,), f.bwd_add)
                        else:
                            gb = qsum(qgo, dim=(0,), quant=make_quant_function(f.bwd_add, f.bwd_rnd, f.rbits_add))
                gbs.append(f.grad_quant(gb.reshape(-1)))
        second.join(*gws)
        grad_input = torch.cat(gin, dim=1) if gin else None
        grad_weight = torch.cat(gws, dim=0) if gws else None
        grad_bias = torch.cat(gbs, dim=0) if gbs else None
        return grad_input, grad_weight, grad_bias, None, None, None, None, None


def qconv2d(input, weight, bias, formats, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    """Functional zero-padded 2-D convolution through the implicit GEMM; see ``implicit_conv_eligible`` for when the
    module uses it."""
    return qconv2d_kernel.apply(input, weight, bias, formats, tuple(stride), tuple(padding), tuple(dilation), groups)


# ------------------------------------------------------------------------------------------ mm / matmul
def _matmul_function(fwd_default, mp_fn, name, requantize_unscaled):
    class kernel(torch.autograd.Function):
        @staticmethod
        def forward(ctx, input, other, formats):
            ctx.formats = formats
            qinput, qother = _quantize_operands(ctx, formats, input, other)
            if formats.fwd_use_default_prec:
                with torch.no_grad():
                    output = fwd_default(qinput, qother)
            else:
                output = mp_fn(qinput, qother, formats=formats, use_forward=True)
            output = _unscale(output, ctx.input_scale + ctx.weight_scale)
            ctx.save_for_backward(qinput, qother)
            return formats.output_quant(output)

        @staticmethod
        def backward(ctx, grad_output):
            qinput, qother = ctx.saved_tensors
            f = ctx.formats
            qgrad_input = qgrad_other = None
            qgrad_output, grad_scale = _quantize_grad(f, grad_output)
            second = _second_gradient(qgrad_output, ctx.needs_input_grad[0] and ctx.needs_input_grad[1])
            if ctx.needs_input_grad[0]:
                if f.bwd_use_default_prec:
                    g = fwd_default(qgrad_output, qother.transpose(-2, -1))
                else:
                    g = mp_fn(qgrad_output, qother.transpose(-2, -1), formats=f, use_forward=False)
                # the reference's qmm quantizes the un-unscaled gradient (functional.py:270-272); qmatmul the unscaled one
                qgrad_input = f.grad_quant(_unscale(g, grad_scale + ctx.weight_scale) if requantize_unscaled else g)
            if ctx.needs_input_grad[1]:
                with second:
                    if f.bwd_use_default_prec:
                        g = fwd_default(qinput.transpose(-2, -1), qgrad_output)
                    else:
                        g = mp_fn(qinput.transpose(-2, -1), qgrad_output, formats=f, use_forward=False)
                    qgrad_other = f.grad_quant(_unscale(g, grad_scale + ctx.input_scale) if requantize_unscaled else g)
            second.join(qgrad_other)
            return qgrad_input, qgrad_other, None

    kernel.__name__ = name
    return kernel


qmm_kernel = _matmul_function(torch.mm, mp_mm, "qmm_kernel", False)            # reference functional.py:211-290
qmatmul_kernel = _matmul_function(torch.matmul, mp_bmm, "qmatmul_kernel", True)  # reference functional.py:320-401


def qmm(input: torch.Tensor, mat2: torch.Tensor, formats: QAffineFormats = QAffineFormats()) -> torch.Tensor:
    """(n, m) x (m, p) product through the simulated GEMM (reference functional.py:293-317)."""
    return qmm_kernel.apply(input, mat2, formats)


def qmatmul(input: torch.Tensor, other: torch.Tensor, formats: QAffineFormats = QAffineFormats()) -> torch.Tensor:
    """Batched product for the shape cases of ``float_bmm`` (reference functional.py:404-446)."""
    return qmatmul_kernel.apply(input, other, formats)


# ------------------------------------------------------------------------------------------ softmax
class qsoftmax_kernel(torch.autograd.Function):
    """reference functional.py:1024-1058."""

    @staticmethod
    def forward(ctx, a, dim, formats):
        ctx.formats, ctx.dim = formats, dim
        qinput = formats.input_quant(a)
        if formats.fwd_use_default_prec:
            with torch.no_grad():
                output = torch.nn.functional.softmax(qinput, dim)
        else:
            output = mp_softmax_forward(qinput, dim, formats)
        qoutput = formats.output_quant(output)
        ctx.save_for_backward(qoutput)
        return qoutput

    @staticmethod
    def backward(ctx, grad_output):
        (qoutput,) = ctx.saved_tensors
        f = ctx.formats
        qgrad_output = f.grad_quant(grad_output)
        if f.bwd_use_default_prec:
            weighted = torch.sum(qoutput * qgrad_output, dim=ctx.dim, keepdim=True)
            grad_input = qoutput * (qgrad_output - weighted)
        else:
            grad_input = mp_softmax_backward(qoutput, qgrad_output, ctx.dim, f)
        return f.grad_quant(grad_input), None, None


def qsoftmax(input: torch.Tensor, dim: int, formats: QSoftmaxFormats) -> torch.Tensor:
    """Functional form of ``QSoftmax`` (reference functional.py:1061-1091)."""
    return qsoftmax_kernel.apply(input, dim, formats)


# ------------------------------------------------------------------------------------------ layernorm
class qlayernorm_kernel(torch.autograd.Function):
    """reference functional.py:876-969."""

    @staticmethod
    def forward(ctx, x, normalized_shape, weight, bias, eps, formats):
        ctx.formats, ctx.eps = formats, eps
        qinput = formats.input_quant(x)
        qweight = formats.weight_quant(weight) if weight is not None else torch.ones(normalized_shape, device=x.device)
        qbias = formats.bias_quant(bias) if bias is not None else torch.zeros(normalized_shape, device=x.device)
        if isinstance(normalized_shape, int):
            normalized_shape = torch.Size([normalized_shape])
        elif isinstance(normalized_shape, list):
            normalized_shape = torch.Size(normalized_shape)
        assert isinstance(normalized_shape, torch.Size)
        assert normalized_shape == x.shape[-len(normalized_shape):]
        dims = [-(i + 1) for i in range(len(normalized_shape))]
        ctx.dims = dims
        if formats.fwd_use_default_prec:
            C = qweight.numel()
            mean = x.sum(dims, keepdim=True) / C
            xshift = x - mean
            rstd = ((xshift ** 2).sum(dims, keepdim=True) / C + eps) ** -0.5
            output = xshift * rstd * qweight + qbias
        else:
            output, mean, rstd = mp_layernorm_forward(qinput, qweight, qbias, eps, dims, formats)
        ctx.save_for_backward(qinput, qweight, qbias, mean, rstd)
        return formats.output_quant(output)

    @staticmethod
    def backward(ctx, grad_output):
        qinput, qweight, qbias, mean, rstd = ctx.saved_tensors
        f, dims = ctx.formats, ctx.dims
        qgrad_output = f.grad_quant(grad_output)
        if f.bwd_use_default_prec:
            lead = tuple(range(qinput.dim() - len(dims)))
            m = mean.reshape(mean.shape[:len(lead)] + (1,) * len(dims)) if mean.dim() == len(lead) else mean
            r = rstd.reshape(m.shape) if rstd.dim() == len(lead) else rstd
            norm = (qinput - m) * r
            grad_bias = grad_output.sum(lead)
            grad_weight = (grad_output * norm).sum(lead)
            grad_norm = grad_output * qweight
            grad_input = (grad_norm - grad_norm.mean(dims, keepdim=True)
                          - norm * (grad_norm * norm).mean(dims, keepdim=True)) * r
        else:
            grad_input, grad_weight, grad_bias = mp_layernorm_backward(qinput, qgrad_output, qweight, qbias, mean, rstd, dims, f)
        qgi = f.grad_quant(grad_input) if ctx.needs_input_grad[0] else None
        qgw = f.grad_quant(grad_weight) if ctx.needs_input_grad[2] else None
        qgb = f.grad_quant(grad_bias) if ctx.needs_input_grad[3] else None
        return qgi, None, qgw, qgb, None, None


def qlayernorm(x: torch.Tensor, normalized_shape, weight: torch.Tensor | None, bias: torch.Tensor | None, eps: float,
               formats: QLayerNormFormats) -> torch.Tensor:
    """Functional form of ``QLayerNorm`` (reference functional.py:972-1021)."""
    return qlayernorm_kernel.apply(x, normalized_shape, weight, bias, eps, formats)
