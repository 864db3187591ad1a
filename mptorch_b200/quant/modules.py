"""``nn.Module`` layers whose arithmetic runs through the simulated low-precision kernels.

Subclasses of the corresponding ``torch.nn`` layers (so ``state_dict`` layouts are unchanged), with the constructor
arguments and behaviour of the reference's ``mptorch/quant/modules``: ``QLinear`` (linear.py:12-135), ``QSoftmax``
(softmax.py:14-94), ``QLayerNorm`` (layernorm.py:13-172), ``QConv2d`` (conv.py:326-640, as unfold + qlinear) and
``Quantizer`` (quantizer.py:8).  Transposed / 1-D / 3-D convolutions, batch norm, GELU and pooling of the reference
are not on the accelerated path and are not provided.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..number import Number
from .functional import implicit_conv_eligible, qconv2d, qlayernorm, qlinear, qsoftmax
from .quant_format import QAffineFormats, QLayerNormFormats, QSoftmaxFormats
from .quant_function import quantizer

__all__ = ["Quantizer", "QLinear", "QLazyLinear", "QConv2d", "QLayerNorm", "QSoftmax"]


def ste_function(fwd_quant: Callable[[torch.Tensor], torch.Tensor], bwd_quant: Callable[[torch.Tensor], torch.Tensor]):
    """Straight-through estimator: ``fwd_quant`` on the way forward, ``bwd_quant`` on the gradient."""

    class round(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return fwd_quant(x) if x is not None else x

        @staticmethod
        def backward(ctx, grad_output):
            return bwd_quant(grad_output)

    return round.apply


class _QuantSignals:
    """Mixin holding the Qw/Qb/Qi/Qo straight-through quantizers derived from ``self.formats``."""

    def reset_quant_function(self):
        f = self.formats
        if hasattr(f, "weight_quant"):
            self.Qw = ste_function(f.weight_quant, f.grad_quant)
            self.Qb = ste_function(f.bias_quant, f.grad_quant)
        self.Qi = ste_function(f.input_quant, f.grad_quant)
        self.Qo = ste_function(f.output_quant, f.grad_quant)

    def quant_function(self, fwd_quant, bwd_quant):
        return ste_function(fwd_quant, bwd_quant)

    def quant_parameters(self):
        """Quantize weight and bias in place with ``formats.weight_quant`` / ``formats.bias_quant``."""
        if getattr(self, "weight", None) is not None:
            self.weight.data = self.formats.weight_quant(self.weight.data)
        if getattr(self, "bias", None) is not None:
            self.bias.data = self.formats.bias_quant(self.bias.data)


class Quantizer(nn.Module):
    """Quantizes activations forward and gradients backward (reference modules/quantizer.py:8-60)."""

    def __init__(self, forward_number: Number | None = None, backward_number: Number | None = None,
                 forward_rounding: str = "stochastic", backward_rounding: str = "stochastic"):
        super().__init__()
        self.quantize = quantizer(forward_number, backward_number, forward_rounding, backward_rounding)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.quantize(x)


class QLinear(nn.Linear, _QuantSignals):
    """``nn.Linear`` whose forward and backward GEMMs round every multiply and add to ``formats``."""

    def __init__(self, in_features: int, out_features: int, formats: QAffineFormats, bias: bool = True) -> None:
        super().__init__(in_features, out_features, bias)
        self.formats = formats
        self.reset_quant_function()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.formats.fwd_use_default_prec and self.formats.bwd_use_default_prec:
            return self.Qo(F.linear(self.Qi(input), self.Qw(self.weight), self.Qb(self.bias)))
        return qlinear(input, self.weight, self.bias, self.formats)


class QLazyLinear(nn.modules.lazy.LazyModuleMixin, QLinear):
    """``QLinear`` with ``in_features`` inferred at the first call (reference modules/linear.py:138-201)."""

    cls_to_become = QLinear
    weight: nn.parameter.UninitializedParameter
    bias: nn.parameter.UninitializedParameter

    def __init__(self, out_features: int, formats: QAffineFormats, bias: bool = True, device=None, dtype=None) -> None:
        factory = {"device": device, "dtype": dtype}
        super().__init__(0, 0, formats, False)
        self.weight = nn.parameter.UninitializedParameter(**factory)
        self.out_features = out_features
        if bias:
            self.bias = nn.parameter.UninitializedParameter(**factory)

    def reset_parameters(self) -> None:
        if not self.has_uninitialized_params() and self.in_features != 0:
            super().reset_parameters()

    def initialize_parameters(self, input) -> None:
        if self.has_uninitialized_params():
            with torch.no_grad():
                self.in_features = input.shape[-1]
                self.weight.materialize((self.out_features, self.in_features))
                if self.bias is not None:
                    self.bias.materialize((self.out_features,))
                self.reset_parameters()


class QConv2d(nn.Conv2d, _QuantSignals):
    """``nn.Conv2d`` computed as im2col followed by the simulated GEMM, group by group.

    The unfolded K ordering is channel-major then kernel row, kernel column (``F.unfold``), the same as the
    reference's ``unfoldNd`` (conv.py:591-617), so each output sees its products in the same order."""

    def __init__(self, in_channels, out_channels, kernel_size, formats: QAffineFormats, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, padding_mode: str = "zeros") -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode)
        self.formats = formats
        self.params_are_quantized = False
        self.reset_quant_function()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if not self.params_are_quantized:
            self.quant_parameters()
            self.params_are_quantized = True
        f = self.formats
        if f.fwd_use_default_prec:
            if self.padding_mode != "zeros":
                x = F.pad(self.Qi(input), self._reversed_padding_repeated_twice, mode=self.padding_mode)
                return self.Qo(F.conv2d(x, self.Qw(self.weight), self.Qb(self.bias), self.stride, (0, 0), self.dilation, self.groups))
            return self.Qo(F.conv2d(self.Qi(input), self.Qw(self.weight), self.Qb(self.bias), self.stride, self.padding,
                                    self.dilation, self.groups))
        if implicit_conv_eligible(f, input) and not isinstance(self.padding, str):
            # one implicit GEMM per group on the NCHW input: same products in the same order, no unfolded tensor
            if self.padding_mode != "zeros":
                x = F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode)
                return qconv2d(x, self.weight, self.bias, f, self.stride, (0, 0), self.dilation, self.groups)
            return qconv2d(input, self.weight, self.bias, f, self.stride, self.padding, self.dilation, self.groups)
        batch, in_channel, in_h, in_w = input.shape
        num_filter, _, kh, kw = self.weight.shape
        pad = self.padding if not isinstance(self.padding, str) else (0, 0)
        out_h = (in_h + 2 * pad[0] - self.dilation[0] * (kh - 1) - 1) // self.stride[0] + 1
        out_w = (in_w + 2 * pad[1] - self.dilation[1] * (kw - 1) - 1) // self.stride[1] + 1

        def group_conv(X, W, b):
            if self.padding_mode != "zeros":
                X = F.pad(X, self._reversed_padding_repeated_twice, mode=self.padding_mode)
                cols = F.unfold(X, self.kernel_size, dilation=self.dilation, padding=(0, 0), stride=self.stride)
            else:
                cols = F.unfold(X, self.kernel_size, dilation=self.dilation, padding=pad, stride=self.stride)
            cols = cols.transpose(1, 2).contiguous()                    # [batch, L, C*kh*kw]
            n, L, k = cols.shape
            y = qlinear(cols.view(n * L, k), W.reshape(W.size(0), -1).contiguous(), b, f).view(n, L, -1)
            return y.transpose(1, 2).reshape(batch, -1, out_h, out_w)

        gc, gf = in_channel // self.groups, num_filter // self.groups
        outs = [group_conv(input[:, i * gc:(i + 1) * gc], self.weight[i * gf:(i + 1) * gf],
                           None if self.bias is None else self.bias[i * gf:(i + 1) * gf]) for i in range(self.groups)]
        return outs[0] if self.groups == 1 else torch.cat(outs, dim=1)


class QSoftmax(nn.Softmax, _QuantSignals):
    """``nn.Softmax`` with rounded subtraction, exponential and accumulation (or the log-sum-exp form)."""

    def __init__(self, dim: int, formats: QSoftmaxFormats) -> None:
        super().__init__(dim)
        self.formats = formats
        self.reset_quant_function()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.formats.fwd_use_default_prec and self.formats.bwd_use_default_prec:
            return self.Qo(F.softmax(self.Qi(input), dim=self.dim))
        return qsoftmax(input, dim=self.dim, formats=self.formats)


class QLayerNorm(nn.LayerNorm, _QuantSignals):
    """``nn.LayerNorm`` with rounded accumulations, multiplies, divisions and square root."""

    def __init__(self, normalized_shape, formats: QLayerNormFormats, eps: float = 1e-5, elementwise_affine: bool = True,
                 bias: bool = True) -> None:
        super().__init__(normalized_shape, eps, elementwise_affine, bias)
        self.formats = formats
        self.quant_parameters()
        self.reset_quant_function()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.formats.fwd_use_default_prec and self.formats.bwd_use_default_prec:
            return self.Qo(F.layer_norm(self.Qi(input), list(self.normalized_shape), self.Qw(self.weight), self.Qb(self.bias), self.eps))
        return qlayernorm(input, normalized_shape=list(self.normalized_shape), weight=self.weight, bias=self.bias,
                          eps=self.eps, formats=self.formats)
