"""Format/configuration objects for the quantized layers (pure Python; no arithmetic).

Same classes, constructor arguments and attributes as the reference's ``mptorch/quant/quant_format.py``
(``make_quant_function`` :19-44, ``QAffineFormats`` :47-230, ``QLayerNormFormats`` :233-329, ``QSoftmaxFormats``
:332-447, ``QGELUFormats`` :450-473).
"""
from __future__ import annotations

from typing import Callable

import torch

from ..number import Binary8, BlockFloatingPoint, FixedPoint, FloatingPoint, FloatType, Number, SuperNormalFloat
from .quant_function import binary8_quantize, block_quantize, fixed_point_quantize, float_quantize, superfp_quantize

__all__ = ["QAffineFormats", "QSoftmaxFormats", "QLayerNormFormats", "QGELUFormats", "make_quant_function"]


def id_quant(x):
    return x


def make_quant_function(num: Number, rounding: str, prng_bits: int = 0) -> Callable:
    """A tensor -> tensor quantizer for ``num`` with the given rounding.  Float quantizers carry what they do as
    attributes (``forward_number``, ``forward_rounding``), so that callers which can fuse them into a larger kernel
    (tensor scaling, the implicit convolution) recognise them."""
    if isinstance(num, FloatingPoint):
        def q(x):
            return float_quantize(x, num.exp, num.man, rounding, num.subnormals, num.saturate, prng_bits)

        q.forward_number, q.forward_rounding = num, rounding
        return q
    if isinstance(num, FixedPoint):
        return lambda x: fixed_point_quantize(x, num.wl, num.fl, num.clamp, num.symmetric, rounding)
    if isinstance(num, SuperNormalFloat):
        return lambda x: superfp_quantize(x, num.exp, num.man, num.binades, rounding, num.saturate)
    if isinstance(num, BlockFloatingPoint):
        return lambda x: block_quantize(x, num.wl, num.dim, rounding)
    if isinstance(num, Binary8):
        return lambda x: binary8_quantize(x, num.P, rounding, num.overflow_policy, num.signed, num.subnormals, prng_bits)
    raise NotImplementedError


def _split_mac(mac):
    """(add, mul, fma) from a MAC spec: one format means fused multiply-add, a pair is (add, mul)."""
    if not isinstance(mac, tuple):
        mac = (mac,)
    if len(mac) > 1:
        return mac[0], mac[1], False
    if len(mac) == 1:
        return mac[0], mac[0], True
    return None, None, False


class QAffineFormats:
    """Formats for linear / convolution / matmul layers: MAC formats for the forward and backward GEMMs
    (``(add, mul)`` tuple, or a single format for FMA), rounding modes, signal quantizers (a callable, or a
    ``(Number, rounding)`` pair), Kahan compensation, optional tensor scaling, and random bits for
    stochastic rounding."""

    def __init__(self, fwd_mac=None, bwd_mac=None, fwd_rnd: str | None = None, bwd_rnd: str | None = None,
                 weight_quant=id_quant, bias_quant=id_quant, input_quant=id_quant, output_quant=id_quant,
                 grad_quant=id_quant, compensated: bool | None = None, use_scaling: bool = False,
                 weight_scaled_format: FloatType | None = None, input_scaled_format: FloatType | None = None,
                 grad_scaled_format: FloatType | None = None, scale_margin: int = 0, rbits=0) -> None:
        self.fwd_use_default_prec = fwd_mac is None
        if fwd_mac is not None:
            self.fwd_add, self.fwd_mul, self.fwd_fma = _split_mac(fwd_mac)
        self.bwd_use_default_prec = bwd_mac is None
        if bwd_mac is not None:
            self.bwd_add, self.bwd_mul, self.bwd_fma = _split_mac(bwd_mac)
        self.fwd_rnd = fwd_rnd if (fwd_rnd or not fwd_mac) else "nearest"
        self.bwd_rnd = bwd_rnd if (bwd_rnd or not bwd_mac) else "nearest"
        if isinstance(rbits, tuple):
            self.rbits_add, self.rbits_mul = (rbits[0], rbits[1]) if len(rbits) > 1 else (rbits[0], rbits[0])
        else:
            self.rbits_add = self.rbits_mul = rbits
        self.compensated = compensated
        self.weight_scaled_format = weight_scaled_format
        self.input_scaled_format = input_scaled_format
        self.grad_scaled_format = grad_scaled_format

        def resolve(spec, scaled_attr=None):
            if isinstance(spec, tuple):
                num, rnd = spec
                if scaled_attr and getattr(self, scaled_attr) is None and isinstance(num, FloatType):
                    setattr(self, scaled_attr, num)
                return make_quant_function(num, rnd, self.rbits_add)
            return spec

        self.weight_quant = resolve(weight_quant, "weight_scaled_format")
        self.bias_quant = resolve(bias_quant)
        self.input_quant = resolve(input_quant, "input_scaled_format")
        self.output_quant = resolve(output_quant)
        self.grad_quant = resolve(grad_quant, "grad_scaled_format")
        self.use_scaling = use_scaling
        self.scale_margin = scale_margin

    def __repr__(self) -> str:
        out = []
        for tag, default in (("fwd", self.fwd_use_default_prec), ("bwd", self.bwd_use_default_prec)):
            if default:
                out.append("default_" + tag)
            elif getattr(self, tag + "_fma"):
                out += [f"{tag}_fma={getattr(self, tag + '_add')}", f"{tag}_rnd={getattr(self, tag + '_rnd')}"]
            else:
                out += [f"{tag}_mul={getattr(self, tag + '_mul')}", f"{tag}_add={getattr(self, tag + '_add')}",
                        f"{tag}_rnd={getattr(self, tag + '_rnd')}"]
        for name in ("weight_scaled_format", "input_scaled_format", "grad_scaled_format"):
            if getattr(self, name) is not None:
                out.append(f"{name}={getattr(self, name)}")
        if self.use_scaling:
            out.append(f"scale bias margin={self.scale_margin}")
        out += [f"rbits_add={self.rbits_add}", f"rbits_mul={self.rbits_mul}"]
        return "QAffineFormats ({})".format(", ".join(out))

    __str__ = __repr__


class QLayerNormFormats:
    """Formats for layer normalisation: accumulate / multiply / divide / square-root formats forward, accumulate /
    multiply / divide backward; the low-precision path is used only when every format of a direction is given."""

    def __init__(self, fwd_acc=None, fwd_mul=None, fwd_div=None, fwd_sqrt=None, bwd_acc=None, bwd_mul=None, bwd_div=None,
                 fwd_rnd: str | None = "nearest", bwd_rnd: str | None = "nearest", input_quant=id_quant,
                 output_quant=id_quant, grad_quant=id_quant, weight_quant=id_quant, bias_quant=id_quant) -> None:
        self.fwd_use_default_prec = None in (fwd_acc, fwd_mul, fwd_div, fwd_sqrt)
        if not self.fwd_use_default_prec:
            self.fwd_acc, self.fwd_mul, self.fwd_div, self.fwd_sqrt = fwd_acc, fwd_mul, fwd_div, fwd_sqrt
        self.bwd_use_default_prec = None in (bwd_acc, bwd_mul, bwd_div)
        if not self.bwd_use_default_prec:
            self.bwd_acc, self.bwd_mul, self.bwd_div = bwd_acc, bwd_mul, bwd_div
        self.fwd_rnd, self.bwd_rnd = fwd_rnd, bwd_rnd
        self.input_quant, self.output_quant, self.grad_quant = input_quant, output_quant, grad_quant
        self.weight_quant, self.bias_quant = weight_quant, bias_quant

    def __repr__(self) -> str:
        out = ["default_fwd"] if self.fwd_use_default_prec else [
            f"fwd_acc={self.fwd_acc}", f"fwd_mul={self.fwd_mul}", f"fwd_div={self.fwd_div}", f"fwd_sqrt={self.fwd_sqrt}",
            f"fwd_rnd={self.fwd_rnd}"]
        out += ["default_bwd"] if self.bwd_use_default_prec else [
            f"bwd_acc={self.bwd_acc}", f"bwd_mul={self.bwd_mul}", f"bwd_div={self.bwd_div}", f"bwd_rnd={self.bwd_rnd}"]
        return "QLayerNormFormats ({})".format(" , ".join(out))

    __str__ = __repr__


class QSoftmaxFormats:
    """Formats for softmax: ``fwd_off`` with ``fwd_exp`` + ``fwd_acc`` selects the division form, ``fwd_off`` with
    ``fwd_lse`` the log-sum-exp form; ``bwd_add`` + ``bwd_mul`` the low-precision backward."""

    def __init__(self, fwd_off=None, fwd_exp=None, fwd_acc=None, fwd_lse=None, bwd_add=None, bwd_mul=None,
                 fwd_rnd: str | None = "nearest", bwd_rnd: str | None = "nearest", input_quant=id_quant,
                 output_quant=id_quant, grad_quant=id_quant) -> None:
        self.fwd_use_default_prec = fwd_off is None
        if fwd_off is not None:
            self.fwd_off = fwd_off
            if fwd_acc is not None and fwd_exp is not None:
                self.fwd_acc, self.fwd_exp, self.use_lse = fwd_acc, fwd_exp, False
            elif fwd_lse is not None:
                self.fwd_lse, self.use_lse = fwd_lse, True
            else:
                raise ValueError("Incomplete softmax format, missing fwd_acc/fwd_exp or fwd_lse.")
        self.bwd_use_default_prec = bwd_add is None or bwd_mul is None
        if not self.bwd_use_default_prec:
            self.bwd_add, self.bwd_mul = bwd_add, bwd_mul
        self.fwd_rnd, self.bwd_rnd = fwd_rnd, bwd_rnd
        self.input_quant, self.output_quant, self.grad_quant = input_quant, output_quant, grad_quant

    def __repr__(self) -> str:
        if self.fwd_use_default_prec:
            out = ["default_fwd"]
        elif self.use_lse:
            out = [f"fwd_off={self.fwd_off}", f"fwd_lse={self.fwd_lse}", f"fwd_rnd={self.fwd_rnd}"]
        else:
            out = [f"fwd_off={self.fwd_off}", f"fwd_exp={self.fwd_exp}", f"fwd_acc={self.fwd_acc}", f"fwd_rnd={self.fwd_rnd}"]
        out += ["default_bwd"] if self.bwd_use_default_prec else [
            f"bwd_add={self.bwd_add}", f"bwd_mul={self.bwd_mul}", f"bwd_rnd={self.bwd_rnd}"]
        return "QSoftmaxFormats ({})".format(", ".join(out))

    __str__ = __repr__


class QGELUFormats:
    """Signal quantizers of the GELU activation (kept for API compatibility)."""

    def __init__(self, input_quant=id_quant, inter_quant=id_quant, output_quant=id_quant, grad_quant=id_quant):
        self.input_quant, self.inter_quant = input_quant, inter_quant
        self.output_quant, self.grad_quant = output_quant, grad_quant
