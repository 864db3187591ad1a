"""Host-side API checks that need no GPU: format descriptors, format/config classes, argument validation, and the
refusal to compute on CPU tensors (there is no CPU fallback)."""
import pytest
import torch

import mptorch_b200 as mp
import mptorch_b200.quant as q
from mptorch_b200 import backend


def test_number_formats_match_reference_definitions():
    """Values from the reference's number.py formulas (:139-158, :313-374)."""
    f = mp.FloatingPoint(5, 2, subnormals=True, saturate=False)
    assert (f.normal_max, f.normal_min, f.subnormal_min) == (57344.0, 2.0 ** -14, 2.0 ** -16)
    assert mp.FloatingPoint(4, 3).normal_max == 240.0 and mp.FloatingPoint(4, 3).subnormal_min is None
    assert mp.FloatingPoint(8, 23).is_fp32 and mp.FloatingPoint(5, 10).is_fp16 and mp.FloatingPoint(8, 7).is_bfloat16
    b = mp.Binary8(3, signed=True, subnormals=True, overflow_policy="saturate_maxfloat")
    assert (b.man, b.exp, b.normal_max) == (2, 5, 49152.0)
    assert mp.Binary8(3, overflow_policy="saturate_maxfloat2").normal_max == 57344.0
    assert mp.Binary8(4, signed=False).exp == 5
    s = mp.SuperNormalFloat(4, 3, (2, 1))
    assert s.binades == (2, 1)
    with pytest.raises(AssertionError):
        mp.FloatingPoint(9, 2)
    with pytest.raises(AssertionError):
        mp.Binary8(8)


def test_affine_formats_semantics():
    fp = mp.FloatingPoint
    add, mul = fp(5, 10, True, False), fp(4, 3, True, False)
    f = q.QAffineFormats(fwd_mac=(add, mul), bwd_mac=mul, weight_quant=(fp(4, 3, True, True), "nearest"), rbits=(3, 4))
    assert f.fwd_add is add and f.fwd_mul is mul and not f.fwd_fma            # tuple order is (add, mul)
    assert f.bwd_add is mul and f.bwd_fma                                     # a single format means FMA
    assert f.fwd_rnd == "nearest" and f.bwd_rnd == "nearest"
    assert f.weight_scaled_format.man == 3 and (f.rbits_add, f.rbits_mul) == (3, 4)
    d = q.QAffineFormats()
    assert d.fwd_use_default_prec and d.bwd_use_default_prec and d.rbits_add == 0
    assert "fwd_mul=FloatingPoint (exponent=4, mantissa=3)" in repr(f)


def test_softmax_and_layernorm_formats():
    fp = mp.FloatingPoint(5, 10, True, False)
    s = q.QSoftmaxFormats(fwd_off=fp, fwd_exp=fp, fwd_acc=fp)
    assert not s.use_lse and not s.fwd_use_default_prec and s.bwd_use_default_prec
    assert q.QSoftmaxFormats(fwd_off=fp, fwd_lse=fp).use_lse
    with pytest.raises(ValueError):
        q.QSoftmaxFormats(fwd_off=fp)
    ln = q.QLayerNormFormats(fwd_acc=fp, fwd_mul=fp, fwd_div=fp)      # sqrt missing -> default precision
    assert ln.fwd_use_default_prec
    assert not q.QLayerNormFormats(fwd_acc=fp, fwd_mul=fp, fwd_div=fp, fwd_sqrt=fp).fwd_use_default_prec


def test_public_names_of_the_reference_are_importable():
    for name in ["float_quantize", "binary8_quantize", "superfp_quantize", "block_quantize", "fixed_point_quantize",
                 "quantizer", "mp_mm", "mp_bmm", "float_mm", "float_bmm", "fxp_mm", "fxp_bmm", "superfp_mm", "superfp_bmm",
                 "mp_softmax_forward", "mp_softmax_backward", "float_softmax_forward", "float_softmax_lse_forward",
                 "float_softmax_backward", "mp_layernorm_forward", "mp_layernorm_backward", "float_layernorm_forward",
                 "float_layernorm_backward", "cublas_mm", "cublas_bmm", "cublas_acceleration", "QAffineFormats",
                 "QSoftmaxFormats", "QLayerNormFormats", "QGELUFormats", "QLinear", "QLazyLinear", "QConv2d", "QSoftmax",
                 "QLayerNorm", "Quantizer", "mx_quantize", "nvfp4_quantize"]:
        assert hasattr(q, name), name
    with pytest.raises(NotImplementedError):
        q.fxp_mm(None, None)
    with pytest.raises(NotImplementedError):
        q.block_quantize(torch.zeros(2), 8)


def test_no_cpu_fallback():
    x = torch.randn(4, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        q.float_quantize(x, 5, 2, "nearest")
    with pytest.raises(RuntimeError, match="CUDA"):
        q.float_mm(x, x, 2, 5, 2, 5)
    with pytest.raises(RuntimeError, match="CUDA"):
        backend.float_quantize_nearest(x, 2, 5, True, True)
    with pytest.raises(AssertionError):
        q.float_quantize(x, 5, 2, "up")
    with pytest.raises(AssertionError):
        q.binary8_quantize(x, 3, "nearest", prng_bits=40)


def test_partition_tensor_matches_reference_rule():
    """quant_cuda/quant.cu:678-726: (outer, channel, inner) for a softmax dim and for trailing layernorm dims."""
    assert backend.partition_tensor((4, 37, 5), 1) == (4, 37, 5)
    assert backend.partition_tensor((4, 37, 5), -1) == (148, 5, 1)
    assert backend.partition_tensor((4, 37, 5), 0) == (1, 4, 185)
    assert backend.partition_tensor((6, 5, 48), [-1]) == (30, 48, 1)
    assert backend.partition_tensor((4, 6, 8), [-1, -2]) == (4, 48, 1)
    with pytest.raises(ValueError):          # first-to-last order makes the reference overrun the tensor: refused here
        backend.partition_tensor((4, 6, 8), [-2, -1])


def test_order_knobs():
    assert backend.get_accum_order() == "cuda" and backend.get_reduce_order() == "cuda"
    with q.orders(accum="seq", reduce="seq"):
        assert backend.get_accum_order() == "seq" and backend.get_reduce_order() == "seq"
    assert backend.get_accum_order() == "cuda"
    with pytest.raises(ValueError):
        backend.set_accum_order("random")


def test_default_precision_layers_run_anywhere():
    """With no MAC formats the layers are plain torch ops plus straight-through quantizers (identity here)."""
    lin = q.QLinear(8, 4, q.QAffineFormats())
    x = torch.randn(3, 8, requires_grad=True)
    lin(x).sum().backward()
    assert x.grad.shape == (3, 8)
    assert q.QSoftmax(-1, q.QSoftmaxFormats())(torch.randn(2, 5)).sum().item() == pytest.approx(2.0, abs=1e-5)
    assert q.QLayerNorm(8, q.QLayerNormFormats())(torch.randn(2, 8)).shape == (2, 8)
    assert q.QConv2d(3, 4, 3, q.QAffineFormats(), padding=1)(torch.randn(1, 3, 8, 8)).shape == (1, 4, 8, 8)


def test_optimizer_wrapper_recognises_fusable_quantizers():
    """QOptim fuses only quantizers whose format and rounding it can read; everything else is called per tensor."""
    import mptorch_b200.quant as q
    from mptorch_b200 import Binary8, FloatingPoint
    from mptorch_b200.optim import _fusable

    near = q.quantizer(forward_number=FloatingPoint(5, 10, True, True), forward_rounding="nearest")
    sr = q.quantizer(forward_number=FloatingPoint(5, 10, True, True), forward_rounding="stochastic")
    b8 = q.quantizer(forward_number=Binary8(3), forward_rounding="nearest")
    assert _fusable(near, False)[1] == "nearest" and _fusable(near, False)[0].man == 10
    assert _fusable(sr, False) is None and _fusable(sr, True)[1] == "stochastic"
    assert _fusable(b8, False) is None
    assert _fusable(lambda t: t, True) is None


def test_streamed_gemm_and_multi_quantize_reject_cpu_execution():
    import mptorch_b200.quant as q

    a, b = torch.zeros(4, 4), torch.zeros(4, 4)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            q.float_mm_streamed(a, b)
    with pytest.raises(RuntimeError):
        q.float_quantize_multi([a], 4, 3, "nearest")
    with pytest.raises(RuntimeError):
        q.float_mm_streamed(a, b.t())            # non-contiguous operand


def test_implicit_conv_needs_cuda_and_plain_nearest_formats():
    import mptorch_b200.quant as q
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.quant.functional import implicit_conv_eligible

    f = q.QAffineFormats(fwd_mac=(FloatingPoint(5, 10, True, False), FloatingPoint(4, 3, True, False)), fwd_rnd="nearest")
    assert not implicit_conv_eligible(f, torch.zeros(1))          # CPU tensor


def test_k_panels_of_the_streamed_product():
    """Host logic of float_mm_streamed's K-panel pipeline: the panels tile [0, K) in order, every boundary but the end
    is a multiple of 8 (the group size of the CUDA accumulation order), the first panel is short, the last one is at
    least 512 steps, and short K disables the pipeline."""
    from mptorch_b200.quant.quant_function import _k_panels

    assert _k_panels(0) is None and _k_panels(1000) is None and _k_panels(1791) is None
    for K in (1792, 1800, 2048, 2053, 3000, 4096, 8191, 8192, 10000, 65536, 100003):
        panels = _k_panels(K)
        assert panels[0][0] == 0 and panels[-1][1] == K
        assert all(a[1] == b[0] for a, b in zip(panels, panels[1:]))
        assert all(k1 > k0 for k0, k1 in panels)
        assert all(k1 % 8 == 0 for _, k1 in panels[:-1])
        assert panels[0][1] == 256 and panels[-1][1] - panels[-1][0] >= 512
        assert max(k1 - k0 for k0, k1 in panels) <= 3072


def test_second_gradient_context_is_inert_on_cpu():
    """The two-stream backward helper does nothing for CPU tensors (and when switched off)."""
    import torch

    from mptorch_b200.quant import functional as F

    s = F._second_gradient(torch.zeros(3))
    with s:
        y = torch.ones(3) * 2
    s.join(y, None)
    assert s.side is None and float(y.sum()) == 6.0
