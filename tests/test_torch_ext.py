"""The quant_cuda-compatible PyTorch C++ extension (mptorch_b200/torch_ext/quant_b200.cpp) over the C ABI."""
import pytest
import torch

NAMES = ["float_quantize_nearest", "float_quantize_stochastic", "binary8_quantize_nearest", "binary8_quantize_stochastic",
         "binary8_quantize_truncate", "superfp_quantize_nearest", "float_quantize_nearest_mm", "float_quantize_nearest_bmm",
         "float_quantize_nearest_mm_fma", "float_quantize_nearest_bmm_fma", "float_quantize_stochastic_mm",
         "float_quantize_stochastic_bmm", "float_quantize_stochastic_mm_fma", "float_quantize_stochastic_bmm_fma",
         "float_quantize_nearest_softmax_forward", "float_quantize_nearest_softmax_lse_forward",
         "float_quantize_nearest_softmax_backward", "float_quantize_layernorm_forward", "float_quantize_layernorm_backward",
         "superfp_quantize_nearest_mm", "superfp_quantize_nearest_bmm", "superfp_quantize_nearest_mm_fma", "superfp_quantize_nearest_bmm_fma",
         "superfp_quantize_nearest_softmax_forward", "superfp_quantize_nearest_softmax_lse_forward", "superfp_quantize_nearest_softmax_backward",
         "binary8_quantize_nearest_softmax_forward", "binary8_quantize_nearest_softmax_lse_forward", "binary8_quantize_nearest_softmax_backward",
         "superfp_quantize_layernorm_forward", "superfp_quantize_layernorm_backward", "binary8_quantize_layernorm_forward",
         "binary8_quantize_layernorm_backward",
         # no quant_cuda counterpart
         "float_quantize_truncate", "qsum_rows", "float_conv2d_nearest", "mx_quantize", "nvfp4_quantize", "float_quantize_multi", "scale_quantize"]


@pytest.fixture(scope="module")
def ext():
    from mptorch_b200 import torch_ext

    return torch_ext.load()


def test_extension_exports_the_reference_module_interface(ext):
    """Every hot-path name the reference registers in quant_cuda (pybind_cuda.cpp:734-927) is present."""
    for n in NAMES:
        assert callable(getattr(ext, n)), n
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.float_quantize_nearest(torch.zeros(4), 2, 5, True, True)
    # the overflow policy is an enum of the module, as in the reference (pybind_cuda.cpp:784-787), used as
    # module.OverflowPolicy.SATURATE_INFTY by quant_function.py:372-374
    pol = ext.OverflowPolicy
    assert [int(pol.SATURATE_INFTY), int(pol.SATURATE_MAXFLOAT), int(pol.SATURATE_MAXFLOAT2)] == [0, 1, 2]
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.binary8_quantize_nearest(torch.zeros(4), 3, True, pol.SATURATE_MAXFLOAT, True)


@pytest.mark.gpu
def test_extension_matches_ctypes_backend(ext):
    from mptorch_b200 import backend as be

    x = torch.randn(1 << 16, device="cuda") * 4
    assert torch.equal(ext.float_quantize_nearest(x, 3, 4, True, True), be.float_quantize_nearest(x, 3, 4, True, True))
    torch.manual_seed(3)
    a = ext.float_quantize_stochastic(x, 3, 4, 20, True, True)
    torch.manual_seed(3)
    assert torch.equal(a, be.float_quantize_stochastic(x, 3, 4, 20, True, True))
    assert torch.equal(ext.binary8_quantize_nearest(x, 3, True, 1, True), be.binary8_quantize_nearest(x, 3, True, 1, True))
    a, b = torch.randn(3, 70, 40, device="cuda"), torch.randn(3, 40, 52, device="cuda")
    c1, c2 = torch.empty(3, 70, 52, device="cuda"), torch.empty(3, 70, 52, device="cuda")
    ext.float_quantize_nearest_bmm(a, b, c1, 70, 52, 40, 10, 5, 3, 4, True, False, False)
    be.float_quantize_nearest_bmm(a, b, c2, 70, 52, 40, 10, 5, 3, 4, True, False, False)
    assert torch.equal(c1, c2)
    ext.float_quantize_nearest_mm_fma(a[0].contiguous(), b[0].contiguous(), c1[0], 70, 52, 40, 2, 5, True, False, False)
    be.float_quantize_nearest_mm_fma(a[0].contiguous(), b[0].contiguous(), c2[0], 70, 52, 40, 2, 5, True, False, False)
    assert torch.equal(c1[0], c2[0])
    s = torch.randn(4, 9, 200, device="cuda")
    o1, o2 = torch.empty_like(s), torch.empty_like(s)
    ext.float_quantize_nearest_softmax_forward(s, o1, -1, 10, 5, 10, 5, 10, 5, True, False)
    be.float_quantize_nearest_softmax_forward(s, o2, -1, 10, 5, 10, 5, 10, 5, True, False)
    assert torch.equal(o1, o2)
    w, bias = torch.randn(200, device="cuda"), torch.randn(200, device="cuda")
    y1, m1, r1 = torch.empty_like(s), torch.empty(4, 9, device="cuda"), torch.empty(4, 9, device="cuda")
    y2, m2, r2 = torch.empty_like(s), torch.empty(4, 9, device="cuda"), torch.empty(4, 9, device="cuda")
    ext.float_quantize_layernorm_forward(s, w, bias, y1, m1, r1, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, True, False)
    be.float_quantize_layernorm_forward(s, w, bias, y2, m2, r2, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, True, False)
    assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(r1, r2)


@pytest.mark.gpu
def test_extension_as_the_quant_cuda_module(ext):
    """The swap a maintainer of the reference would make: the reference's call sites use the module object (binary8 with
    the module's own OverflowPolicy enum, superfp and binary8 reductions, the GEMM families), here with the extension
    object in place of quant_cuda and the ctypes route as the comparison."""
    from mptorch_b200 import backend as be

    x = torch.randn(1 << 14, device="cuda") * 30
    for name, po in (("SATURATE_INFTY", 0), ("SATURATE_MAXFLOAT", 1), ("SATURATE_MAXFLOAT2", 2)):
        pol = getattr(ext.OverflowPolicy, name)
        want = be._binary8(x, 3, True, po, True, 0)
        assert torch.equal(ext.binary8_quantize_nearest(x, 3, True, pol, True).view(torch.int32), want.view(torch.int32))
        got, ref = ext.binary8_quantize_truncate(x, 4, False, pol, True), be._binary8(x, 4, False, po, True, 2)    # unsigned: negatives are NaN
        assert bool(((got == ref) | (got.isnan() & ref.isnan())).all())
    a, b = torch.randn(2, 50, 40, device="cuda"), torch.randn(2, 40, 36, device="cuda")
    c1, c2 = torch.empty(2, 50, 36, device="cuda"), torch.empty(2, 50, 36, device="cuda")
    ext.superfp_quantize_nearest_bmm(a, b, c1, 50, 36, 40, 3, 4, 2, 4, 1, 1, 2, 2, False)
    be.mm_fmt(a, b, c2, 2, 50, 36, 40, be.Format.superfp(3, 4, 1, 1, False), be.Format.superfp(2, 4, 2, 2, False), False)
    assert torch.equal(c1.view(torch.int32), c2.view(torch.int32))
    s = torch.randn(3, 7, 96, device="cuda")
    o1, o2 = torch.empty_like(s), torch.empty_like(s)
    ext.binary8_quantize_nearest_softmax_forward(s, o1, -1, 4, ext.OverflowPolicy.SATURATE_MAXFLOAT, True, 4, 1, True, 5, 1, True, True)
    be.softmax_forward_fmt(s, o2, -1, be.Format.binary8(4, True, 1, True), be.Format.binary8(4, True, 1, True), be.Format.binary8(5, True, 1, True))
    assert torch.equal(o1.view(torch.int32), o2.view(torch.int32))
    w, bias = torch.randn(96, device="cuda"), torch.randn(96, device="cuda")
    y1, m1, r1 = torch.empty_like(s), torch.empty(3, 7, device="cuda"), torch.empty(3, 7, device="cuda")
    y2, m2, r2 = torch.empty_like(s), torch.empty(3, 7, device="cuda"), torch.empty(3, 7, device="cuda")
    ext.superfp_quantize_layernorm_forward(s, w, bias, y1, m1, r1, 1e-5, [-1], 10, 5, 1, 1, 10, 5, 1, 1, 10, 5, 1, 1, 10, 5, 1, 1, False)
    f = be.Format.superfp(10, 5, 1, 1, False)
    be.layernorm_forward_fmt(s, w, bias, y2, m2, r2, 1e-5, [-1], f, f, f, f)
    assert torch.equal(y1.view(torch.int32), y2.view(torch.int32)) and torch.equal(r1, r2)
    # new entry points
    q1 = ext.mx_quantize(s, "e2m1", 32, True, True)
    saved, be._ext = be._ext, None
    try:
        q2 = be.mx_quantize(s, "e2m1", 32, True, True)
        assert all(torch.equal(u, v) for u, v in zip(q1, q2))
        assert torch.equal(ext.qsum_rows(s[0], 10, 5, True, False), be.qsum_rows(s[0], 10, 5, True, False))
    finally:
        be._ext = saved


@pytest.mark.gpu
def test_backend_routes_agree(ext):
    """The hot entry points give the same bits through the C++ extension and through ctypes."""
    from mptorch_b200 import backend as be

    a, b = torch.randn(3, 70, 40, device="cuda"), torch.randn(3, 40, 52, device="cuda")
    s = torch.randn(4, 9, 200, device="cuda")
    w, bias = torch.randn(200, device="cuda"), torch.randn(200, device="cuda")

    def run():
        c = torch.empty(3, 70, 52, device="cuda")
        be.float_quantize_nearest_bmm(a, b, c, 70, 52, 40, 10, 5, 3, 4, True, False, False)
        o = torch.empty_like(s)
        be.float_quantize_nearest_softmax_forward(s, o, -1, 10, 5, 10, 5, 10, 5, True, False)
        y, m, r = torch.empty_like(s), torch.empty(4, 9, device="cuda"), torch.empty(4, 9, device="cuda")
        be.float_quantize_layernorm_forward(s, w, bias, y, m, r, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, True, False)
        gi, gg, gb = torch.empty_like(s), torch.empty(200, device="cuda"), torch.empty(200, device="cuda")
        be.float_quantize_layernorm_backward(s, o, w, bias, m, r, gi, gg, gb, [-1], 10, 5, 10, 5, 10, 5, True, False)
        return [c, o, y, m, r, gi, gg, gb, be.float_quantize_nearest(s, 3, 4, True, True)]

    saved = be._ext
    try:
        be._ext = ext
        via_ext = run()
        be._ext = None
        via_ctypes = run()
    finally:
        be._ext = saved
    for u, v in zip(via_ext, via_ctypes):
        assert torch.equal(u.view(torch.int32), v.view(torch.int32))
