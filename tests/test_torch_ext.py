"""The quant_cuda-compatible PyTorch C++ extension (mptorch_b200/torch_ext/quant_b200.cpp) over the C ABI."""
import pytest
import torch

NAMES = ["float_quantize_nearest", "float_quantize_stochastic", "binary8_quantize_nearest", "binary8_quantize_stochastic",
         "binary8_quantize_truncate", "superfp_quantize_nearest", "float_quantize_nearest_mm", "float_quantize_nearest_bmm",
         "float_quantize_nearest_mm_fma", "float_quantize_nearest_bmm_fma", "float_quantize_stochastic_mm",
         "float_quantize_stochastic_bmm", "float_quantize_stochastic_mm_fma", "float_quantize_stochastic_bmm_fma",
         "float_quantize_nearest_softmax_forward", "float_quantize_nearest_softmax_lse_forward",
         "float_quantize_nearest_softmax_backward", "float_quantize_layernorm_forward", "float_quantize_layernorm_backward"]


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
