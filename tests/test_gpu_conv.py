"""QConv2d through the implicit GEMM (`mpt_float_conv2d_nearest`) against the unfold + GEMM composition it replaces.

Both paths form the same products in the same order (K = channel, kernel row, kernel column) and accumulate them in
the same association, so outputs and all three gradients must agree bit for bit; the composition itself is pinned to
the oracle in test_gpu_layers.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    import mptorch_b200.quant as quant

    return quant


def fp(e, m, sub=True, sat=False):
    from mptorch_b200 import FloatingPoint

    return FloatingPoint(e, m, sub, sat)


def bits_equal(a, b):
    a, b = a.contiguous(), b.contiguous()
    same = a.view(torch.int32) == b.view(torch.int32)
    return bool((same | (a.isnan() & b.isnan())).all())


def run(q, conv, x, g, implicit, monkeypatch):
    import mptorch_b200.quant.modules as modules

    if not implicit:
        monkeypatch.setattr(modules, "implicit_conv_eligible", lambda f, t: False)
    calls = []
    if implicit:
        real = modules.qconv2d
        monkeypatch.setattr(modules, "qconv2d", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    for p in conv.parameters():
        p.grad = None
    xi = x.clone().requires_grad_()
    y = conv(xi)
    y.backward(g)
    monkeypatch.undo()
    if implicit:
        assert calls, "the implicit path was not taken"
    return y.detach(), xi.grad, conv.weight.grad.clone(), None if conv.bias is None else conv.bias.grad.clone()


CASES = [
    # n, c, h, w, cout, kernel, stride, padding, dilation, groups, bias, padding_mode
    (2, 3, 9, 11, 5, 3, 1, 1, 1, 1, True, "zeros"),
    (3, 4, 12, 10, 6, 3, 2, 1, 1, 2, True, "zeros"),
    (2, 4, 13, 13, 8, (3, 2), (1, 2), (2, 0), (2, 1), 1, False, "zeros"),
    (2, 8, 8, 8, 8, 1, 1, 0, 1, 4, True, "zeros"),
    (1, 2, 6, 7, 3, 5, 1, 2, 1, 1, True, "reflect"),
    (4, 16, 32, 32, 64, 3, 1, 1, 1, 1, True, "zeros"),
    (2, 6, 10, 10, 130, 3, 1, 0, 1, 1, False, "zeros"),
    (1, 1, 5, 5, 1, 7, 1, 3, 1, 1, True, "zeros"),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("order", ["cuda", "seq"])
@pytest.mark.parametrize("fma", [False, True])
@pytest.mark.parametrize("sub", [True, False])
def test_implicit_conv_equals_unfold_composition(q, monkeypatch, case, order, fma, sub):
    """`sub` False: MAC formats without subnormals (the settling rounding of the implicit kernels against that of the
    plain GEMM, which is pinned against the reference's CUDA kernel)."""
    n, c, h, w, cout, k, s, p, d, groups, bias, mode = case
    add, mul = fp(5, 10, sub), fp(4, 3, sub)
    mac = (add,) if fma else (add, mul)
    wq = q.quantizer(forward_number=fp(5, 2, True, True), forward_rounding="nearest")
    fmt = q.QAffineFormats(fwd_mac=mac, bwd_mac=mac, fwd_rnd="nearest", bwd_rnd="nearest", weight_quant=wq, input_quant=wq,
                           grad_quant=q.quantizer(forward_number=fp(5, 10, True, True), forward_rounding="nearest"))
    torch.manual_seed(hash(case) % 1000)
    conv = q.QConv2d(c, cout, k, fmt, stride=s, padding=p, dilation=d, groups=groups, bias=bias, padding_mode=mode).cuda()
    x = torch.randn(n, c, h, w, device="cuda")
    with q.orders(accum=order):
        y0 = conv(x)
        g = torch.randn_like(y0)
        a = run(q, conv, x, g, True, monkeypatch)
        b = run(q, conv, x, g, False, monkeypatch)
    names = ["output", "grad_input", "grad_weight", "grad_bias"]
    for nm, u, v in zip(names, a, b):
        if u is None:
            assert v is None
            continue
        assert u.shape == v.shape, nm
        assert bits_equal(u, v), (nm, case, order, fma, (u != v).sum().item())


def test_implicit_conv_other_formats_and_special_values(q, monkeypatch):
    """e5m2 MACs (overflowing sums), an input with inf / NaN / huge values: the exact path inside the kernel."""
    fmt = q.QAffineFormats(fwd_mac=(fp(5, 2), fp(5, 2)), bwd_mac=(fp(5, 2), fp(5, 2)), fwd_rnd="nearest", bwd_rnd="nearest")
    torch.manual_seed(1)
    conv = q.QConv2d(3, 4, 3, fmt, padding=1).cuda()
    x = torch.randn(2, 3, 8, 8, device="cuda") * 50
    x[0, 1, 2, 3] = float("inf")
    x[1, 0, 5, 5] = float("nan")
    x[1, 2, 0, 0] = 1e30
    g = torch.randn(2, 4, 8, 8, device="cuda")
    a = run(q, conv, x, g, True, monkeypatch)
    b = run(q, conv, x, g, False, monkeypatch)
    assert bits_equal(a[0], b[0])
    assert bits_equal(a[2], b[2]), "weight gradient through the implicit GEMM"


def test_implicit_weight_gradient_entry_point(q):
    """mpt_float_conv2d_wgrad_nearest against the unfold + float_mm composition it replaces, directly: groups, strides,
    dilation, padding, a K (images x positions) that is not a multiple of the 8-wide tile, and gradients that overflow."""
    from mptorch_b200 import backend as be

    torch.manual_seed(7)
    for (n, c, h, w, cout, k, s, p, d, groups) in [(3, 4, 9, 7, 6, (3, 2), (2, 1), (1, 0), (1, 2), 2), (2, 3, 11, 11, 70, (3, 3), (1, 1), (1, 1), (1, 1), 1),
                                                    (1, 2, 5, 5, 2, (5, 5), (1, 1), (2, 2), (1, 1), 1),
                                                    # 10 x 18 tiles of 128 x 64: more than the SM count, the 128-row instantiation
                                                    # (the cases above have few tiles and take the 16-row one)
                                                    (1, 128, 4, 4, 1280, (3, 3), (1, 1), (1, 1), (1, 1), 1)]:
        x = torch.randn(n, c, h, w, device="cuda")
        oh = (h + 2 * p[0] - d[0] * (k[0] - 1) - 1) // s[0] + 1
        ow = (w + 2 * p[1] - d[1] * (k[1] - 1) - 1) // s[1] + 1
        go = torch.randn(n, cout, oh, ow, device="cuda") * 30
        cg, og = c // groups, cout // groups
        for order in ("cuda", "seq"):
            for (ma, ea, mm, em, fma) in [(10, 5, 3, 4, False), (2, 5, 2, 5, False), (7, 8, 7, 8, True)]:
                got = torch.full((cout, cg * k[0] * k[1]), float("nan"), device="cuda")
                be.float_conv2d_wgrad_nearest(go, x, got, groups, k, s, p, d, ma, ea, mm, em, True, False, fma=fma, order=order)
                for g in range(groups):
                    cols = torch.nn.functional.unfold(x[:, g * cg:(g + 1) * cg], k, dilation=d, padding=p, stride=s).transpose(1, 2).reshape(-1, cg * k[0] * k[1]).contiguous()
                    a = go[:, g * og:(g + 1) * og].reshape(n, og, -1).transpose(1, 2).reshape(-1, og).t().contiguous()
                    want = torch.empty(og, cols.shape[1], device="cuda")
                    if fma:
                        be.float_quantize_nearest_mm_fma(a, cols, want, og, cols.shape[1], a.shape[1], ma, ea, True, False, False, order=order)
                    else:
                        be.float_quantize_nearest_mm(a, cols, want, og, cols.shape[1], a.shape[1], ma, ea, mm, em, True, False, False, order=order)
                    assert bits_equal(got[g * og:(g + 1) * og], want), ((n, c, h, w, cout, k, s, p, d, groups), order, ma, ea, fma, g)


def test_ineligible_configurations_take_the_unfold_path(q):
    from mptorch_b200.quant.functional import implicit_conv_eligible

    x = torch.zeros(1, device="cuda")
    sr = q.quantizer(forward_number=fp(4, 3, True, True), forward_rounding="stochastic")
    base = dict(fwd_mac=(fp(5, 10), fp(4, 3)), bwd_mac=(fp(5, 10), fp(4, 3)))
    assert implicit_conv_eligible(q.QAffineFormats(**base, fwd_rnd="nearest", bwd_rnd="nearest"), x)
    assert not implicit_conv_eligible(q.QAffineFormats(**base, fwd_rnd="stochastic", bwd_rnd="nearest"), x)
    assert not implicit_conv_eligible(q.QAffineFormats(**base, fwd_rnd="nearest", bwd_rnd="nearest", input_quant=sr), x)
    assert not implicit_conv_eligible(q.QAffineFormats(**base, fwd_rnd="nearest", bwd_rnd="nearest", compensated=True), x)
    assert not implicit_conv_eligible(q.QAffineFormats(), x)
