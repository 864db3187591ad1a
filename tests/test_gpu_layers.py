"""The autograd layers on the GPU: forward and backward results rebuilt from oracle calls (bit for bit), and the
reference's own tolerance tests (tests/test_qlinear.py, test_qsoftmax.py, test_qlayernorm.py, test_mm.py, test_scaling.py
of the reference) re-expressed against this package."""
import numpy as np
import pytest
import torch

import mptorch_b200 as mp
import mptorch_b200.quant as q
from conftest import mismatch_report, same_bits
from mptorch_b200.quant import functional as Fq

pytestmark = pytest.mark.gpu

fp = mp.FloatingPoint


def npy(t):
    return t.detach().cpu().numpy()


def test_qlinear_forward_backward_rebuilt_from_oracle(oracle):
    """QLinear on a 3-D input with (add e5m10, mul e4m3) MACs and e4m3 signal quantizers: every tensor the layer
    produces is recomputed with oracle calls in the order the reference's qlinear_kernel prescribes."""
    add, mul = fp(5, 10, True, False), fp(4, 3, True, False)
    sig = fp(4, 3, True, True)
    fmt = q.QAffineFormats(fwd_mac=(add, mul), bwd_mac=(add, mul), fwd_rnd="nearest", bwd_rnd="nearest",
                           weight_quant=(sig, "nearest"), input_quant=(sig, "nearest"), grad_quant=(fp(5, 2, True, True), "nearest"))
    torch.manual_seed(3)
    lin = q.QLinear(40, 24, fmt, bias=True).cuda()
    x = torch.randn(3, 10, 40, device="cuda", requires_grad=True)
    y = lin(x)
    g = torch.randn_like(y)
    y.backward(g)

    Q = lambda v, f: oracle.float_quantize(v, f.man, f.exp, "nearest", f.subnormals, f.saturate)
    gq = fp(5, 2, True, True)
    qx, qw = Q(npy(x), sig), Q(npy(lin.weight), sig)
    want_y = oracle.mm(qx.reshape(30, 40), qw.T.copy(), add.man, add.exp, mul.man, mul.exp, True, False, False, "tile8").reshape(3, 10, 24)
    want_y = want_y + npy(lin.bias).reshape(1, 24)
    assert same_bits(npy(y), want_y), mismatch_report(npy(y), want_y)
    qg = Q(npy(g), gq)
    want_dx = Q(oracle.mm(qg.reshape(30, 24), qw, add.man, add.exp, mul.man, mul.exp, True, False, False, "tile8").reshape(3, 10, 40), gq)
    assert same_bits(npy(x.grad), want_dx), mismatch_report(npy(x.grad), want_dx)
    # dW: batched [3, 24, 10] x [3, 10, 40], grad_quant per batch entry, then autograd's fp32 sum over the batch
    dw_b = oracle.mm(np.ascontiguousarray(qg.transpose(0, 2, 1)), qx, add.man, add.exp, mul.man, mul.exp, True, False, False, "tile8")
    want_dw = Q(dw_b, gq).sum(0, dtype=np.float32)
    np.testing.assert_allclose(npy(lin.weight.grad), want_dw, rtol=0, atol=0)
    # bias gradient: rounded sequential sums over dim 0 then dim 1 in the add format, then grad_quant
    s0 = np.stack([oracle.qsum_rows(qg[:, t, :], add.man, add.exp, True, False) for t in range(10)])
    want_db = Q(oracle.qsum_rows(s0, add.man, add.exp, True, False), gq)
    assert same_bits(npy(lin.bias.grad), want_db), mismatch_report(npy(lin.bias.grad), want_db)


def test_fast_bias_gradient_equals_reference_loop():
    """The one-launch column sum gives the same bits as the reference's per-slice quantize loop (qsum)."""
    g = torch.randn(5, 17, 24, device="cuda")
    add = fp(5, 10, True, False)
    fast = Fq._qsum_dims_fast(g, (0, 1), add).reshape(24)
    loop = Fq.qsum(g, dim=(0, 1), quant=lambda v: q.float_quantize(v, 5, 10, "nearest", True, False))
    assert torch.equal(fast.view(torch.int32), loop.reshape(24).view(torch.int32))


def test_qlinear_tolerance_like_reference_test():
    """reference tests/test_qlinear.py:24-90: e8m12 MACs, 11x1034 -> 542, fwd atol 1e-2, grads 1e-3."""
    f12 = fp(8, 12, True, False)
    for fmt in (q.QAffineFormats(fwd_mac=(f12, f12), bwd_mac=(f12, f12)), q.QAffineFormats(fwd_mac=f12, bwd_mac=f12)):
        torch.manual_seed(0)
        ref = torch.nn.Linear(1034, 542).cuda()
        lin = q.QLinear(1034, 542, fmt).cuda()
        lin.load_state_dict(ref.state_dict())
        x = torch.randn(11, 1034, device="cuda")
        xr, xq = x.clone().requires_grad_(), x.clone().requires_grad_()
        yr, yq = ref(xr), lin(xq)
        assert torch.allclose(yr, yq, atol=1e-2)
        yr.sum().backward(); yq.sum().backward()
        assert torch.allclose(xr.grad, xq.grad, atol=1e-3)
        assert torch.allclose(ref.weight.grad, lin.weight.grad, atol=1e-2)
        assert torch.allclose(ref.bias.grad, lin.bias.grad, atol=1e-3)


def test_float_mm_tolerance_like_reference_test():
    """reference tests/test_mm.py:24-131: e8m22 formats vs torch.mm, atol 1e-4, shapes 78x101x145 and batched."""
    a, b = torch.randn(78, 101, device="cuda"), torch.randn(101, 145, device="cuda")
    for fma in (False, True):
        for comp in (False, True):
            c = q.float_mm(a, b, 22, 8, 22, 8, "nearest", fma, True, False, comp)
            assert torch.allclose(c, a @ b, atol=1e-4)
        c = q.float_mm(a, b, 22, 8, 22, 8, "stochastic", fma, True, False)
        assert torch.allclose(c, a @ b, atol=1e-3)
    a3, b3 = torch.randn(40, 78, 101, device="cuda"), torch.randn(40, 101, 50, device="cuda")
    assert torch.allclose(q.float_bmm(a3, b3, 22, 8, 22, 8, "nearest", False, True, False), torch.bmm(a3, b3), atol=1e-4)
    assert torch.allclose(q.float_bmm(a3, b, 22, 8, 22, 8, "nearest", False, True, False), a3 @ b, atol=1e-4)
    a4, b4 = torch.randn(2, 3, 20, 30, device="cuda"), torch.randn(2, 3, 30, 10, device="cuda")
    assert torch.allclose(q.float_bmm(a4, b4, 22, 8, 22, 8, "nearest", True, True, False), a4 @ b4, atol=1e-4)
    with pytest.raises(Exception):
        q.float_bmm(a4, b3[:, :30, :10].contiguous(), 22, 8, 22, 8)


def test_qmatmul_and_qmm_gradients(oracle):
    add, mul = fp(5, 10, True, False), fp(4, 3, True, False)
    fmt = q.QAffineFormats(fwd_mac=(add, mul), bwd_mac=(add, mul))
    a = torch.randn(2, 3, 16, 8, device="cuda", requires_grad=True)
    b = torch.randn(2, 3, 8, 12, device="cuda", requires_grad=True)
    y = Fq.qmatmul(a, b, fmt)
    g = torch.randn_like(y)
    y.backward(g)
    want = oracle.mm(npy(a).reshape(6, 16, 8), npy(b).reshape(6, 8, 12), 10, 5, 3, 4, True, False, False, "tile8").reshape(2, 3, 16, 12)
    assert same_bits(npy(y), want)
    want_da = oracle.mm(npy(g).reshape(6, 16, 12), np.ascontiguousarray(npy(b).reshape(6, 8, 12).transpose(0, 2, 1)), 10, 5, 3, 4, True, False, False, "tile8")
    assert same_bits(npy(a.grad).reshape(6, 16, 8), want_da)
    want_db = oracle.mm(np.ascontiguousarray(npy(a).reshape(6, 16, 8).transpose(0, 2, 1)), npy(g).reshape(6, 16, 12), 10, 5, 3, 4, True, False, False, "tile8")
    assert same_bits(npy(b.grad).reshape(6, 8, 12), want_db)
    m1 = torch.randn(9, 7, device="cuda", requires_grad=True)
    m2 = torch.randn(7, 5, device="cuda", requires_grad=True)
    Fq.qmm(m1, m2, fmt).sum().backward()
    assert m1.grad.shape == (9, 7) and m2.grad.shape == (7, 5)


def test_qsoftmax_like_reference_test():
    """reference tests/test_qsoftmax.py:68-111: e5m10, shape (20,30,40), every dim, division and LSE forms, atol 1e-3."""
    h = fp(5, 10, True, False)
    for fmt in (q.QSoftmaxFormats(fwd_off=h, fwd_exp=h, fwd_acc=h, bwd_add=h, bwd_mul=h),
                q.QSoftmaxFormats(fwd_off=h, fwd_lse=h, bwd_add=h, bwd_mul=h)):
        for dim in (0, 1, 2):
            x = torch.randn(20, 30, 40, device="cuda")
            xr, xq = x.clone().requires_grad_(), x.clone().requires_grad_()
            yr = torch.softmax(xr, dim)
            yq = q.QSoftmax(dim, fmt)(xq)
            assert torch.allclose(yr, yq, atol=1e-3 if not fmt.use_lse else 1e-2)
            g = torch.randn_like(yr)
            yr.backward(g); yq.backward(g)
            assert torch.allclose(xr.grad, xq.grad, atol=1e-2)


def test_qlayernorm_like_reference_test():
    """reference tests/test_qlayernorm.py:45-91: e8m23 formats agree with torch to 1e-5."""
    f32 = fp(8, 23, True, False)
    fmt = q.QLayerNormFormats(fwd_acc=f32, fwd_mul=f32, fwd_div=f32, fwd_sqrt=f32, bwd_acc=f32, bwd_mul=f32, bwd_div=f32)
    for shape, nshape in (((10, 20, 30), [30]), ((4, 6, 8), [6, 8])):
        ref = torch.nn.LayerNorm(nshape).cuda()
        with torch.no_grad():
            ref.weight.normal_(); ref.bias.normal_()
        ln = q.QLayerNorm(nshape, fmt).cuda()
        ln.load_state_dict(ref.state_dict())
        x = torch.randn(*shape, device="cuda")
        xr, xq = x.clone().requires_grad_(), x.clone().requires_grad_()
        yr, yq = ref(xr), ln(xq)
        assert torch.allclose(yr, yq, atol=1e-5)
        g = torch.randn_like(yr)
        yr.backward(g); yq.backward(g)
        assert torch.allclose(xr.grad, xq.grad, atol=1e-4)
        assert torch.allclose(ref.weight.grad, ln.weight.grad, atol=1e-4)
        assert torch.allclose(ref.bias.grad, ln.bias.grad, atol=1e-4)


def test_scaled_qlinear_like_reference_test():
    """reference tests/test_scaling.py:97-127: e4m3/e5m2 signals with tensor scaling, atol 1e-1 against fp32."""
    e4, e5 = fp(4, 3, True, True), fp(5, 2, True, True)
    acc = fp(8, 23, True, False)
    fmt = q.QAffineFormats(fwd_mac=(acc, acc), bwd_mac=(acc, acc), weight_quant=(e4, "nearest"), input_quant=(e4, "nearest"),
                           grad_quant=(e5, "nearest"), use_scaling=True)
    torch.manual_seed(1)
    ref = torch.nn.Linear(64, 32).cuda()
    lin = q.QLinear(64, 32, fmt).cuda()
    lin.load_state_dict(ref.state_dict())
    x = torch.randn(16, 64, device="cuda") * 1e-3
    assert torch.allclose(ref(x), lin(x), atol=1e-1)
    assert not torch.allclose(lin(x), torch.zeros_like(lin(x)))


def test_qconv2d_matches_unfold_composition(oracle):
    add, mul = fp(5, 10, True, False), fp(4, 3, True, False)
    fmt = q.QAffineFormats(fwd_mac=(add, mul), bwd_mac=(add, mul))
    torch.manual_seed(2)
    conv = q.QConv2d(4, 6, 3, fmt, stride=1, padding=1, groups=2, bias=True).cuda()
    x = torch.randn(2, 4, 7, 7, device="cuda", requires_grad=True)
    y = conv(x)
    assert y.shape == (2, 6, 7, 7)
    y.sum().backward()
    assert x.grad.shape == x.shape and conv.weight.grad.shape == conv.weight.shape
    # group 0 forward rebuilt: unfold (channel-major K order) then the oracle GEMM
    cols = torch.nn.functional.unfold(x[:, :2].detach(), 3, padding=1).transpose(1, 2).reshape(98, 18)
    w0 = conv.weight[:3].detach().reshape(3, 18)
    want = oracle.mm(npy(cols), npy(w0).T.copy(), 10, 5, 3, 4, True, False, False, "tile8") + npy(conv.bias[:3]).reshape(1, 3)
    got = npy(y[:, :3]).transpose(0, 2, 3, 1).reshape(98, 3)
    assert same_bits(got, want.astype(np.float32)), mismatch_report(got, want)
    ref = torch.nn.functional.conv2d(x.detach(), conv.weight.detach(), conv.bias.detach(), padding=1, groups=2)
    assert torch.allclose(y, ref, atol=0.3)


def test_quantizer_module_and_ste():
    qz = q.Quantizer(fp(4, 3, True, True), fp(5, 2, True, True), "nearest", "nearest").cuda()
    x = torch.randn(64, device="cuda", requires_grad=True)
    y = qz(x)
    assert torch.equal(y, q.float_quantize(x.detach(), 4, 3, "nearest", True, True))
    g = torch.randn(64, device="cuda")
    y.backward(g)
    assert torch.equal(x.grad, q.float_quantize(g, 5, 2, "nearest", True, True))


def test_fused_tensor_scaling_equals_reference_sequence():
    """compute_bias -> scale -> quantize as two kernels against the reference's sequence of torch operations and the
    quantizer call (functional.py:39-53), bit for bit, scales included; then a scaled QLinear forward and backward with
    the fused path on and off."""
    g = torch.Generator(device="cuda").manual_seed(21)
    fmt = mp.FloatingPoint(4, 3, True, True)
    quant = q.quant_format.make_quant_function(fmt, "nearest")
    for shape in [(64, 48), (5, 33, 70), (2, 3, 16, 8), (1, 1)]:
        x = torch.randn(shape, device="cuda", generator=g) * (10.0 ** torch.randint(-6, 6, shape[:-2] + (1, 1), device="cuda", generator=g).float())
        for margin in (0, 2):
            for qq in (quant, Fq.id_quant):
                got, s = Fq._scaled_quant(x, fmt, margin, qq)
                ws = Fq.compute_bias(x, fmt, margin)
                want = qq(Fq.scale(x, ws))
                assert s.shape == ws.shape and torch.equal(s, ws), (shape, margin)
                assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (shape, margin)
    z = torch.zeros(4, 4, device="cuda")                     # amax = 0: the reference yields inf * 0 = NaN everywhere
    got, s = Fq._scaled_quant(z, fmt, 0, quant)
    assert torch.isinf(s).all() and torch.isnan(got).all()

    f = q.QAffineFormats(fwd_mac=(mp.FloatingPoint(5, 10, True, False), fmt), bwd_mac=(mp.FloatingPoint(5, 10, True, False), fmt),
                         weight_quant=(fmt, "nearest"), input_quant=(fmt, "nearest"), grad_quant=(mp.FloatingPoint(5, 2, True, True), "nearest"),
                         use_scaling=True, scale_margin=1)
    torch.manual_seed(5)
    lin = q.QLinear(48, 40, f).cuda()
    xin = (torch.randn(3, 20, 48, device="cuda") * 1e-3)
    outs = []
    for fused in (True, False):
        spec = Fq._float_nearest_spec
        if not fused:
            Fq._float_nearest_spec = lambda quant: None
        try:
            xi = xin.clone().requires_grad_(True)
            lin.zero_grad()
            y = lin(xi)
            (y * torch.linspace(-1, 1, y.numel(), device="cuda").view_as(y)).sum().backward()
            outs.append((y.detach().clone(), xi.grad.clone(), lin.weight.grad.clone(), lin.bias.grad.clone()))
        finally:
            Fq._float_nearest_spec = spec
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("grad_rounding", ["nearest", "stochastic"])
def test_two_stream_backward_equals_one_stream_backward(grad_rounding):
    """The input gradient and the weight gradient of a layer are launched on two streams; gradients, repeated steps and
    a stochastic gradient quantizer (seeds drawn on the host in the same order) give the bits of the one-stream pass."""
    add, mul = fp(5, 10, True, False), fp(4, 3, True, False)
    fmt = q.QAffineFormats(fwd_mac=(add, mul), bwd_mac=(add, mul), fwd_rnd="nearest", bwd_rnd="nearest",
                           weight_quant=(fp(4, 3, True, True), "nearest"), input_quant=(fp(4, 3, True, True), "nearest"),
                           grad_quant=(fp(5, 2, True, True), grad_rounding))
    results = []
    for overlap in (True, False):
        Fq.overlap_backward_gemms = overlap
        try:
            torch.manual_seed(5)
            lin1, lin2 = q.QLinear(192, 320, fmt, bias=True).cuda(), q.QLinear(320, 64, fmt, bias=True).cuda()
            x = torch.randn(4, 256, 192, device="cuda", requires_grad=True)
            a = torch.randn(2, 3, 128, 64, device="cuda", requires_grad=True)
            b = torch.randn(2, 3, 64, 96, device="cuda", requires_grad=True)
            out = []
            for step in range(3):
                for t in (x, a, b, *lin1.parameters(), *lin2.parameters()):
                    t.grad = None
                y = lin2(torch.nn.functional.gelu(lin1(x)))
                z = Fq.qmatmul(a, b, fmt)
                (y.square().mean() + z.square().mean()).backward()
                out += [t.grad.clone() for t in (x, a, b, *lin1.parameters(), *lin2.parameters())]
            torch.cuda.synchronize()
            results.append(out)
        finally:
            Fq.overlap_backward_gemms = True
    for u, v in zip(*results):
        assert torch.equal(u.view(torch.int32), v.view(torch.int32))
