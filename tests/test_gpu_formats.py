"""GPU parity of the GEMM and the softmax / layernorm kernels with supernormal-float and binary8 rounding formats.

Against the CPU oracle: GEMM, softmax backward and layernorm (built from +, -, *, /, sqrt) bit for bit in both
association orders.  Against the reference's own CUDA extension on the same GPU (oracle/_ref/quant_cuda, built from
the unmodified reference sources): everything, including the expf/logf softmax forwards, bit for bit."""
import numpy as np
import pytest
import torch

from conftest import mismatch_report, same_bits

pytestmark = pytest.mark.gpu

ORDERS = [("cuda", "tile8", "tree64"), ("seq", "seq", "seq")]
SFP = [(2, 5, 1, 1), (3, 4, 2, 1), (7, 8, 1, 1), (2, 5, 1, 3)]        # man, exp, binades_l, binades_u
B8 = [(3, True, "saturate_maxfloat"), (4, True, "saturate_infty"), (5, False, "saturate_maxfloat2"), (2, True, "saturate_maxfloat")]


@pytest.fixture(scope="module")
def q():
    import mptorch_b200.quant as quant

    return quant


@pytest.fixture(scope="module")
def ref_cuda():
    from oracle.build_ref import load_ref

    try:
        mod = load_ref("quant_cuda")
    except Exception as ex:  # pragma: no cover
        pytest.skip("reference quant_cuda could not be loaded: %r" % (ex,))
    if mod is None:
        pytest.skip("oracle/_ref/quant_cuda not built")
    return mod


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def bits_equal(a, b):
    a, b = a.contiguous(), b.contiguous()
    same = a.view(torch.int32) == b.view(torch.int32)
    return bool((same | (a.isnan() & b.isnan())).all())


# ------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("shape", [(64, 64, 64), (37, 129, 53), (130, 8, 70), (5, 1, 3)])
@pytest.mark.parametrize("order", ORDERS)
def test_superfp_mm_vs_oracle(q, oracle, shape, order):
    M, K, N = shape
    rng = np.random.default_rng(M * 1000 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    for (man, exp, bl, bu) in SFP:
        for sat in (False, True):
            for fma in (False, True):
                with q.orders(accum=order[0]):
                    got = q.superfp_mm(dev(a), dev(b), man, exp, (bl, bu), man, exp, (bl, bu), "nearest", fma, sat).cpu().numpy()
                f = oracle.fmt_superfp(man, exp, bl, bu, sat)
                want = oracle.mm_fmt(a, b, f, f, fma, order[1])
                assert same_bits(got, want), f"superfp m{man}e{exp} b({bl},{bu}) sat={sat} fma={fma}: " + mismatch_report(got, want)


@pytest.mark.parametrize("order", ORDERS)
def test_superfp_mm_mixed_formats_and_range(q, oracle, order):
    """Different add and multiply formats, inputs spanning the supernormal binades at both ends of the range."""
    rng = np.random.default_rng(11)
    a = (rng.standard_normal((48, 96)) * np.exp2(rng.integers(-12, 12, (48, 96)))).astype(np.float32)
    b = (rng.standard_normal((96, 40)) * np.exp2(rng.integers(-12, 12, (96, 40)))).astype(np.float32)
    with q.orders(accum=order[0]):
        got = q.superfp_mm(dev(a), dev(b), 3, 5, (2, 2), 2, 4, 1, "nearest", False, False).cpu().numpy()
    want = oracle.mm_fmt(a, b, oracle.fmt_superfp(3, 5, 2, 2, False), oracle.fmt_superfp(2, 4, 1, 1, False), False, order[1])
    assert same_bits(got, want), mismatch_report(got, want)


@pytest.mark.parametrize("order", ORDERS)
def test_superfp_bmm_shapes(q, oracle, order):
    rng = np.random.default_rng(3)
    f = oracle.fmt_superfp(2, 5, 1, 1, False)
    a3 = rng.standard_normal((3, 20, 33)).astype(np.float32)
    b3 = rng.standard_normal((3, 33, 17)).astype(np.float32)
    b2 = rng.standard_normal((33, 17)).astype(np.float32)
    a4 = rng.standard_normal((2, 2, 9, 16)).astype(np.float32)
    b4 = rng.standard_normal((2, 2, 16, 7)).astype(np.float32)
    with q.orders(accum=order[0]):
        got33 = q.superfp_bmm(dev(a3), dev(b3), 2, 5, 1, 2, 5, 1, "nearest", False).cpu().numpy()
        got32 = q.superfp_bmm(dev(a3), dev(b2), 2, 5, 1, 2, 5, 1, "nearest", False).cpu().numpy()
        got44 = q.superfp_bmm(dev(a4), dev(b4), 2, 5, 1, 2, 5, 1, "nearest", True).cpu().numpy()
    assert same_bits(got33, oracle.mm_fmt(a3, b3, f, f, False, order[1]))
    assert same_bits(got32, oracle.mm_fmt(a3.reshape(60, 33), b2, f, f, False, order[1]).reshape(3, 20, 17))
    assert same_bits(got44, oracle.mm_fmt(a4.reshape(4, 9, 16), b4.reshape(4, 16, 7), f, f, True, order[1]).reshape(2, 2, 9, 7))


def test_mp_mm_dispatches_supernormal(q, oracle):
    from mptorch_b200.number import SuperNormalFloat
    from mptorch_b200.quant import QAffineFormats

    rng = np.random.default_rng(9)
    a = rng.standard_normal((33, 70)).astype(np.float32)
    b = rng.standard_normal((70, 21)).astype(np.float32)
    fmt = SuperNormalFloat(exp=5, man=2, binades=1, saturate=False)
    formats = QAffineFormats(fwd_mac=(fmt, fmt), fwd_rnd="nearest", bwd_mac=(fmt, fmt), bwd_rnd="nearest")
    with q.orders(accum="seq"):
        got = q.mp_mm(dev(a), dev(b), formats, use_forward=True).cpu().numpy()
    f = oracle.fmt_superfp(2, 5, 1, 1, False)
    want = oracle.mm_fmt(a, b, f, f, bool(formats.fwd_fma), "seq")
    assert same_bits(got, want), mismatch_report(got, want)


def test_mm_fmt_binary8_and_mixed_kinds(oracle):
    """The generic entry point takes any pair of formats; the reference has no binary8 GEMM, the oracle defines it."""
    from mptorch_b200 import backend as be

    rng = np.random.default_rng(21)
    a = rng.standard_normal((50, 77)).astype(np.float32)
    b = rng.standard_normal((77, 31)).astype(np.float32)
    cases = [
        (be.Format.binary8(4, True, 1, True), be.Format.binary8(3, True, 1, True), oracle.fmt_binary8(4, True, 1, True), oracle.fmt_binary8(3, True, 1, True)),
        (be.Format.float(10, 5, True, False), be.Format.superfp(2, 5, 1, 1, False), oracle.fmt_float(10, 5, True, False), oracle.fmt_superfp(2, 5, 1, 1, False)),
        (be.Format.float(7, 8, True, False), be.Format.binary8(4, True, 0, True), oracle.fmt_float(7, 8, True, False), oracle.fmt_binary8(4, True, 0, True)),
    ]
    for order, oorder in (("cuda", "tile8"), ("seq", "seq")):
        for fa, fm, ofa, ofm in cases:
            for fma in (False, True):
                c = torch.empty(50, 31, device="cuda")
                be.mm_fmt(dev(a), dev(b), c, 1, 50, 31, 77, fa, fm, fma, order)
                want = oracle.mm_fmt(a, b, ofa, ofm, fma, oorder)
                assert same_bits(c.cpu().numpy(), want), mismatch_report(c.cpu().numpy(), want)


def test_mm_fmt_float_equals_float_entry(oracle):
    """A float descriptor through the generic entry point takes the same kernels as the float entry point."""
    from mptorch_b200 import backend as be

    a = torch.randn(300, 520, device="cuda")
    b = torch.randn(520, 260, device="cuda")
    for (e, m) in [(5, 2), (4, 3), (8, 7)]:
        c1 = torch.empty(300, 260, device="cuda")
        c2 = torch.empty(300, 260, device="cuda")
        be.float_quantize_nearest_mm(a, b, c1, 300, 260, 520, m, e, m, e, True, False, False)
        be.mm_fmt(a, b, c2, 1, 300, 260, 520, be.Format.float(m, e, True, False), be.Format.float(m, e, True, False), False)
        assert bits_equal(c1, c2)


def test_superfp_mm_vs_reference_cuda(ref_cuda):
    from mptorch_b200 import backend as be

    for (M, K, N) in [(256, 256, 256), (78, 101, 145)]:
        a = torch.randn(M, K, device="cuda")
        b = torch.randn(K, N, device="cuda")
        for (man, exp, bl, bu) in SFP:
            want = torch.zeros(M, N, device="cuda")
            ref_cuda.superfp_quantize_nearest_mm(a, b, want, M, N, K, man, exp, man, exp, bl, bu, bl, bu, False)
            got = torch.empty(M, N, device="cuda")
            be.superfp_quantize_nearest_mm(a, b, got, M, N, K, man, exp, man, exp, bl, bu, bl, bu, False, order="cuda")
            assert bits_equal(got, want), ("mm", M, K, N, man, exp, bl, bu)
            want = torch.zeros(M, N, device="cuda")
            ref_cuda.superfp_quantize_nearest_mm_fma(a, b, want, M, N, K, man, exp, bl, bu, False)
            got = torch.empty(M, N, device="cuda")
            be.superfp_quantize_nearest_mm_fma(a, b, got, M, N, K, man, exp, bl, bu, False, order="cuda")
            assert bits_equal(got, want), ("mm_fma", M, K, N, man, exp, bl, bu)
    a = torch.randn(5, 64, 48, device="cuda")
    b = torch.randn(5, 48, 72, device="cuda")
    want = torch.zeros(5, 64, 72, device="cuda")
    ref_cuda.superfp_quantize_nearest_bmm(a, b, want, 64, 72, 48, 2, 5, 2, 5, 1, 1, 1, 1, False)
    got = torch.empty(5, 64, 72, device="cuda")
    be.superfp_quantize_nearest_bmm(a, b, got, 64, 72, 48, 2, 5, 2, 5, 1, 1, 1, 1, False, order="cuda")
    assert bits_equal(got, want)


# ------------------------------------------------------------------------------------------ softmax
def _ofmt(oracle, kind, spec, sat_or_sub=None):
    if kind == "superfp":
        man, exp, bl, bu = spec
        return oracle.fmt_superfp(man, exp, bl, bu, False)
    P, sg, pol = spec
    return oracle.fmt_binary8(P, sg, pol, True)


@pytest.mark.parametrize("shape,dim", [((4, 37, 5), 1), ((4, 37, 5), 2), ((3, 200), -1), ((5, 130), 0)])
@pytest.mark.parametrize("order", ORDERS)
def test_softmax_backward_formats_exact(q, oracle, shape, dim, order):
    rng = np.random.default_rng(17)
    y = rng.random(shape).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    for (man, exp, bl, bu) in SFP:
        with q.orders(reduce=order[0]):
            got = q.superfp_softmax_backward(dev(y), dev(g), dim, man, exp, (bl, bu), man, exp, (bl, bu)).cpu().numpy()
        f = oracle.fmt_superfp(man, exp, bl, bu, False)
        want = oracle.softmax_backward_fmt(y, g, dim, f, f, order[2])
        assert same_bits(got, want), f"superfp {man},{exp},{bl},{bu}: " + mismatch_report(got, want)
    for (P, sg, pol) in B8:
        with q.orders(reduce=order[0]):
            got = q.binary8_softmax_backward(dev(y), dev(g), dim, P, pol, sg, P, pol, sg, "nearest", True).cpu().numpy()
        f = oracle.fmt_binary8(P, sg, pol, True)
        want = oracle.softmax_backward_fmt(y, g, dim, f, f, order[2])
        assert same_bits(got, want), f"binary8 P{P} {sg} {pol}: " + mismatch_report(got, want)


@pytest.mark.parametrize("order", ORDERS)
def test_softmax_forward_formats_close_to_oracle(q, oracle, order):
    """expf / logf differ between the CUDA math library and glibc in the last place: compare to a few quanta here,
    bit for bit against the reference CUDA kernels below."""
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((6, 150)) * 2).astype(np.float32)
    for (man, exp, bl, bu) in [(7, 8, 1, 1), (10, 5, 1, 1)]:
        with q.orders(reduce=order[0]):
            got = q.superfp_softmax_forward(dev(x), -1, man, exp, (bl, bu), man, exp, (bl, bu), man, exp, (bl, bu)).cpu().numpy()
            got2 = q.superfp_softmax_lse_forward(dev(x), -1, man, exp, (bl, bu), man, exp, (bl, bu)).cpu().numpy()
        f = oracle.fmt_superfp(man, exp, bl, bu, False)
        tol = 4.0 * 2.0 ** (-man)
        np.testing.assert_allclose(got, oracle.softmax_forward_fmt(x, -1, f, f, f, order[2]), rtol=tol, atol=tol * 1e-3)
        np.testing.assert_allclose(got2, oracle.softmax_lse_forward_fmt(x, -1, f, f, order[2]), rtol=tol, atol=tol * 1e-3)


def test_softmax_formats_vs_reference_cuda(q, ref_cuda):
    from mptorch_b200 import backend as be

    x = torch.randn(6, 40, 256, device="cuda") * 3
    g = torch.randn_like(x)
    pol = {"saturate_infty": ref_cuda.OverflowPolicy.SATURATE_INFTY, "saturate_maxfloat": ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT,
           "saturate_maxfloat2": ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT2}
    for dim in (-1, 1):
        for (man, exp, bl, bu) in SFP:
            want = torch.zeros_like(x)
            ref_cuda.superfp_quantize_nearest_softmax_forward(x, want, dim, man, exp, bl, bu, man, exp, bl, bu, man, exp, bl, bu, False)
            got = q.superfp_softmax_forward(x, dim, man, exp, (bl, bu), man, exp, (bl, bu), man, exp, (bl, bu))
            assert bits_equal(got, want), ("superfp softmax", man, exp, bl, bu, dim)
            want2 = torch.zeros_like(x)
            ref_cuda.superfp_quantize_nearest_softmax_lse_forward(x, want2, dim, man, exp, bl, bu, man, exp, bl, bu, False)
            got2 = q.superfp_softmax_lse_forward(x, dim, man, exp, (bl, bu), man, exp, (bl, bu))
            assert bits_equal(got2, want2), ("superfp softmax lse", man, exp, bl, bu, dim)
            want3 = torch.zeros_like(x)
            ref_cuda.superfp_quantize_nearest_softmax_backward(want, g, want3, dim, man, exp, bl, bu, man, exp, bl, bu, False)
            got3 = q.superfp_softmax_backward(want, g, dim, man, exp, (bl, bu), man, exp, (bl, bu))
            assert bits_equal(got3, want3), ("superfp softmax bwd", man, exp, bl, bu, dim)
        for (P, sg, po) in B8:
            want = torch.zeros_like(x)
            ref_cuda.binary8_quantize_nearest_softmax_forward(x, want, dim, P, pol[po], sg, P, pol[po], sg, P, pol[po], sg, True)
            got = q.binary8_softmax_forward(x, dim, P, po, sg, P, po, sg, P, po, sg, "nearest", True)
            assert bits_equal(got, want), ("binary8 softmax", P, sg, po, dim)
            want2 = torch.zeros_like(x)
            ref_cuda.binary8_quantize_nearest_softmax_lse_forward(x, want2, dim, P, pol[po], sg, P, pol[po], sg, True)
            got2 = q.binary8_softmax_lse_forward(x, dim, P, po, sg, P, po, sg, "nearest", True)
            assert bits_equal(got2, want2), ("binary8 softmax lse", P, sg, po, dim)
            want3 = torch.zeros_like(x)
            ref_cuda.binary8_quantize_nearest_softmax_backward(want, g, want3, dim, P, pol[po], sg, P, pol[po], sg, True)
            got3 = q.binary8_softmax_backward(want, g, dim, P, po, sg, P, po, sg, "nearest", True)
            assert bits_equal(got3, want3), ("binary8 softmax bwd", P, sg, po, dim)


# ------------------------------------------------------------------------------------------ layernorm
@pytest.mark.parametrize("shape,dims", [((4, 33, 96), [-1]), ((3, 5, 8, 12), [-1, -2]), ((7, 300), [-1])])
@pytest.mark.parametrize("order", ORDERS)
def test_layernorm_formats_exact(q, oracle, shape, dims, order):
    rng = np.random.default_rng(23)
    x = (rng.standard_normal(shape) * 2 + 0.25).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    nshape = [shape[d] for d in sorted(dims)]
    w = rng.standard_normal(nshape).astype(np.float32)
    b = rng.standard_normal(nshape).astype(np.float32)
    specs = [("superfp", s) for s in SFP[:3]] + [("binary8", s) for s in B8[:3]]
    for kind, spec in specs:
        f = _ofmt(oracle, kind, spec)
        with q.orders(reduce=order[0]):
            if kind == "superfp":
                man, exp, bl, bu = spec
                bn = (bl, bu)
                y, mean, rstd = q.superfp_layernorm_forward(dev(x), dev(w), dev(b), 1e-5, dims, man, exp, bn, man, exp, bn, man, exp, bn, man, exp, bn)
                gi, gw, gb = q.superfp_layernorm_backward(dev(x), dev(g), dev(w), dev(b), mean, rstd, dims, man, exp, bn, man, exp, bn, man, exp, bn)
            else:
                P, sg, pol = spec
                y, mean, rstd = q.binary8_layernorm_forward(dev(x), dev(w), dev(b), 1e-5, dims, P, pol, sg, P, pol, sg, P, pol, sg, P, pol, sg, "nearest", True)
                gi, gw, gb = q.binary8_layernorm_backward(dev(x), dev(g), dev(w), dev(b), mean, rstd, dims, P, pol, sg, P, pol, sg, P, pol, sg, "nearest", True)
        wy, wmean, wrstd = oracle.layernorm_forward_fmt(x, w, b, 1e-5, dims, f, f, f, f, order[2])
        tag = f"{kind} {spec} "
        assert same_bits(y.cpu().numpy(), wy), tag + "y: " + mismatch_report(y.cpu().numpy(), wy)
        assert same_bits(mean.cpu().numpy().ravel(), wmean), tag + "mean"
        assert same_bits(rstd.cpu().numpy().ravel(), wrstd), tag + "rstd"
        wgi, wgw, wgb = oracle.layernorm_backward_fmt(x, g, w, wmean, wrstd, dims, f, f, f, order[2])
        assert same_bits(gi.cpu().numpy(), wgi), tag + "grad_input: " + mismatch_report(gi.cpu().numpy(), wgi)
        assert same_bits(gw.cpu().numpy().ravel(), wgw), tag + "grad_gamma"
        assert same_bits(gb.cpu().numpy().ravel(), wgb), tag + "grad_beta"


def test_layernorm_formats_vs_reference_cuda(q, ref_cuda):
    xl = torch.randn(4, 64, 384, device="cuda") * 2 + 0.3
    gl = torch.randn_like(xl)
    w = torch.randn(384, device="cuda")
    b = torch.randn(384, device="cuda")
    pol = {"saturate_infty": ref_cuda.OverflowPolicy.SATURATE_INFTY, "saturate_maxfloat": ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT,
           "saturate_maxfloat2": ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT2}

    def fresh():
        return (torch.zeros_like(xl), torch.zeros(4, 64, device="cuda"), torch.zeros(4, 64, device="cuda"), torch.zeros_like(xl),
                torch.zeros(384, device="cuda"), torch.zeros(384, device="cuda"))

    for (man, exp, bl, bu) in SFP[:3]:
        y, mean, rstd, gi, gg, gb = fresh()
        ref_cuda.superfp_quantize_layernorm_forward(xl, w, b, y, mean, rstd, 1e-5, [-1], man, exp, bl, bu, man, exp, bl, bu, man, exp, bl, bu,
                                                    man, exp, bl, bu, False)
        bn = (bl, bu)
        oy, om, orr = q.superfp_layernorm_forward(xl, w, b, 1e-5, [-1], man, exp, bn, man, exp, bn, man, exp, bn, man, exp, bn)
        assert bits_equal(oy, y) and bits_equal(om, mean) and bits_equal(orr, rstd), ("superfp layernorm fwd", man, exp, bl, bu)
        ref_cuda.superfp_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, gi, gg, gb, [-1], man, exp, bl, bu, man, exp, bl, bu, man, exp,
                                                     bl, bu, False)
        ogi, ogg, ogb = q.superfp_layernorm_backward(xl, gl, w, b, mean, rstd, [-1], man, exp, bn, man, exp, bn, man, exp, bn)
        assert bits_equal(ogi, gi) and bits_equal(ogg, gg) and bits_equal(ogb, gb), ("superfp layernorm bwd", man, exp, bl, bu)
    for (P, sg, po) in B8[:3]:
        y, mean, rstd, gi, gg, gb = fresh()
        ref_cuda.binary8_quantize_layernorm_forward(xl, w, b, y, mean, rstd, 1e-5, [-1], P, pol[po], sg, P, pol[po], sg, P, pol[po], sg, P,
                                                    pol[po], sg, True)
        oy, om, orr = q.binary8_layernorm_forward(xl, w, b, 1e-5, [-1], P, po, sg, P, po, sg, P, po, sg, P, po, sg, "nearest", True)
        assert bits_equal(oy, y) and bits_equal(om, mean) and bits_equal(orr, rstd), ("binary8 layernorm fwd", P, sg, po)
        ref_cuda.binary8_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, gi, gg, gb, [-1], P, pol[po], sg, P, pol[po], sg, P, pol[po], sg, True)
        ogi, ogg, ogb = q.binary8_layernorm_backward(xl, gl, w, b, mean, rstd, [-1], P, po, sg, P, po, sg, P, po, sg, "nearest", True)
        assert bits_equal(ogi, gi) and bits_equal(ogg, gg) and bits_equal(ogb, gb), ("binary8 layernorm bwd", P, sg, po)
