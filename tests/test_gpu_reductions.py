"""GPU parity of the quantized softmax / layernorm / column-sum kernels vs the CPU oracle.

Everything built from +, -, *, /, sqrt is compared bit for bit in both association orders.  The softmax forward
passes call expf/logf: the CUDA math library and glibc agree to within an ulp but not always bit for bit, so against
the CPU oracle they are held to a stated tolerance here; their bit-exact pin is the same-GPU comparison with the
reference's own CUDA kernels in test_gpu_vs_reference_cuda.py."""
import numpy as np
import pytest
import torch

from conftest import golden, mismatch_report, same_bits

pytestmark = pytest.mark.gpu

FMTS = [(5, 10), (8, 7), (4, 3), (8, 23), (5, 2)]
ORDERS = [("cuda", "tree64"), ("seq", "seq")]


@pytest.fixture(scope="module")
def q():
    import mptorch_b200.quant as quant

    return quant


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


@pytest.mark.parametrize("shape,dim", [((4, 37, 5), 1), ((4, 37, 5), 0), ((4, 37, 5), 2), ((3, 200), -1), ((2, 3, 64), -1), ((7, 1), 1), ((5, 130), 1)])
@pytest.mark.parametrize("order", ORDERS)
def test_softmax_backward_exact(q, oracle, shape, dim, order):
    rng = np.random.default_rng(abs(hash((shape, dim))) % 2**32)
    y = rng.random(shape).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    for (e, m) in FMTS:
        with q.orders(reduce=order[0]):
            got = q.float_softmax_backward(dev(y), dev(g), dim, m, e, m, e, "nearest", True, False).cpu().numpy()
        want = oracle.softmax_backward(y, g, dim, m, e, m, e, True, False, order[1])
        assert same_bits(got, want), f"e{e}m{m}: " + mismatch_report(got, want)


def _close_softmax(got, want, man):
    """Tolerance for expf/logf library differences: a flipped rounding of one exponential moves a row by at most a
    couple of quanta of the working format."""
    assert np.all(np.isfinite(got) == np.isfinite(want))
    tol = 4.0 * 2.0 ** (-min(man, 23))
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * 1e-3)
    frac_exact = np.mean(got.view(np.uint32) == want.view(np.uint32))
    return frac_exact


@pytest.mark.parametrize("shape,dim", [((4, 37, 5), 1), ((4, 37, 5), 2), ((6, 300), -1), ((2, 3, 64), -1)])
@pytest.mark.parametrize("order", ORDERS)
def test_softmax_forward_close_to_oracle(q, oracle, shape, dim, order):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    for (e, m) in [(5, 10), (8, 7), (8, 23)]:
        with q.orders(reduce=order[0]):
            got = q.float_softmax_forward(dev(x), dim, m, e, m, e, m, e, "nearest", True, False).cpu().numpy()
            got_lse = q.float_softmax_lse_forward(dev(x), dim, m, e, m, e, "nearest", True, False).cpu().numpy()
        want = oracle.softmax_forward(x, dim, m, e, m, e, m, e, True, False, order[1])
        want_lse = oracle.softmax_lse_forward(x, dim, m, e, m, e, True, False, order[1])
        _close_softmax(got, want, m)
        _close_softmax(got_lse, want_lse, max(m - 3, 1))   # the LSE recurrence amplifies a flipped rounding


def test_softmax_rows_sum_to_one_and_specials(q):
    x = torch.randn(64, 1024, device="cuda") * 4
    y = q.float_softmax_forward(x, -1, 10, 5, 10, 5, 10, 5, "nearest", True, False)
    assert torch.all((y.sum(-1) - 1).abs() < 2e-2)
    x[3, 5] = float("inf")
    y = q.float_softmax_forward(x, -1, 10, 5, 10, 5, 10, 5, "nearest", True, False)
    assert torch.isnan(y[3]).all() or torch.isnan(y[3, 5])      # inf - inf -> NaN, as in the reference
    assert torch.isfinite(y[4]).all()


@pytest.mark.parametrize("shape,ndims", [((6, 5, 48), 1), ((4, 6, 8), 2), ((3, 130), 1), ((2, 2, 1), 1), ((70, 768), 1)])
@pytest.mark.parametrize("order", ORDERS)
def test_layernorm_forward_backward_exact(q, oracle, shape, ndims, order):
    rng = np.random.default_rng(sum(shape))
    x = (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    nshape = shape[len(shape) - ndims:]
    w = rng.standard_normal(nshape).astype(np.float32)
    b = rng.standard_normal(nshape).astype(np.float32)
    dims = [-(i + 1) for i in range(ndims)]
    for (e, m) in FMTS:
        with q.orders(reduce=order[0]):
            y, mean, rstd = q.float_layernorm_forward(dev(x), dev(w), dev(b), 1e-5, dims, m, e, m, e, m, e, m, e, "nearest", True, False)
        wy, wmean, wrstd = oracle.layernorm_forward(x, w.ravel(), b.ravel(), 1e-5, dims, m, e, m, e, m, e, m, e, True, False, order[1])
        assert same_bits(y.cpu().numpy(), wy), f"y e{e}m{m}: " + mismatch_report(y.cpu().numpy(), wy)
        assert same_bits(mean.cpu().numpy().ravel(), wmean), f"mean e{e}m{m}: " + mismatch_report(mean.cpu().numpy().ravel(), wmean)
        assert same_bits(rstd.cpu().numpy().ravel(), wrstd), f"rstd e{e}m{m}"
        with q.orders(reduce=order[0]):
            gi, gw, gb = q.float_layernorm_backward(dev(x), dev(g), dev(w), dev(b), mean, rstd, dims, m, e, m, e, m, e, "nearest", True, False)
        wgi, wgg, wgb = oracle.layernorm_backward(x, g, w.ravel(), wmean, wrstd, dims, m, e, m, e, m, e, True, False, order[1])
        assert same_bits(gi.cpu().numpy(), wgi), f"gi e{e}m{m}: " + mismatch_report(gi.cpu().numpy(), wgi)
        assert same_bits(gw.cpu().numpy().ravel(), wgg), f"gw e{e}m{m}: " + mismatch_report(gw.cpu().numpy().ravel(), wgg)
        assert same_bits(gb.cpu().numpy().ravel(), wgb), f"gb e{e}m{m}"


def test_layernorm_seq_matches_reference_fixture(q):
    """Against the reference CPU extension's outputs (tests/golden/reductions_seq.npz)."""
    g = golden("reductions_seq.npz")
    x, gr, w, b = g["ln_x"], g["ln_g"], g["ln_w"], g["ln_b"]
    for (e, m) in [(5, 10), (8, 7), (8, 23)]:
        with q.orders(reduce="seq"):
            y, mean, rstd = q.float_layernorm_forward(dev(x), dev(w), dev(b), 1e-5, [-1], m, e, m, e, m, e, m, e)
            gi, gw, gb = q.float_layernorm_backward(dev(x), dev(gr), dev(w), dev(b), mean, rstd, [-1], m, e, m, e, m, e)
        for got, name in ((y, "ln_fwd_y"), (mean, "ln_fwd_mean"), (rstd, "ln_fwd_rstd"), (gi, "ln_bwd_gi"), (gw, "ln_bwd_gg"), (gb, "ln_bwd_gb")):
            want = g[f"{name}_e{e}m{m}"].view(np.float32)
            assert same_bits(got.cpu().numpy().ravel(), want.ravel()), f"{name} e{e}m{m}"


def test_softmax_backward_seq_matches_reference_fixture(q):
    g = golden("reductions_seq.npz")
    for dim in (0, 1, 2):
        for (e, m) in [(5, 10), (8, 7), (4, 3)]:
            y = g[f"sm_fwd_dim{dim}_e{e}m{m}"].view(np.float32)
            with q.orders(reduce="seq"):
                got = q.float_softmax_backward(dev(y), dev(g["sm_g"]), dim, m, e, m, e).cpu().numpy()
            want = g[f"sm_bwd_dim{dim}_e{e}m{m}"].view(np.float32)
            assert same_bits(got, want), mismatch_report(got, want)


def test_qsum_rows(q, oracle):
    rng = np.random.default_rng(4)
    for (rows, cols) in [(1, 1), (17, 5), (300, 130), (8, 1000), (0, 4)]:
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        for (e, m) in FMTS:
            got = q.qsum_rows(dev(x), e, m, True, False).cpu().numpy()
            want = oracle.qsum_rows(x, m, e, True, False)
            assert same_bits(got, want), f"{rows}x{cols} e{e}m{m}: " + mismatch_report(got, want)


def test_config5_shapes(q, oracle):
    """benchmark config 5 reduction shapes: softmax rows of 1024 and layernorm rows of 768 (rows sampled for the oracle)."""
    g = torch.Generator(device="cuda").manual_seed(5)
    att = torch.randn(8, 12, 128, 1024, device="cuda", generator=g)
    y = q.float_softmax_forward(att, -1, 10, 5, 10, 5, 10, 5)
    gy = torch.randn(att.shape, device="cuda", generator=g)
    dx = q.float_softmax_backward(y, gy, -1, 10, 5, 3, 4)
    want = oracle.softmax_backward(y[1, 2, :16].cpu().numpy(), gy[1, 2, :16].cpu().numpy(), -1, 10, 5, 3, 4, True, False, "tree64")
    assert same_bits(dx[1, 2, :16].cpu().numpy(), want)
    x = torch.randn(8, 1024, 768, device="cuda", generator=g)
    w = torch.randn(768, device="cuda", generator=g)
    b = torch.randn(768, device="cuda", generator=g)
    out, mean, rstd = q.float_layernorm_forward(x, w, b, 1e-5, [-1], 10, 5, 3, 4, 10, 5, 10, 5)
    wy, wm, wr = oracle.layernorm_forward(x[3, :32].cpu().numpy(), w.cpu().numpy(), b.cpu().numpy(), 1e-5, [-1], 10, 5, 3, 4, 10, 5, 10, 5, True, False, "tree64")
    assert same_bits(out[3, :32].cpu().numpy(), wy) and same_bits(mean[3, :32].cpu().numpy(), wm)
    gi, gw, gb = q.float_layernorm_backward(x, gy[:, 0, :, :768].contiguous().reshape(8, 128, 768).repeat(1, 8, 1), w, b, mean, rstd, [-1], 10, 5, 3, 4, 10, 5)
    assert torch.isfinite(gi).all() and gw.shape == (768,) and gb.shape == (768,)
