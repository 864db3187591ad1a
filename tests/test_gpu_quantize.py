"""GPU parity of the elementwise quantizers: CUDA kernels (through the C ABI) vs the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

from conftest import golden, mismatch_report, same_bits

pytestmark = pytest.mark.gpu

POL = ["saturate_infty", "saturate_maxfloat", "saturate_maxfloat2"]


@pytest.fixture(scope="module")
def be():
    from mptorch_b200 import backend

    return backend


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def inputs(seed, n):
    rng = np.random.default_rng(seed)
    rnd = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    return np.concatenate([golden("casters.npz")["in_bits"], rnd]).view(np.float32)


def mixture(n, seed, sigma_small=1e-3):
    """benchmark config 2 value distribution: 90% N(0,1), 5% N(0, sigma_small^2), 5% U(-1e5, 1e5)."""
    rng = np.random.default_rng(seed)
    u = rng.random(n)
    x = rng.standard_normal(n)
    x = np.where(u < 0.90, x, np.where(u < 0.95, x * sigma_small, rng.uniform(-1e5, 1e5, n)))
    return x.astype(np.float32)


@pytest.mark.parametrize("fmt", [(5, 2), (4, 3), (5, 10), (8, 7), (8, 1), (2, 23), (3, 0), (8, 23), (8, 0), (7, 22)])
def test_float_nearest_and_truncate(be, oracle, fmt):
    e, m = fmt
    x = inputs(e * 7 + m, 1 << 18)
    xd = dev(x)
    for sub in (False, True):
        for sat in (False, True):
            got = be.float_quantize_nearest(xd, m, e, sub, sat).cpu().numpy()
            want = oracle.float_quantize(x, m, e, "nearest", sub, sat)
            assert same_bits(got, want), f"nearest sub={sub} sat={sat}: " + mismatch_report(got, want)
            got = be.float_quantize_truncate(xd, m, e, sub, sat).cpu().numpy()
            want = oracle.float_quantize(x, m, e, "truncate", sub, sat)
            assert same_bits(got, want), f"truncate sub={sub} sat={sat}: " + mismatch_report(got, want)


def test_float_nearest_matches_reference_fixture(be):
    g = golden("casters.npz")
    xd = dev(g["in_bits"].view(np.float32))
    n = 0
    for key in g.files:
        if not key.startswith("fp_"):
            continue
        p = key.split("_")
        e, m = p[1][1:].split("m")
        got = be.float_quantize_nearest(xd, int(m), int(e), bool(int(p[2][3:])), bool(int(p[3][3:]))).cpu().numpy()
        want = g[key].view(np.float32)
        assert same_bits(got, want), key + ": " + mismatch_report(got, want)
        n += 1
    assert n == 48


@pytest.mark.parametrize("n", [0, 1, 3, 5, 1027, 4096 + 2])
def test_ragged_sizes_and_unaligned_pointers(be, oracle, n):
    x = mixture(n + 1, 3)
    xd = dev(x)
    for off in (0, 1):
        xs = xd[off:off + n]
        got = be.float_quantize_nearest(xs, 3, 4, True, True).cpu().numpy()
        want = oracle.float_quantize(x[off:off + n], 3, 4, "nearest", True, True)
        assert same_bits(got, want), mismatch_report(got, want)


def test_config2_mixture_all_roundings(be, oracle):
    n = 1 << 22
    for sigma in (1e-3, 1e-6):
        x = mixture(n, 11, sigma)
        xd = dev(x)
        got = be.float_quantize_nearest(xd, 3, 4, True, True).cpu().numpy()
        assert same_bits(got, oracle.float_quantize(x, 3, 4, "nearest", True, True))
        got = be.float_quantize_truncate(xd, 3, 4, True, True).cpu().numpy()
        assert same_bits(got, oracle.float_quantize(x, 3, 4, "truncate", True, True))
        torch.manual_seed(1)
        r = torch.randint_like(xd, 2147483647, dtype=torch.int32)
        got = be.float_quantize_stochastic(xd, 3, 4, 20, True, True, rand=r).cpu().numpy()
        want = oracle.float_quantize(x, 3, 4, "stochastic", True, True, rand=r.cpu().numpy(), rbits=20)
        assert same_bits(got, want), mismatch_report(got, want)
        got = be.binary8_quantize_nearest(xd, 3, True, be.OverflowPolicy.SATURATE_MAXFLOAT, True).cpu().numpy()
        want = oracle.binary8_quantize(x, 3, "nearest", "saturate_maxfloat", True, True)
        assert same_bits(got, want), mismatch_report(got, want)


@pytest.mark.parametrize("fmt", [(5, 2), (4, 3), (8, 7), (5, 10)])
def test_float_stochastic_explicit_bits(be, oracle, fmt):
    e, m = fmt
    x = inputs(99, 1 << 16)
    xd = dev(x)
    rng = np.random.default_rng(8)
    r = rng.integers(0, 2**31 - 1, size=x.size, dtype=np.int64).astype(np.int32)
    rd = dev(r)
    for sub in (False, True):
        for sat in (False, True):
            for rbits in (0, 23 - m, 5):
                got = be.float_quantize_stochastic(xd, m, e, rbits, sub, sat, rand=rd).cpu().numpy()
                want = oracle.float_quantize(x, m, e, "stochastic", sub, sat, rand=r, rbits=rbits)
                assert same_bits(got, want), f"sub={sub} sat={sat} rbits={rbits}: " + mismatch_report(got, want)


def test_float_stochastic_default_draw_is_torch_generator(be, oracle):
    """Without explicit words the draw is randint_like from the torch CUDA generator, as the reference does."""
    x = mixture(1 << 14, 5)
    xd = dev(x)
    torch.manual_seed(42)
    got = be.float_quantize_stochastic(xd, 2, 5, 21, True, False).cpu().numpy()
    torch.manual_seed(42)
    r = torch.randint_like(xd, 2147483647, dtype=torch.int32).cpu().numpy()
    want = oracle.float_quantize(x, 2, 5, "stochastic", True, False, rand=r, rbits=21)
    assert same_bits(got, want)


def test_float_stochastic_philox_matches_oracle_words(be, oracle):
    n = 4096 + 3
    x = mixture(n, 6)
    seed = 0x1234567890ABCDEF
    got = be.float_quantize_stochastic(dev(x), 3, 4, 20, True, True, seed=seed).cpu().numpy()
    words = np.concatenate([oracle.philox(b, 0, 0, 0, seed & 0xFFFFFFFF, seed >> 32) for b in range((n + 3) // 4)])[:n]
    r = (words & 0x7FFFFFFF).astype(np.int32)
    want = oracle.float_quantize(x, 3, 4, "stochastic", True, True, rand=r, rbits=20)
    assert same_bits(got, want), mismatch_report(got, want)


def test_stochastic_rounding_statistics(be):
    """Mean and variance of the rounding error: E[q(x)] = x, Var = (x-lo)(hi-x), for in-range values."""
    x = np.full(1 << 20, 1.3, dtype=np.float32)        # e4m3: neighbours 1.25 and 1.375
    q = be.float_quantize_stochastic(dev(x), 3, 4, 20, True, True, seed=7).cpu().numpy().astype(np.float64)
    assert set(np.unique(q)) == {1.25, 1.375}
    p_up = (np.float32(1.3) - 1.25) / 0.125
    assert abs(q.mean() - float(np.float32(1.3))) < 4 * 0.125 * np.sqrt(p_up * (1 - p_up) / x.size) + 1e-6
    assert abs(q.var() - 0.125**2 * p_up * (1 - p_up)) < 2e-5
    exact = np.array([1.25, -3.5, 0.015625, 240.0], dtype=np.float32)   # representable values are fixed points
    assert same_bits(be.float_quantize_stochastic(dev(exact), 3, 4, 20, True, True, seed=9).cpu().numpy(), exact)


@pytest.mark.parametrize("P", range(1, 8))
def test_binary8_all_modes(be, oracle, P):
    x = inputs(P, 1 << 15)
    xd = dev(x)
    rng = np.random.default_rng(P)
    r = rng.integers(0, 2**31 - 1, size=x.size, dtype=np.int64).astype(np.int32)
    rd = dev(r)
    for sg in (False, True):
        for po in range(3):
            for sub in (False, True):
                got = be.binary8_quantize_nearest(xd, P, sg, po, sub).cpu().numpy()
                want = oracle.binary8_quantize(x, P, "nearest", POL[po], sg, sub)
                assert same_bits(got, want), f"nearest sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)
                got = be.binary8_quantize_truncate(xd, P, sg, po, sub).cpu().numpy()
                want = oracle.binary8_quantize(x, P, "truncate", POL[po], sg, sub)
                assert same_bits(got, want), f"truncate sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)
                prng = 23 - (P - 1)
                got = be.binary8_quantize_stochastic(xd, P, prng, sg, po, sub, rand=rd).cpu().numpy()
                want = oracle.binary8_quantize(x, P, "stochastic", POL[po], sg, sub, rand=r, prng_bits=prng)
                assert same_bits(got, want), f"stochastic sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)


def test_superfp(be, oracle):
    x = inputs(123, 1 << 16)
    xd = dev(x)
    for (e, m, bl, bu) in [(4, 3, 1, 1), (4, 3, 2, 1), (5, 2, 1, 2), (3, 4, 1, 1), (6, 1, 2, 2), (4, 2, 3, 1), (7, 5, 1, 1)]:
        for sat in (False, True):
            got = be.superfp_quantize_nearest(xd, m, e, bl, bu, sat).cpu().numpy()
            want = oracle.superfp_quantize(x, m, e, bl, bu, sat)
            assert same_bits(got, want), f"e{e}m{m} l{bl} u{bu} sat={sat}: " + mismatch_report(got, want)


def test_checks_mirror_reference(be):
    with pytest.raises(RuntimeError):
        be.float_quantize_nearest(torch.zeros(4), 2, 5, True, True)            # not CUDA
    with pytest.raises(RuntimeError):
        be.float_quantize_nearest(torch.zeros(4, 4).cuda().t(), 2, 5, True, True)   # not contiguous
    with pytest.raises(RuntimeError):
        be.float_quantize_nearest(torch.zeros(4).cuda(), 30, 5, True, True)    # bad format -> C ABI error


def test_full_size_properties(be):
    """2^28 elements (benchmark config 2 size): idempotence, sign symmetry and agreement with a sharded run."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(n, device="cuda", generator=g)
    q = be.float_quantize_nearest(x, 3, 4, True, True)
    assert torch.equal(be.float_quantize_nearest(q, 3, 4, True, True), q)
    assert torch.equal(be.float_quantize_nearest(-x, 3, 4, True, True), -q)
    part = be.float_quantize_nearest(x[n // 2 - 1024:n // 2 + 1024].contiguous(), 3, 4, True, True)
    assert torch.equal(part, q[n // 2 - 1024:n // 2 + 1024])
    assert q.abs().max().item() <= 240.0
