"""GPU parity of the MX / NVFP4 block quantizers vs the CPU oracle (bit for bit)."""
import numpy as np
import pytest
import torch

from conftest import mismatch_report, same_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    import mptorch_b200.quant as quant

    return quant


def data(rows, cols, seed):
    """benchmark config 3 distribution: N(0,1) times a per-row scale drawn log-uniform over [1e-3, 1e3]."""
    rng = np.random.default_rng(seed)
    s = 10.0 ** rng.uniform(-3, 3, size=(rows, 1))
    return (rng.standard_normal((rows, cols)) * s).astype(np.float32)


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def specials(x):
    x = x.copy()
    x[0, :32] = 0.0
    x[1, 7] = np.inf
    x[2, 40] = np.nan
    x[3, :64] *= 1e-38
    x[4, :32] = np.float32(1e-45)
    x[5, 3] = 3e38
    x[6, :16] = -0.0
    return x


@pytest.mark.parametrize("elem", ["e4m3", "e2m1"])
@pytest.mark.parametrize("shape,block", [((64, 1024), 32), ((3, 5, 96), 32), ((16, 256), 16), ((7, 100), 32), ((5, 33), 8), ((1, 32), 32)])
def test_mx(q, oracle, elem, shape, block):
    x = data(int(np.prod(shape[:-1])), shape[-1], 3).reshape(shape)
    if shape == (64, 1024):
        x = specials(x)
    got, codes = q.mx_quantize(dev(x), elem, block, return_scales=True)
    want, wcodes = oracle.mx_quantize(x, elem, block)
    assert same_bits(got.cpu().numpy(), want), mismatch_report(got.cpu().numpy(), want)
    assert np.array_equal(codes.cpu().numpy(), wcodes)
    assert same_bits(q.mx_quantize(dev(x), elem, block).cpu().numpy(), want)


@pytest.mark.parametrize("shape", [(64, 1024), (3, 5, 96), (7, 100), (1, 16), (9, 24)])
def test_nvfp4(q, oracle, shape):
    x = data(int(np.prod(shape[:-1])), shape[-1], 4).reshape(shape)
    for gs in (None, 0.37):
        got, sb, sg = q.nvfp4_quantize(dev(x), gs, return_scales=True)
        want, wsb, wsg = oracle.nvfp4_quantize(x, 0.0 if gs is None else gs)
        assert np.float32(sg.item()) == np.float32(wsg)
        assert same_bits(sb.cpu().numpy(), wsb), mismatch_report(sb.cpu().numpy(), wsb)
        assert same_bits(got.cpu().numpy(), want), mismatch_report(got.cpu().numpy(), want)
    xs = specials(data(64, 1024, 5))
    xs[1, 7] = 5e4   # keep the tensor amax finite for the computed-scale arm
    xs[5, 3] = 2e4
    got = q.nvfp4_quantize(dev(xs)).cpu().numpy()
    want, _, _ = oracle.nvfp4_quantize(xs)
    assert same_bits(got, want), mismatch_report(got, want)
    z = np.zeros((4, 32), dtype=np.float32)
    assert same_bits(q.nvfp4_quantize(dev(z)).cpu().numpy(), oracle.nvfp4_quantize(z)[0])


def test_config3_full_size_properties(q, oracle):
    """16384 x 16384 (benchmark config 3): sampled rows equal the oracle; quantization is idempotent."""
    g = torch.Generator(device="cuda").manual_seed(9)
    n = 16384
    x = torch.randn(n, n, device="cuda", generator=g) * (10.0 ** (torch.rand(n, 1, device="cuda", generator=g) * 6 - 3))
    rows = [0, 1, 777, n - 1]
    for elem in ("e4m3", "e2m1"):
        y = q.mx_quantize(x, elem, 32)
        want, _ = oracle.mx_quantize(x[rows].cpu().numpy(), elem, 32)
        assert same_bits(y[rows].cpu().numpy(), want)
        assert torch.equal(q.mx_quantize(y, elem, 32), y)
        del y
    sgv = float(x.abs().max().item() / (448.0 * 6.0))
    y, sb, sg = q.nvfp4_quantize(x, None, return_scales=True)
    want, wsb, _ = oracle.nvfp4_quantize(x[rows].cpu().numpy(), float(sg.item()))
    assert same_bits(y[rows].cpu().numpy(), want)
    assert abs(sg.item() - sgv) <= 1e-6 * sgv


@pytest.mark.parametrize("elem", ["e4m3", "e2m1"])
@pytest.mark.parametrize("shape,block", [((64, 1024), 32), ((3, 5, 96), 32), ((16, 256), 16), ((7, 100), 32), ((5, 34), 8)])
def test_mx_packed_codes(q, oracle, elem, shape, block):
    """The packed element codes (a byte per E4M3 element, two E2M1 elements per byte) equal the oracle's, whose
    encoding is checked against ml_dtypes on the CPU."""
    x = data(int(np.prod(shape[:-1])), shape[-1], 6).reshape(shape)
    if shape == (64, 1024):
        x = specials(x)
    got, sc, codes = q.mx_quantize(dev(x), elem, block, return_scales=True, return_codes=True)
    want, wsc, wcodes = oracle.mx_quantize(x, elem, block, return_codes=True)
    assert same_bits(got.cpu().numpy(), want) and np.array_equal(sc.cpu().numpy(), wsc)
    assert codes.dtype == torch.uint8 and np.array_equal(codes.cpu().numpy(), wcodes)


@pytest.mark.parametrize("shape", [(64, 1024), (3, 5, 96), (7, 100), (1, 16), (9, 24)])
def test_nvfp4_packed_codes_and_nan_rules(q, oracle, shape):
    x = data(int(np.prod(shape[:-1])), shape[-1], 7).reshape(shape)
    got, sb, sg, codes, scodes = q.nvfp4_quantize(dev(x), None, return_scales=True, return_codes=True)
    want, wsb, wsg, wcodes, wscodes = oracle.nvfp4_quantize(x, 0.0, return_codes=True)
    assert same_bits(got.cpu().numpy(), want) and same_bits(sb.cpu().numpy(), wsb)
    assert np.array_equal(codes.cpu().numpy(), wcodes) and np.array_equal(scodes.cpu().numpy(), wscodes)
    # a NaN in an otherwise zero block stays NaN; infinities and NaN do not take part in the tensor scale
    z = np.zeros((4, 64), dtype=np.float32)
    z[1, 3] = np.nan
    z[2, 20] = np.inf
    z[3, 5] = 3.0
    got, sb, sg = q.nvfp4_quantize(dev(z), None, return_scales=True)
    want, wsb, wsg = oracle.nvfp4_quantize(z)
    g = got.cpu().numpy()
    assert np.float32(sg.item()) == np.float32(wsg) == np.float32(3.0 / (448.0 * 6.0))
    assert same_bits(g, want) and np.isnan(g[1, 3]) and g[3, 5] == 3.0 and np.isfinite(g[2, 20])
