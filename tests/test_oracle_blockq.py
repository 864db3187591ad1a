"""MX / NVFP4 oracle definitions: internal consistency and a third-party cross-check of the element encodings with
ml_dtypes (OCP float8_e4m3fn, float4_e2m1fn, float8_e8m0fnu).  The reference has no such quantizers: parity unpinned."""
import numpy as np
import pytest

ml_dtypes = pytest.importorskip("ml_dtypes")


def data(rows, cols, seed):
    rng = np.random.default_rng(seed)
    s = 10.0 ** rng.uniform(-3, 3, size=(rows, 1))
    return (rng.standard_normal((rows, cols)) * s).astype(np.float32)


@pytest.mark.parametrize("elem,dt,emax,top", [("e4m3", "float8_e4m3fn", 8, 448.0), ("e2m1", "float4_e2m1fn", 2, 6.0)])
def test_mx_matches_ml_dtypes_casts(oracle, elem, dt, emax, top):
    x = data(16, 256, 1)
    q, codes = oracle.mx_quantize(x, elem, 32)
    blocks = x.reshape(16, 8, 32)
    amax = np.abs(blocks).max(-1)
    e = np.floor(np.log2(amax)).astype(np.int32) - emax
    assert np.array_equal(codes.astype(np.int32), e + 127)
    # E8M0 codes decode to the same power of two with ml_dtypes
    scale = np.ldexp(1.0, e).astype(np.float32)
    assert np.array_equal(codes.view(ml_dtypes.float8_e8m0fnu).astype(np.float32), scale)
    scaled = blocks / scale[..., None]
    inrange = np.abs(scaled) <= top
    cast = scaled.astype(getattr(ml_dtypes, dt)).astype(np.float32)
    want = np.where(inrange, cast, np.sign(scaled) * top) * scale[..., None]
    assert np.array_equal(q.reshape(16, 8, 32), want.astype(np.float32))
    # idempotent: quantized data quantizes to itself with the same scales
    q2, codes2 = oracle.mx_quantize(q, elem, 32)
    assert np.array_equal(q2, q)


def test_mx_special_blocks(oracle):
    x = np.zeros((3, 64), dtype=np.float32)
    x[1, 5] = np.inf
    x[2, 40] = np.nan
    x[2, 3] = 1.0
    q, codes = oracle.mx_quantize(x, "e4m3", 32)
    assert codes[0, 0] == 0 and codes[0, 1] == 0 and np.all(q[0] == 0)
    assert codes[1, 0] == 0xFF and np.all(np.isnan(q[1, :32])) and np.all(q[1, 32:] == 0)
    assert codes[2, 1] == 0xFF and q[2, 3] == 1.0
    # ragged last block
    r, c = oracle.mx_quantize(np.arange(40, dtype=np.float32).reshape(1, 40), "e2m1", 32)
    assert c.shape == (1, 2) and r.shape == (1, 40)


def test_nvfp4_matches_ml_dtypes_casts(oracle):
    x = data(8, 128, 2)
    q, sb, sg = oracle.nvfp4_quantize(x)
    assert sg == np.float32(np.abs(x).max() / np.float32(448.0 * 6.0))
    blocks = x.reshape(8, 8, 16)
    amax = np.abs(blocks).max(-1)
    ratio = (amax / (np.float32(6.0) * np.float32(sg))).astype(np.float32)
    want_sb = np.minimum(ratio, 448).astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
    assert np.array_equal(sb, want_sb)
    sc = (sb * np.float32(sg)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (blocks / sc[..., None]).astype(np.float32)
    cast = np.clip(v, -6, 6).astype(ml_dtypes.float4_e2m1fn).astype(np.float32)
    want = np.where(sc[..., None] == 0, 0, cast * sc[..., None]).astype(np.float32)
    assert np.array_equal(q.reshape(8, 8, 16), want)
    q2, _, sg2 = oracle.nvfp4_quantize(x, global_scale=0.01)
    assert sg2 == np.float32(0.01) and np.all(np.abs(q2) <= 6 * 448 * 0.01 * 1.001)


def test_packed_codes_decode_with_ml_dtypes(oracle):
    """The packed element and scale codes decode, with ml_dtypes' own types, to the dequantized output."""
    x = data(8, 128, 3)
    for elem, dt in (("e4m3", ml_dtypes.float8_e4m3fn), ("e2m1", ml_dtypes.float4_e2m1fn)):
        q, sc, codes = oracle.mx_quantize(x, elem, 32, return_codes=True)
        if elem == "e4m3":
            vals = codes.view(dt).astype(np.float32)
        else:
            vals = np.stack([codes & 0xF, codes >> 4], -1).reshape(8, 128).astype(np.uint8).view(dt).astype(np.float32)
        scale = np.ldexp(1.0, sc.astype(np.int32) - 127).astype(np.float32)
        assert np.array_equal((vals.reshape(8, 4, 32) * scale[..., None]).reshape(8, 128), q)
    q, sb, sg, codes, scodes = oracle.nvfp4_quantize(x, 0.0, return_codes=True)
    vals = np.stack([codes & 0xF, codes >> 4], -1).reshape(8, 128).astype(np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32)
    assert np.array_equal(scodes.view(ml_dtypes.float8_e4m3fn).astype(np.float32), sb)
    assert np.array_equal((vals.reshape(8, 8, 16) * (sb * np.float32(sg))[..., None]).reshape(8, 128).astype(np.float32), q)
    # NaN handling of NVFP4: kept in a zero block, skipped by the tensor scale
    z = np.zeros((2, 32), dtype=np.float32)
    z[0, 3] = np.nan
    z[1, 7] = np.inf
    z[1, 9] = 2.0
    q, sb, sg = oracle.nvfp4_quantize(z)
    assert np.isnan(q[0, 3]) and np.all(q[0, :3] == 0) and sg == np.float32(2.0 / (448.0 * 6.0)) and q[1, 9] == 2.0
