"""Pins the CPU oracle (oracle/mpt_oracle.c): against the golden fixtures made from the reference's
compiled CPU extension, against the reference's own known-answer vectors, and -- where the reference
build is present -- against the live reference on larger random sweeps."""
import struct

import numpy as np
import pytest
import torch

from conftest import golden, mismatch_report, same_bits

POL = ["saturate_infty", "saturate_maxfloat", "saturate_maxfloat2"]


def b2f(bits):
    return struct.unpack(">f", struct.pack(">I", bits))[0]


# ------------------------------------------------------------------ golden fixtures: casters
def _caster_cases():
    g = golden("casters.npz")
    return [k for k in g.files if k not in ("in_bits", "b8_rand")]


@pytest.mark.parametrize("key", _caster_cases())
def test_caster_matches_reference_fixture(oracle, key):
    g = golden("casters.npz")
    x = g["in_bits"].view(np.float32)
    want = g[key].view(np.float32)
    p = key.split("_")
    if p[0] == "fp":
        e, m = p[1][1:].split("m")
        got = oracle.float_quantize(x, int(m), int(e), "nearest", bool(int(p[2][3:])), bool(int(p[3][3:])))
    elif p[0] == "b8":
        P, sg, po, sub, mode = int(p[1][1:]), int(p[2][2:]), int(p[3][2:]), int(p[4][3:]), p[5]
        if mode == "stochastic":
            got = oracle.binary8_quantize(x, P, mode, POL[po], bool(sg), bool(sub), rand=g["b8_rand"],
                                          prng_bits=int(p[6][4:]))
        else:
            got = oracle.binary8_quantize(x, P, mode, POL[po], bool(sg), bool(sub))
    else:
        e, m = p[1][1:].split("m")
        got = oracle.superfp_quantize(x, int(m), int(e), int(p[2][1:]), int(p[3][1:]), bool(int(p[4][3:])))
    assert same_bits(got, want), mismatch_report(got, want)


# ------------------------------------------------------------------ golden fixtures: GEMM (seq order)
def test_mm_seq_matches_reference_fixture(oracle):
    g = golden("mm_seq.npz")
    n = 0
    for key in g.files:
        p = key.split("_")
        if len(p) < 3 or p[1] not in ("mm", "fma") or p[0] == "big":
            continue
        a, b = g[p[0] + "_a"], g[p[0] + "_b"]
        want = g[key].view(np.float32)
        if p[1] == "mm":
            ea, ma = p[3][1:].split("m")
            em, mm_ = p[5][1:].split("m")
            got = oracle.mm(a, b, int(ma), int(ea), int(mm_), int(em), True, bool(int(p[6][3:])), False, "seq")
        else:
            ea, ma = p[2][1:].split("m")
            got = oracle.mm(a, b, int(ma), int(ea), int(ma), int(ea), True, False, True, "seq")
        assert same_bits(got, want), key + ": " + mismatch_report(got, want)
        n += 1
    assert n >= 30
    got = oracle.mm(g["bmm_a"], g["bmm_b"], 2, 5, 2, 5, True, False, False, "seq")
    assert same_bits(got, g["bmm_e5m2"].view(np.float32))
    for sat in (0, 1):  # overflow to inf / saturation inside the accumulation
        got = oracle.mm(g["big_a"], g["big_b"], 2, 5, 2, 5, True, bool(sat), False, "seq")
        want = g[f"big_mm_e5m2_sat{sat}"].view(np.float32)
        assert same_bits(got, want), mismatch_report(got, want)
        assert not np.all(np.isfinite(want)) or sat


# ------------------------------------------------------------------ golden fixtures: reductions (seq order)
@pytest.mark.parametrize("fmt", [(5, 10), (8, 7), (4, 3)])
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_softmax_seq_matches_reference_fixture(oracle, fmt, dim):
    g = golden("reductions_seq.npz")
    e, m = fmt
    x, gr = g["sm_x"], g["sm_g"]
    y = oracle.softmax_forward(x, dim, m, e, m, e, m, e, True, False, "seq")
    want = g[f"sm_fwd_dim{dim}_e{e}m{m}"].view(np.float32)
    assert same_bits(y, want), mismatch_report(y, want)
    y2 = oracle.softmax_lse_forward(x, dim, m, e, m, e, True, False, "seq")
    want2 = g[f"sm_lse_dim{dim}_e{e}m{m}"].view(np.float32)
    assert same_bits(y2, want2), mismatch_report(y2, want2)
    d = oracle.softmax_backward(want, gr, dim, m, e, m, e, True, False, "seq")
    want3 = g[f"sm_bwd_dim{dim}_e{e}m{m}"].view(np.float32)
    assert same_bits(d, want3), mismatch_report(d, want3)


@pytest.mark.parametrize("fmt", [(5, 10), (8, 7), (8, 23)])
def test_layernorm_seq_matches_reference_fixture(oracle, fmt):
    g = golden("reductions_seq.npz")
    e, m = fmt
    x, gr, w, b = g["ln_x"], g["ln_g"], g["ln_w"], g["ln_b"]
    y, mean, rstd = oracle.layernorm_forward(x, w, b, 1e-5, [-1], m, e, m, e, m, e, m, e, True, False, "seq")
    for got, name in ((y, "y"), (mean, "mean"), (rstd, "rstd")):
        want = g[f"ln_fwd_{name}_e{e}m{m}"].view(np.float32)
        assert same_bits(got.ravel(), want.ravel()), name + ": " + mismatch_report(got, want)
    gi, gg, gb = oracle.layernorm_backward(x, gr, w, mean, rstd, [-1], m, e, m, e, m, e, True, False, "seq")
    for got, name in ((gi, "gi"), (gg, "gg"), (gb, "gb")):
        want = g[f"ln_bwd_{name}_e{e}m{m}"].view(np.float32)
        assert same_bits(got.ravel(), want.ravel()), name + ": " + mismatch_report(got, want)


# ------------------------------------------------------------------ the reference's known-answer vectors
def test_kat_float_quantize(oracle):
    """Values asserted by the reference's tests/test_float_quantize.py:7-41 and test_bfloat16_nearest.py:6-21."""
    q = oracle.float_quantize
    assert q([3.0], 23, 8, "nearest")[0] == 3.0
    assert q([1097.0], 23, 2, "nearest", True, False)[0] == float("inf")
    assert q([1097.0], 23, 2, "nearest", True, True)[0] == np.float32(3.999999761581421)
    assert q([8.0], 23, 3, "nearest", False, False)[0] == 8.0
    assert q([3.1516], 1, 8, "nearest", True, False)[0] == 3.0
    out = q([20.0625, 20.06251, float("inf"), -float("inf")], 7, 8, "nearest", True, False)
    assert list(out) == [20.0, 20.125, float("inf"), -float("inf")]
    # IEEE-like e4m3 (the top exponent code reserved for infinity and NaN) tops out at 240 when saturating
    assert list(q([1.3, 1e-6, 70000.0, -0.3], 3, 4, "nearest", True, True)) == [1.25, 0.0, 240.0, -0.3125]


def test_kat_binary8_signed_nearest(oracle):
    """Vectors of the reference's tests/test_binary8_signed_nearest.py:38-137 (P=1,2,3)."""
    def q(vals, P, pol="saturate_maxfloat", sub=True):
        return list(oracle.binary8_quantize(np.array(vals, dtype=np.float32), P, "nearest", pol, True, sub))

    inf = float("inf")
    f = np.float32
    assert q([1.5, 4.0e-13, 134210000.0, -9.0e-07], 1) == [f(2.0), f(4.5474735e-13), f(134217728.0), f(-9.5367432e-07)]
    p1 = [(0x20800000, 0x20800000), (0x20000000, 0), (0x20000001, 0x20800000), (0x5F000000, 0x5F000000),
          (0x5F800000, 0x5F000000), (0x1F800000, 0)]
    for a, w in p1:
        assert q([b2f(a)], 1) == [f(b2f(w))]
    assert q([inf, -inf], 1) == [f(b2f(0x5F000000)), f(b2f(0xDF000000))]
    assert q([1.5, 2.90e-08, -1.1402e-05, -25000824.0], 2) == [f(1.5), f(2.9802322e-08), f(-1.1444092e-05), f(-25165824.0)]
    p2 = [(0x30000000, 0x30000000), (0x2F800000, 0x2F800000), (0x2F000000, 0), (0x2F000001, 0x2F800000),
          (0x4F000000, 0x4F000000), (0x5F800000, 0x4F000000), (0x2E800000, 0)]
    for a, w in p2:
        assert q([b2f(a)], 2) == [f(b2f(w))]
    for pol, mx, over in (("saturate_maxfloat", 0x47400000, 0x47400000), ("saturate_maxfloat2", 0x47600000, 0x47600000),
                          ("saturate_infty", 0x47400000, 0x7F800000)):
        assert q([1.5, 13.0, 13.000001, -13.0], 3, pol) == [1.5, 12.0, 14.0, -12.0]
        assert q([b2f(0x38000000)], 3, pol) == [f(b2f(0x38000000))]
        assert q([b2f(0x37000000)], 3, pol) == [f(b2f(0x37000000))]
        assert q([b2f(0x36800000)], 3, pol) == [0.0]
        assert q([b2f(0x36800001)], 3, pol) == [f(b2f(0x37000000))]
        assert q([b2f(mx)], 3, pol) == [f(b2f(mx))]
        nxt = mx + 0x00200000 if pol != "saturate_maxfloat2" else mx + 0x00100000
        assert q([b2f(nxt)], 3, pol) == [f(b2f(over))]
        assert q([b2f(0x36000000)], 3, pol) == [0.0]
        want_inf = inf if pol == "saturate_infty" else f(b2f(mx))
        assert q([inf, -inf], 3, pol) == [want_inf, -want_inf]
    # no-subnormal arm (test_no_subnormal_case)
    for a, w in ((1.9e-5, 1.907348633e-5), (2.3e-5, 2.288818359e-5), (2.67e-5, 2.670288086e-5), (9.7e-6, 1.907348633e-5),
                 (9.5e-6, 0.0), (1.5258789e-5, 1.907348633e-5), (2.288818359375e-5, 2.288818359e-5)):
        assert q([a], 3, "saturate_maxfloat", False) == [f(w)]


def test_binary8_truncate_kat(oracle):
    """tests/test_binary8_truncate.py:6-40 of the reference: truncation never rounds up in magnitude."""
    x = np.array([1.9999, -1.9999, 13.9, -13.9, 0.3], dtype=np.float32)
    out = oracle.binary8_quantize(x, 4, "truncate", "saturate_maxfloat", True, True)
    assert np.all(np.abs(out) <= np.abs(x))
    assert list(out) == [1.875, -1.875, 13.0, -13.0, 0.28125]


# ------------------------------------------------------------------ live reference, larger sweeps
FORMATS = [(5, 2), (4, 3), (5, 10), (8, 7), (3, 4), (6, 1), (8, 0), (2, 0), (7, 22), (8, 22), (4, 23)]


@pytest.mark.parametrize("fmt", FORMATS)
def test_float_nearest_vs_live_reference(oracle, ref_cpu, fmt):
    e, m = fmt
    rng = np.random.default_rng(e * 100 + m)
    bits = rng.integers(0, 2**32, size=1 << 20, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    xt = torch.from_numpy(x.copy())
    for sub in (False, True):
        for sat in (False, True):
            want = ref_cpu.float_quantize_nearest(xt, m, e, sub, sat).numpy()
            got = oracle.float_quantize(x, m, e, "nearest", sub, sat)
            assert same_bits(got, want), f"sub={sub} sat={sat}: " + mismatch_report(got, want)


def test_float_nearest_dense_sweep_vs_live_reference(oracle, ref_cpu):
    """Every 61st fp32 pattern (70 M values) through the headline format e5m2 and through e4m3."""
    for (e, m, sub, sat) in ((5, 2, True, False), (4, 3, True, True)):
        for start in range(0, 2**32, 2**28):
            bits = np.arange(start, start + 2**28, 61, dtype=np.uint64).astype(np.uint32)
            x = bits.view(np.float32)
            want = ref_cpu.float_quantize_nearest(torch.from_numpy(x.copy()), m, e, sub, sat).numpy()
            got = oracle.float_quantize(x, m, e, "nearest", sub, sat)
            assert same_bits(got, want), mismatch_report(got, want)


@pytest.mark.parametrize("P", range(1, 8))
def test_binary8_vs_live_reference(oracle, ref_cpu, P):
    rng = np.random.default_rng(P)
    bits = rng.integers(0, 2**32, size=1 << 18, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    xt = torch.from_numpy(x.copy())
    pol = [ref_cpu.OverflowPolicy.SATURATE_INFTY, ref_cpu.OverflowPolicy.SATURATE_MAXFLOAT,
           ref_cpu.OverflowPolicy.SATURATE_MAXFLOAT2]
    for sg in (False, True):
        for po in range(3):
            for sub in (False, True):
                want = ref_cpu.binary8_quantize_nearest(xt, P, sg, pol[po], sub).numpy()
                got = oracle.binary8_quantize(x, P, "nearest", POL[po], sg, sub)
                assert same_bits(got, want), f"nearest sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)
                want = ref_cpu.binary8_quantize_truncate(xt, P, sg, pol[po], sub).numpy()
                got = oracle.binary8_quantize(x, P, "truncate", POL[po], sg, sub)
                assert same_bits(got, want), f"truncate sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)
                prng = 23 - (P - 1)
                torch.manual_seed(5)
                rnd = torch.randint_like(xt, 2147483647, dtype=torch.int32)
                torch.manual_seed(5)
                want = ref_cpu.binary8_quantize_stochastic(xt, P, prng, sg, pol[po], sub).numpy()
                got = oracle.binary8_quantize(x, P, "stochastic", POL[po], sg, sub, rand=rnd.numpy(), prng_bits=prng)
                assert same_bits(got, want), f"stochastic sg={sg} po={po} sub={sub}: " + mismatch_report(got, want)


def test_superfp_vs_live_reference(oracle, ref_cpu):
    rng = np.random.default_rng(11)
    bits = rng.integers(0, 2**32, size=1 << 19, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    xt = torch.from_numpy(x.copy())
    for (e, m, bl, bu) in [(4, 3, 1, 1), (4, 3, 2, 1), (5, 2, 1, 2), (3, 4, 1, 1), (6, 1, 2, 2), (4, 2, 3, 1), (7, 5, 1, 1)]:
        for sat in (False, True):
            want = ref_cpu.superfp_quantize_nearest(xt, m, e, bl, bu, sat).numpy()
            got = oracle.superfp_quantize(x, m, e, bl, bu, sat)
            assert same_bits(got, want), f"e{e}m{m} l{bl} u{bu} sat={sat}: " + mismatch_report(got, want)


def test_mm_config1_vs_live_reference(oracle, ref_cpu):
    """benchmark config 1 at reduced M,N (full K=256): e5m2 multiply and add, nearest, sequential K."""
    torch.manual_seed(0)
    a, b = torch.randn(48, 256), torch.randn(256, 40)
    c = torch.zeros(48, 40)
    ref_cpu.float_quantize_nearest_mm(a, b, c, 48, 40, 256, 2, 5, 2, 5, True, False, False)
    got = oracle.mm(a.numpy(), b.numpy(), 2, 5, 2, 5, True, False, False, "seq")
    assert same_bits(got, c.numpy()), mismatch_report(got, c.numpy())


def test_tile8_equals_composition_of_pinned_casts(oracle):
    """The tile8 order is the reference CUDA kernel's (quant_cuda/mm_kernel.h:34-70); restate it once more
    here from the elementwise casts only, independently of the C loop."""
    rng = np.random.default_rng(3)
    M, K, N = 5, 24, 6
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    qa = lambda v: oracle.float_quantize(v, 2, 5, "nearest", True, False)
    qm = lambda v: oracle.float_quantize(v, 3, 4, "nearest", True, False)
    outer = np.zeros((M, N), np.float32)
    for t in range(K // 8 + 1):
        inner = np.zeros((M, N), np.float32)
        for k in range(8 * t, 8 * t + 8):
            col = a[:, k:k + 1] if k < K else np.zeros((M, 1), np.float32)
            row = b[k:k + 1, :] if k < K else np.zeros((1, N), np.float32)
            inner = qa(inner + qm(col * row))
        outer = qa(outer + inner)
    got = oracle.mm(a, b, 2, 5, 3, 4, True, False, False, "tile8")
    assert same_bits(got, outer), mismatch_report(got, outer)
    seq = oracle.mm(a, b, 2, 5, 3, 4, True, False, False, "seq")
    assert not same_bits(seq, outer)


# ------------------------------------------------------------------ superfp / binary8 arithmetic vs the live reference
def test_superfp_mm_vs_live_reference(oracle, ref_cpu):
    torch.manual_seed(21)
    a, b = torch.randn(19, 45), torch.randn(45, 13)
    for (ma, ea, la, ua, mm_, em, lm, um) in [(3, 4, 1, 1, 2, 4, 2, 1), (2, 5, 1, 2, 2, 5, 1, 2), (4, 3, 1, 1, 3, 4, 1, 1)]:
        for sat in (False, True):
            c = torch.zeros(19, 13)
            ref_cpu.superfp_quantize_nearest_mm(a, b, c, 19, 13, 45, ma, ea, mm_, em, la, ua, lm, um, sat)
            got = oracle.mm_fmt(a.numpy(), b.numpy(), oracle.fmt_superfp(ma, ea, la, ua, sat), oracle.fmt_superfp(mm_, em, lm, um, sat), False, "seq")
            assert same_bits(got, c.numpy()), mismatch_report(got, c.numpy())
            c = torch.zeros(19, 13)
            ref_cpu.superfp_quantize_nearest_mm_fma(a, b, c, 19, 13, 45, ma, ea, la, ua, sat)
            f = oracle.fmt_superfp(ma, ea, la, ua, sat)
            got = oracle.mm_fmt(a.numpy(), b.numpy(), f, f, True, "seq")
            assert same_bits(got, c.numpy()), mismatch_report(got, c.numpy())
    a3, b3 = torch.randn(3, 8, 20), torch.randn(3, 20, 6)
    c3 = torch.zeros(3, 8, 6)
    ref_cpu.superfp_quantize_nearest_bmm(a3, b3, c3, 8, 6, 20, 3, 4, 2, 4, 1, 1, 2, 1, False)
    got = oracle.mm_fmt(a3.numpy(), b3.numpy(), oracle.fmt_superfp(3, 4, 1, 1), oracle.fmt_superfp(2, 4, 2, 1), False, "seq")
    assert same_bits(got, c3.numpy())


def test_superfp_and_binary8_reductions_vs_live_reference(oracle, ref_cpu):
    torch.manual_seed(22)
    x = torch.randn(3, 33, 4) * 2
    g = torch.randn(3, 33, 4)
    pol = [ref_cpu.OverflowPolicy.SATURATE_INFTY, ref_cpu.OverflowPolicy.SATURATE_MAXFLOAT, ref_cpu.OverflowPolicy.SATURATE_MAXFLOAT2]
    sf = oracle.fmt_superfp(3, 5, 2, 1, False)
    for dim in (0, 1, 2):
        y = torch.zeros_like(x)
        ref_cpu.superfp_quantize_nearest_softmax_forward(x, y, dim, 3, 5, 2, 1, 3, 5, 2, 1, 3, 5, 2, 1, False)
        assert same_bits(oracle.softmax_forward_fmt(x.numpy(), dim, sf, sf, sf, "seq"), y.numpy())
        y2 = torch.zeros_like(x)
        ref_cpu.superfp_quantize_nearest_softmax_lse_forward(x, y2, dim, 3, 5, 2, 1, 3, 5, 2, 1, False)
        assert same_bits(oracle.softmax_lse_forward_fmt(x.numpy(), dim, sf, sf, "seq"), y2.numpy())
        d = torch.zeros_like(x)
        ref_cpu.superfp_quantize_nearest_softmax_backward(y, g, d, dim, 3, 5, 2, 1, 3, 5, 2, 1, False)
        assert same_bits(oracle.softmax_backward_fmt(y.numpy(), g.numpy(), dim, sf, sf, "seq"), d.numpy())
        for (P, sg, po) in [(4, True, 1), (3, True, 0), (5, False, 2)]:
            bf = oracle.fmt_binary8(P, sg, po, True)
            yb = torch.zeros_like(x)
            ref_cpu.binary8_quantize_nearest_softmax_forward(x, yb, dim, P, pol[po], sg, P, pol[po], True, P, pol[po], sg, True)
            bo = oracle.fmt_binary8(P, True, po, True)    # the offset x - max is negative: signed format
            assert same_bits(oracle.softmax_forward_fmt(x.numpy(), dim, bf, bo, bf, "seq"), yb.numpy())
            db = torch.zeros_like(x)
            ref_cpu.binary8_quantize_nearest_softmax_backward(yb, g, db, dim, P, pol[po], True, P, pol[po], True, True)
            bs = oracle.fmt_binary8(P, True, po, True)
            assert same_bits(oracle.softmax_backward_fmt(yb.numpy(), g.numpy(), dim, bs, bs, "seq"), db.numpy())
    xl = torch.randn(4, 5, 24) + 0.3
    gl = torch.randn(4, 5, 24)
    w, b = torch.randn(24), torch.randn(24)
    for fmt, call_f, call_b, args in (
            (oracle.fmt_superfp(4, 5, 1, 1, False), ref_cpu.superfp_quantize_layernorm_forward, ref_cpu.superfp_quantize_layernorm_backward,
             lambda n: sum(([4, 5, 1, 1] for _ in range(n)), []) + [False]),
            (oracle.fmt_binary8(5, True, 1, True), ref_cpu.binary8_quantize_layernorm_forward, ref_cpu.binary8_quantize_layernorm_backward,
             lambda n: sum(([5, pol[1], True] for _ in range(n)), []) + [True])):
        y = torch.zeros_like(xl); mean = torch.zeros(4, 5); rstd = torch.zeros(4, 5)
        call_f(xl, w, b, y, mean, rstd, 1e-5, [-1], *args(4))
        oy, om, orr = oracle.layernorm_forward_fmt(xl.numpy(), w.numpy(), b.numpy(), 1e-5, [-1], fmt, fmt, fmt, fmt, "seq")
        assert same_bits(oy, y.numpy()) and same_bits(om, mean.numpy().ravel()) and same_bits(orr, rstd.numpy().ravel())
        gi = torch.zeros_like(xl); gg = torch.zeros(24); gb = torch.zeros(24)
        call_b(xl, gl, w, b, mean, rstd, gi, gg, gb, [-1], *args(3))
        ogi, ogg, ogb = oracle.layernorm_backward_fmt(xl.numpy(), gl.numpy(), w.numpy(), om, orr, [-1], fmt, fmt, fmt, "seq")
        assert same_bits(ogi, gi.numpy()) and same_bits(ogg, gg.numpy()) and same_bits(ogb, gb.numpy())
