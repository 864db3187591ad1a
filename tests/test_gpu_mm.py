"""GPU parity of the per-MAC rounded GEMM: CUDA kernels (through the C ABI) vs the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

from conftest import golden, mismatch_report, same_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from mptorch_b200 import backend

    return backend


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def gpu_mm(be, a, b, fadd, fmul, sub=True, sat=False, fma=False, order="cuda", comp=False):
    ad, bd = dev(a), dev(b)
    batched = ad.dim() == 3
    M, K = ad.shape[-2:]
    N = bd.shape[-1]
    c = torch.full((ad.shape[0], M, N) if batched else (M, N), float("nan"), device="cuda")
    if fma:
        fn = be.float_quantize_nearest_bmm_fma if batched else be.float_quantize_nearest_mm_fma
        fn(ad, bd, c, M, N, K, fadd[1], fadd[0], sub, sat, comp, order=order)
    else:
        fn = be.float_quantize_nearest_bmm if batched else be.float_quantize_nearest_mm
        fn(ad, bd, c, M, N, K, fadd[1], fadd[0], fmul[1], fmul[0], sub, sat, comp, order=order)
    return c.cpu().numpy()


def cpu_mm(oracle, a, b, fadd, fmul, sub=True, sat=False, fma=False, order="cuda", comp=False):
    return oracle.mm(a, b, fadd[1], fadd[0], fmul[1], fmul[0], sub, sat, fma, "tile8" if order == "cuda" else "seq", comp)


# (add, mul) pairs; (4,3)/(5,10) and (5,2)/(8,7) have a multiply format finer than the add format
FORMATS = [((5, 2), (5, 2)), ((5, 10), (4, 3)), ((8, 7), (5, 2)), ((4, 3), (4, 3)), ((8, 23), (5, 2)), ((6, 21), (3, 0)),
           ((4, 3), (5, 10)), ((5, 2), (8, 7))]
SHAPES = [(78, 101, 145), (64, 256, 48), (9, 32, 12), (1, 1, 1), (130, 8, 70), (17, 40, 4), (128, 64, 64), (5, 7, 3)]


def test_config1_sequential_256(be, oracle):
    """benchmark config 1: 256x256x256, N(0,1), e5m2 multiply and add, nearest, sequential K."""
    rng = np.random.default_rng(2025)
    a = rng.standard_normal((256, 256)).astype(np.float32)
    b = rng.standard_normal((256, 256)).astype(np.float32)
    got = gpu_mm(be, a, b, (5, 2), (5, 2), order="seq")
    want = cpu_mm(oracle, a, b, (5, 2), (5, 2), order="seq")
    assert same_bits(got, want), mismatch_report(got, want)
    got = gpu_mm(be, a, b, (5, 2), (5, 2), order="cuda")
    want = cpu_mm(oracle, a, b, (5, 2), (5, 2), order="cuda")
    assert same_bits(got, want), mismatch_report(got, want)


def test_seq_matches_reference_fixture(be):
    """Against outputs of the reference's own CPU extension (tests/golden/mm_seq.npz)."""
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
            got = gpu_mm(be, a, b, (int(ea), int(ma)), (int(em), int(mm_)), sat=bool(int(p[6][3:])), order="seq")
        else:
            ea, ma = p[2][1:].split("m")
            got = gpu_mm(be, a, b, (int(ea), int(ma)), None, fma=True, order="seq")
        assert same_bits(got, want), key + ": " + mismatch_report(got, want)
        n += 1
    assert n >= 30
    got = gpu_mm(be, g["bmm_a"], g["bmm_b"], (5, 2), (5, 2), order="seq")
    assert same_bits(got, g["bmm_e5m2"].view(np.float32))
    for sat in (0, 1):
        got = gpu_mm(be, g["big_a"], g["big_b"], (5, 2), (5, 2), sat=bool(sat), order="seq")
        want = g[f"big_mm_e5m2_sat{sat}"].view(np.float32)
        assert same_bits(got, want), mismatch_report(got, want)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("order", ["cuda", "seq"])
def test_shapes_formats(be, oracle, shape, order):
    M, K, N = shape
    rng = np.random.default_rng(M * 1000 + K * 10 + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    for fadd, fmul in FORMATS:
        for fma in (False, True):
            got = gpu_mm(be, a, b, fadd, fmul, fma=fma, order=order)
            want = cpu_mm(oracle, a, b, fadd, fmul, fma=fma, order=order)
            assert same_bits(got, want), f"{fadd}/{fmul} fma={fma}: " + mismatch_report(got, want)


@pytest.mark.parametrize("order", ["cuda", "seq"])
def test_value_ranges_that_leave_the_fast_path(be, oracle, order):
    """Overflow to inf, saturation, tiny values, specials: the exact path must take over seamlessly."""
    rng = np.random.default_rng(17)
    M, K, N = 40, 72, 36
    base_a = rng.standard_normal((M, K)).astype(np.float32)
    base_b = rng.standard_normal((K, N)).astype(np.float32)
    cases = {
        "huge": (base_a * 300, base_b * 300),
        "mid": (base_a * 20, base_b * 20),
        "tiny": (base_a * 1e-4, base_b * 1e-3),
        "subnormal_sums": (base_a * 3e-3, base_b * 3e-3),
        "denormal_products": (base_a * 1e-20, base_b * 1e-20),
    }
    sp_a, sp_b = base_a.copy(), base_b.copy()
    sp_a[3, 5] = np.inf; sp_a[7, 1] = np.nan; sp_b[2, 9] = -np.inf; sp_a[11, :] = 0.0; sp_b[:, 4] = -0.0
    cases["specials"] = (sp_a, sp_b)
    one_big = base_a.copy(); one_big[0, 0] = 3e4
    cases["one_big"] = (one_big, base_b)
    for name, (a, b) in cases.items():
        for fadd, fmul in [((5, 2), (5, 2)), ((5, 10), (4, 3)), ((8, 7), (5, 2)), ((8, 7), (8, 7)), ((4, 3), (5, 10))]:
            for sat in (False, True):
                for fma in (False, True):
                    got = gpu_mm(be, a, b, fadd, fmul, sat=sat, fma=fma, order=order)
                    want = cpu_mm(oracle, a, b, fadd, fmul, sat=sat, fma=fma, order=order)
                    assert same_bits(got, want), f"{name} {fadd}/{fmul} sat={sat} fma={fma}: " + mismatch_report(got, want)


def test_without_subnormals(be, oracle):
    rng = np.random.default_rng(5)
    a = (rng.standard_normal((33, 50)) * 0.05).astype(np.float32)
    b = (rng.standard_normal((50, 20)) * 0.05).astype(np.float32)
    for order in ("cuda", "seq"):
        got = gpu_mm(be, a, b, (5, 2), (4, 3), sub=False, order=order)
        want = cpu_mm(oracle, a, b, (5, 2), (4, 3), sub=False, order=order)
        assert same_bits(got, want), mismatch_report(got, want)


def test_batched(be, oracle):
    rng = np.random.default_rng(6)
    a = rng.standard_normal((5, 70, 33)).astype(np.float32)
    b = rng.standard_normal((5, 33, 20)).astype(np.float32)
    for order in ("cuda", "seq"):
        for fma in (False, True):
            got = gpu_mm(be, a, b, (5, 10), (4, 3), fma=fma, order=order)
            want = cpu_mm(oracle, a, b, (5, 10), (4, 3), fma=fma, order=order)
            assert same_bits(got, want), mismatch_report(got, want)


def test_batched_mixed_ranges(be, oracle):
    """The fast-path decision is made per batch entry: one entry with huge / special values next to ordinary ones."""
    rng = np.random.default_rng(61)
    a = rng.standard_normal((4, 40, 48)).astype(np.float32)
    b = rng.standard_normal((4, 48, 36)).astype(np.float32)
    a[1] *= 500.0
    b[1] *= 500.0
    a[2, 3, 4] = np.inf
    b[3, 0, 0] = np.nan
    for order in ("cuda", "seq"):
        for fma in (False, True):
            got = gpu_mm(be, a, b, (5, 2), (5, 2), fma=fma, order=order)
            want = cpu_mm(oracle, a, b, (5, 2), (5, 2), fma=fma, order=order)
            assert same_bits(got, want), f"{order} fma={fma}: " + mismatch_report(got, want)


def test_attention_shapes(be, oracle):
    """benchmark config 5 attention GEMM shapes at reduced batch: [B,1024,64]x[B,64,1024] rows sampled."""
    rng = np.random.default_rng(8)
    a = rng.standard_normal((2, 96, 64)).astype(np.float32)
    b = rng.standard_normal((2, 64, 1024)).astype(np.float32)
    got = gpu_mm(be, a, b, (5, 10), (4, 3))
    want = cpu_mm(oracle, a, b, (5, 10), (4, 3))
    assert same_bits(got, want), mismatch_report(got, want)


def test_compensated(be, oracle):
    rng = np.random.default_rng(9)
    a = rng.standard_normal((30, 45)).astype(np.float32)
    b = rng.standard_normal((45, 22)).astype(np.float32)
    for fma in (False, True):
        got = gpu_mm(be, a, b, (5, 10), (4, 3), fma=fma, comp=True)
        want = cpu_mm(oracle, a, b, (5, 10), (4, 3), fma=fma, comp=True)
        assert same_bits(got, want), f"fma={fma}: " + mismatch_report(got, want)


@pytest.mark.parametrize("fmts", FORMATS)
@pytest.mark.parametrize("fma", [False, True])
def test_compensated_range_checked_path(be, oracle, fmts, fma):
    """Kahan GEMM on operands that stay in range (packed FP-pipe roundings), that overflow part of the way (the
    per-group fallback to the whole-domain casters), and that hold zeros, negative zeros and tiny values."""
    fadd, fmul = fmts
    rng = np.random.default_rng(90)
    for (M, K, N), scale in [((70, 203, 52), 1.0), ((33, 64, 40), 40.0), ((16, 96, 24), 1e-3), ((130, 40, 70), 6.0)]:
        a = (rng.standard_normal((M, K)) * scale).astype(np.float32)
        b = rng.standard_normal((K, N)).astype(np.float32)
        a[rng.random((M, K)) < 0.1] = 0.0
        b[rng.random((K, N)) < 0.1] = -0.0
        for sat in (False, True):
            got = gpu_mm(be, a, b, fadd, fmul, sat=sat, fma=fma, comp=True)
            want = cpu_mm(oracle, a, b, fadd, fmul, sat=sat, fma=fma, comp=True)
            assert same_bits(got, want), f"{fmts} fma={fma} {(M, K, N)} x{scale} sat={sat}: " + mismatch_report(got, want)
    a = rng.standard_normal((3, 48, 72)).astype(np.float32)
    b = rng.standard_normal((3, 72, 36)).astype(np.float32)
    a[1] *= 300.0
    b[2, 5, 5] = np.inf
    got = gpu_mm(be, a, b, fadd, fmul, fma=fma, comp=True)
    want = cpu_mm(oracle, a, b, fadd, fmul, fma=fma, comp=True)
    assert same_bits(got, want), f"batched {fmts} fma={fma}: " + mismatch_report(got, want)


def test_fma_cancellation_into_fp32_denormals(be, oracle):
    """A fused multiply-add can cancel to a nonzero fp32 denormal (exact product minus an equal-sized sum), which an
    8-bit-exponent format rounds in its own way: operands around 2^-48 must not take the FP-pipe rounding."""
    a = np.zeros((8, 8), np.float32)
    b = np.zeros((8, 8), np.float32)
    a[:, 0] = -np.float32(2.0 ** -48)
    b[0, :] = np.float32(2.0 ** -48)
    a[:, 1] = np.float32((1 + 2.0 ** -23) * 2.0 ** -48)
    b[1, :] = np.float32((1 - 2.0 ** -23) * 2.0 ** -48)
    a[:, 2:] = np.float32(2.0 ** -47)
    b[2:, :] = np.float32(2.0 ** -49)
    for order in ("seq", "cuda"):
        for fadd in ((8, 7), (8, 10)):
            got = gpu_mm(be, a, b, fadd, fadd, fma=True, order=order)
            want = cpu_mm(oracle, a, b, fadd, fadd, fma=True, order=order)
            assert same_bits(got, want), f"{order} {fadd}: " + mismatch_report(got, want)


@pytest.mark.parametrize("fma", [False, True])
def test_stochastic_range_checked_path(be, oracle, fma):
    """Stochastic GEMM: in-range operands (straight-line rounding), overflowing ones (fallback), saturation, zeros."""
    rng = np.random.default_rng(91)
    seed = 0x1234ABCD5678
    for (fadd, rb_a), (fmul, rb_m) in [(((5, 10), 13), ((4, 3), 20)), (((5, 2), 21), ((5, 2), 8)), (((8, 7), 16), ((8, 7), 16))]:
        for (M, K, N), scale in [((40, 77, 36), 1.0), ((20, 64, 24), 200.0), ((12, 33, 20), 1e-4)]:
            a = (rng.standard_normal((M, K)) * scale).astype(np.float32)
            b = rng.standard_normal((K, N)).astype(np.float32)
            a[rng.random((M, K)) < 0.1] = 0.0
            for sat, sub in ((False, True), (True, True), (False, False), (True, False)):      # without subnormals too
                c = torch.full((M, N), float("nan"), device="cuda")
                if fma:
                    be.float_quantize_stochastic_mm_fma(dev(a), dev(b), c, M, N, K, fadd[1], fadd[0], rb_a, sub, sat, seed=seed)
                    want = oracle.mm_sr(a, b, fadd[1], fadd[0], rb_a, fadd[1], fadd[0], rb_a, sub, sat, True, seed)
                else:
                    be.float_quantize_stochastic_mm(dev(a), dev(b), c, M, N, K, fadd[1], fadd[0], rb_a, fmul[1], fmul[0], rb_m, sub, sat, seed=seed)
                    want = oracle.mm_sr(a, b, fadd[1], fadd[0], rb_a, fmul[1], fmul[0], rb_m, sub, sat, False, seed)
                got = c.cpu().numpy()
                assert same_bits(got, want), f"{fadd} {fmul} fma={fma} {(M, K, N)} x{scale} sat={sat} sub={sub}: " + mismatch_report(got, want)


def test_stochastic_matches_oracle_philox(be, oracle):
    rng = np.random.default_rng(10)
    a = rng.standard_normal((3, 20, 37)).astype(np.float32)
    b = rng.standard_normal((3, 37, 24)).astype(np.float32)
    seed = 0xDEADBEEF12345
    c = torch.zeros(3, 20, 24, device="cuda")
    be.float_quantize_stochastic_bmm(dev(a), dev(b), c, 20, 24, 37, 10, 5, 13, 3, 4, 20, True, False, seed=seed)
    want = oracle.mm_sr(a, b, 10, 5, 13, 3, 4, 20, True, False, False, seed)
    assert same_bits(c.cpu().numpy(), want), mismatch_report(c.cpu().numpy(), want)
    c2 = torch.zeros(20, 24, device="cuda")
    be.float_quantize_stochastic_mm_fma(dev(a[0]), dev(b[0]), c2, 20, 24, 37, 10, 5, 13, True, False, seed=seed)
    want = oracle.mm_sr(a[0], b[0], 10, 5, 13, 10, 5, 13, True, False, True, seed)
    assert same_bits(c2.cpu().numpy(), want), mismatch_report(c2.cpu().numpy(), want)


def test_stochastic_statistics(be):
    """SR accumulation is unbiased: the mean over many seeds approaches the fp32 product."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((16, 64)).astype(np.float32)
    b = rng.standard_normal((64, 16)).astype(np.float32)
    ad, bd = dev(a), dev(b)
    acc = torch.zeros(16, 16, device="cuda", dtype=torch.float64)
    reps = 200
    for s in range(reps):
        c = torch.zeros(16, 16, device="cuda")
        be.float_quantize_stochastic_mm(ad, bd, c, 16, 16, 64, 7, 8, 16, 7, 8, 16, True, False, seed=s)
        acc += c.double()
    exact = torch.from_numpy(a.astype(np.float64) @ b.astype(np.float64)).cuda()
    err = (acc / reps - exact).abs().max().item()
    assert err < 0.05, err


def test_empty_and_degenerate(be):
    c = torch.full((4, 6), 7.0, device="cuda")
    be.float_quantize_nearest_mm(torch.zeros(4, 0, device="cuda"), torch.zeros(0, 6, device="cuda"), c, 4, 6, 0, 2, 5, 2, 5, True, False, False)
    assert torch.equal(c, torch.zeros_like(c))
    c0 = torch.zeros(0, 6, device="cuda")
    be.float_quantize_nearest_mm(torch.zeros(0, 3, device="cuda"), torch.zeros(3, 6, device="cuda"), c0, 0, 6, 3, 2, 5, 2, 5, True, False, False)


def test_exact_path_without_workspace(oracle):
    """Calling the C ABI with no workspace still gives the same bits (exact casts only)."""
    from mptorch_b200 import _cabi

    rng = np.random.default_rng(12)
    a = rng.standard_normal((50, 64)).astype(np.float32)
    b = rng.standard_normal((64, 44)).astype(np.float32)
    ad, bd = dev(a), dev(b)
    c = torch.zeros(50, 44, device="cuda")
    _cabi.call("mpt_float_mm_nearest", _cabi.ptr(ad), _cabi.ptr(bd), _cabi.ptr(c), 1, 50, 44, 64, 2, 5, 2, 5, 1, 0, 0, 1,
               None, 0, _cabi.stream_ptr(c.device))
    want = oracle.mm(a, b, 2, 5, 2, 5, True, False, False, "tile8")
    assert same_bits(c.cpu().numpy(), want)


@pytest.mark.parametrize("fmts", [((5, 2), (5, 2)), ((5, 10), (4, 3)), ((8, 7), (5, 2))])
def test_full_size_row_samples_and_sharding(be, oracle, fmts):
    """benchmark config 4 at its largest size, 8192^3, for the headline format pair and both sweep pairs: sampled
    rows equal the oracle bit for bit (rows of C are independent), and a row-sharded run equals the
    single launch (the multi-GPU decomposition)."""
    fadd, fmul = fmts
    S = 8192
    g = torch.Generator(device="cuda").manual_seed(77)
    a = torch.randn(S, S, device="cuda", generator=g)
    b = torch.randn(S, S, device="cuda", generator=g)
    c = torch.empty(S, S, device="cuda")
    be.float_quantize_nearest_mm(a, b, c, S, S, S, fadd[1], fadd[0], fmul[1], fmul[0], True, False, False, order="cuda")
    rows = [0, 1, S // 2 + 3, S - 1]
    want = oracle.mm(a[rows].cpu().numpy(), b.cpu().numpy(), fadd[1], fadd[0], fmul[1], fmul[0], True, False, False, "tile8")
    got = c[rows].cpu().numpy()
    assert same_bits(got, want), mismatch_report(got, want)
    # row shard [S/4, S/2) computed alone
    lo, hi = S // 4, S // 2
    cs = torch.empty(hi - lo, S, device="cuda")
    be.float_quantize_nearest_mm(a[lo:hi].contiguous(), b, cs, hi - lo, S, S, fadd[1], fadd[0], fmul[1], fmul[0], True, False, False, order="cuda")
    assert torch.equal(cs.view(torch.int32), c[lo:hi].view(torch.int32))
    if fmts == ((5, 2), (5, 2)):
        be.float_quantize_nearest_mm(a, b, c, S, S, S, fadd[1], fadd[0], fmul[1], fmul[0], True, False, False, order="seq")
        want = oracle.mm(a[rows[:2]].cpu().numpy(), b.cpu().numpy(), fadd[1], fadd[0], fmul[1], fmul[0], True, False, False, "seq")
        assert same_bits(c[rows[:2]].cpu().numpy(), want)


def test_short_wide_products_equal_the_backend_call(be):
    """float_mm / float_bmm compute products with at most 64 rows and many columns as the transposed problem (full CTA
    tiles); the bits must equal the direct backend call, for both accumulation orders, plain, fused and compensated."""
    import mptorch_b200.quant as q

    g = torch.Generator(device="cuda").manual_seed(31)
    a = torch.randn(3, 64, 200, device="cuda", generator=g)
    b = torch.randn(3, 200, 320, device="cuda", generator=g)
    for order in ("cuda", "seq"):
        with q.orders(accum=order):
            for fma in (False, True):
                for comp in (False, True):
                    got = q.float_bmm(a, b, man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest", fma=fma, subnormals=True,
                                      saturate=False, compensated=comp)
                    want = torch.empty(3, 64, 320, device="cuda")
                    if fma:
                        be.float_quantize_nearest_bmm_fma(a, b, want, 64, 320, 200, 10, 5, True, False, comp, order=order)
                    else:
                        be.float_quantize_nearest_bmm(a, b, want, 64, 320, 200, 10, 5, 3, 4, True, False, comp, order=order)
                    assert got.shape == want.shape and torch.equal(got.contiguous().view(torch.int32), want.view(torch.int32)), (order, fma, comp)
    got = q.float_mm(a[0, :17].contiguous(), b[0], man_add=2, exp_add=5, man_mul=2, exp_mul=5, rounding="nearest", fma=False, subnormals=True, saturate=False)
    want = torch.empty(17, 320, device="cuda")
    be.float_quantize_nearest_mm(a[0, :17].contiguous(), b[0], want, 17, 320, 200, 2, 5, 2, 5, True, False, False)
    assert torch.equal(got.contiguous().view(torch.int32), want.view(torch.int32))


def test_streamed_host_operands_equal_one_call():
    """float_mm_streamed (host operands, row blocks overlapped with the copies) gives the bits of one float_mm call."""
    import mptorch_b200.quant as q

    torch.manual_seed(3)
    a = torch.randn(1000, 384).pin_memory()
    b = torch.randn(384, 520).pin_memory()
    want = q.float_mm(a.cuda(), b.cuda(), man_add=2, exp_add=5, man_mul=2, exp_mul=5, rounding="nearest", fma=False,
                      subnormals=True, saturate=False).cpu()
    for block in (128, 333, 1000, 4096):
        got = q.float_mm_streamed(a, b, block_rows=block, man_add=2, exp_add=5, man_mul=2, exp_mul=5, rounding="nearest", fma=False,
                                  subnormals=True, saturate=False)
        assert got.is_pinned() and torch.equal(got.view(torch.int32), want.view(torch.int32)), block
    out = torch.empty(1000, 520)                       # pageable output and inputs still work
    got = q.float_mm_streamed(a.clone(), b.clone(), out=out, block_rows=256, man_add=10, exp_add=5, man_mul=3, exp_mul=4,
                              rounding="nearest", fma=True, subnormals=True, saturate=False)
    want = q.float_mm(a.cuda(), b.cuda(), man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest", fma=True,
                      subnormals=True, saturate=False).cpu()
    assert got is out and torch.equal(got.view(torch.int32), want.view(torch.int32))
    with pytest.raises(RuntimeError):
        q.float_mm_streamed(a.cuda(), b)


@pytest.mark.parametrize("order", ["cuda", "seq"])
@pytest.mark.parametrize("fma", [False, True])
def test_product_in_k_pieces_equals_one_call(order, fma):
    """mpt_float_mm_nearest_piece: pieces along K that continue the running sums held in C leave the bits of the single
    call, for both orders, fused or not, with a ragged last piece, a piece shorter than a K slab, sums that pass
    through both signs of zero, overflow and NaN, and a product whose range check fails (exact path)."""
    import mptorch_b200.backend as be
    import mptorch_b200.quant as q

    g = torch.Generator(device="cuda").manual_seed(17)
    M, K, N = 200, 701, 136
    a = torch.randn(M, K, device="cuda", generator=g)
    b = torch.randn(K, N, device="cuda", generator=g)
    a[3] = 0.0
    a[4] = -a[4].abs() * 1e-12            # products below the smallest subnormal
    a[5, ::2] = 300.0                     # sums that overflow e5m2's range: the exact path and infinities
    a[6, 100] = float("nan")
    a[7, :64] = 0.0
    b[:, 9] = -0.0
    fmt = dict(man_add=2, exp_add=5, man_mul=2, exp_mul=5)
    with be.orders(accum=order):
        want = q.float_mm(a, b, rounding="nearest", fma=fma, subnormals=True, saturate=False, **fmt)
        for cuts in ([0, 8, 16, 48, 400, 701], [0, 696, 701], [0, 256, 701], [0, 701]):
            c = torch.full((M, N), float("nan"), device="cuda")
            for i, (k0, k1) in enumerate(zip(cuts[:-1], cuts[1:])):
                flags = (be.MM_PIECE_FROM_C if i else 0) | (be.MM_PIECE_MORE if k1 < K else 0)
                be.float_mm_nearest_piece(a[:, k0:k1].contiguous(), b[k0:k1].contiguous(), c, 2, 5, 2, 5, True, False, fma, flags)
            same = (c.view(torch.int32) == want.view(torch.int32)) | (c.isnan() & want.isnan())
            assert bool(same.all()), (order, fma, cuts, int((~same).sum()))
    with pytest.raises(RuntimeError):     # a piece that another follows must be whole groups of 8 steps
        be.float_mm_nearest_piece(a[:, :10].contiguous(), b[:10].contiguous(), c, 2, 5, 2, 5, True, False, fma, be.MM_PIECE_MORE)


def test_streamed_k_panel_pipeline_equals_one_call():
    """Host operands long enough along K for the K-panel pipeline of float_mm_streamed (panels of A's columns and B's
    rows copied under the kernels of the panels before): bits of one float_mm call, K not a multiple of 8 included."""
    import mptorch_b200.backend as be
    import mptorch_b200.quant as q
    from mptorch_b200.quant.quant_function import _k_panels

    torch.manual_seed(5)
    for (M, K, N), fma, order in (((300, 2053, 260), False, "cuda"), ((129, 1800, 72), True, "cuda"), ((260, 3000, 200), False, "seq")):
        assert _k_panels(K) is not None
        a = torch.randn(M, K).pin_memory()
        b = torch.randn(K, N).pin_memory()
        with be.orders(accum=order):
            want = q.float_mm(a.cuda(), b.cuda(), man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest", fma=fma,
                              subnormals=True, saturate=False).cpu()
            for block in (64, 1024):
                got = q.float_mm_streamed(a, b, block_rows=block, man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest",
                                          fma=fma, subnormals=True, saturate=False)
                assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (M, K, N, fma, order, block)
    assert _k_panels(1000) is None


def test_transposed_operands_are_copied_by_the_transpose_kernel():
    """backend.transpose_last2 against torch for ragged, batched and vector-friendly shapes, and the GEMM on a
    transposed view against the GEMM on torch's dense copy of it."""
    import mptorch_b200.backend as be
    import mptorch_b200.quant as q

    g = torch.Generator(device="cuda").manual_seed(2)
    for shape in ((1, 1), (3, 5), (64, 64), (65, 127), (7, 300, 200), (2, 3, 128, 64), (1000, 3), (2, 1024, 768), (5, 0, 4)):
        x = torch.randn(*shape, device="cuda", generator=g)
        y = be.transpose_last2(x)
        assert y.is_contiguous() and torch.equal(y, x.transpose(-2, -1).contiguous()), shape
    x = torch.randn(4000, device="cuda", generator=g)[1:3601].view(60, 60)      # 4-byte aligned only
    assert torch.equal(be.transpose_last2(x.contiguous()), x.t().contiguous())
    a = torch.randn(96, 200, device="cuda", generator=g)
    w = torch.randn(72, 200, device="cuda", generator=g)
    kw = dict(man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest", fma=False, subnormals=True, saturate=False)
    assert torch.equal(q.float_mm(a, w.t(), **kw), q.float_mm(a, w.t().contiguous(), **kw))
    a3 = torch.randn(3, 200, 96, device="cuda", generator=g)
    b3 = torch.randn(3, 200, 40, device="cuda", generator=g)
    assert torch.equal(q.float_bmm(a3.transpose(-2, -1), b3, **kw), q.float_bmm(a3.transpose(-2, -1).contiguous(), b3, **kw))
