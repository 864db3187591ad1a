"""Same-GPU comparison with the reference's own CUDA extension (oracle/_ref/quant_cuda, the unmodified
reference sources compiled for sm_100a).  It pins the "cuda" accumulation order and the elementwise casts
against the code this library replaces.  Only kernels whose memory accesses are bounds-checked in the
reference source are run (elementwise quantizers, mm_impl / bmm_impl, mm_fma_impl, the Kahan-compensated
mm_kahan_impl family, whose loads carry the same guards); its stochastic GEMM (racy, out-of-range state
indexing) is never launched."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


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


@pytest.fixture(scope="module")
def be():
    from mptorch_b200 import backend

    return backend


def bits_equal(a, b):
    a, b = a.contiguous(), b.contiguous()
    same = a.view(torch.int32) == b.view(torch.int32)
    return bool((same | (a.isnan() & b.isnan())).all())


def test_float_quantize_nearest(ref_cuda, be):
    g = torch.Generator(device="cuda").manual_seed(1)
    bits = torch.randint(-2**31, 2**31 - 1, (1 << 22,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    x = bits.view(torch.float32)
    for (e, m) in [(5, 2), (4, 3), (5, 10), (8, 7), (3, 0)]:
        for sub in (False, True):
            for sat in (False, True):
                assert bits_equal(be.float_quantize_nearest(x, m, e, sub, sat), ref_cuda.float_quantize_nearest(x, m, e, sub, sat)), (e, m, sub, sat)


def test_float_quantize_stochastic_same_seed(ref_cuda, be):
    x = torch.randn(1 << 20, device="cuda") * 3
    for (e, m, prng) in [(4, 3, 20), (5, 2, 21), (5, 2, 4), (8, 7, 16)]:
        torch.manual_seed(123)
        want = ref_cuda.float_quantize_stochastic(x, m, e, prng, True, True)
        torch.manual_seed(123)
        got = be.float_quantize_stochastic(x, m, e, prng, True, True)
        assert bits_equal(got, want), (e, m, prng)


def test_binary8(ref_cuda, be):
    g = torch.Generator(device="cuda").manual_seed(2)
    bits = torch.randint(-2**31, 2**31 - 1, (1 << 20,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    x = bits.view(torch.float32)
    pol = [ref_cuda.OverflowPolicy.SATURATE_INFTY, ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT, ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT2]
    for P in (1, 3, 4, 7):
        for sg in (False, True):
            for po in range(3):
                assert bits_equal(be.binary8_quantize_nearest(x, P, sg, po, True), ref_cuda.binary8_quantize_nearest(x, P, sg, pol[po], True)), (P, sg, po)
                assert bits_equal(be.binary8_quantize_truncate(x, P, sg, po, True), ref_cuda.binary8_quantize_truncate(x, P, sg, pol[po], True)), (P, sg, po)


def _mismatches(got, want):
    """Number of elements whose bits differ (two NaNs of any payload count as equal)."""
    diff = got.view(torch.int32) != want.view(torch.int32)
    diff &= ~(got.isnan() & want.isnan())
    return int(diff.sum().item())


@pytest.mark.parametrize("fmt", [(5, 2), (4, 3), (5, 10), (8, 7)])
def test_float_quantize_nearest_all_bit_patterns(ref_cuda, be, fmt):
    """Every one of the 2^32 fp32 bit patterns, in 16 chunks of 2^28, through this library's nearest quantizer and
    through the reference's float_kernel_nearest (quant_cuda/fp_kernel.cu:12-58, 164-172), for the four formats
    of the benchmark configurations with subnormals and saturation on and off."""
    e, m = fmt
    chunk = 1 << 28
    for sub in (True, False):
        for sat in (True, False):
            bad = 0
            for c in range(16):
                lo = -(1 << 31) + c * chunk
                x = torch.arange(lo, lo + chunk, dtype=torch.int32, device="cuda").view(torch.float32)
                got = be.float_quantize_nearest(x, m, e, sub, sat)
                want = ref_cuda.float_quantize_nearest(x, m, e, sub, sat)
                bad += _mismatches(got, want)
                del x, got, want
            assert bad == 0, (e, m, sub, sat, bad)


def test_binary8_p3_nearest_all_bit_patterns(ref_cuda, be):
    """All 2^32 inputs through binary8 P=3 signed nearest (benchmark config 2's arm: saturate_maxfloat, subnormals),
    plus the other two overflow policies, against the reference's kernel (quant_cuda/binary8_kernel.cu:11-276)."""
    pol = [ref_cuda.OverflowPolicy.SATURATE_INFTY, ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT, ref_cuda.OverflowPolicy.SATURATE_MAXFLOAT2]
    chunk = 1 << 28
    for po in (1, 0, 2):
        bad = 0
        for c in range(16):
            lo = -(1 << 31) + c * chunk
            x = torch.arange(lo, lo + chunk, dtype=torch.int32, device="cuda").view(torch.float32)
            got = be.binary8_quantize_nearest(x, 3, True, po, True)
            want = ref_cuda.binary8_quantize_nearest(x, 3, True, pol[po], True)
            bad += _mismatches(got, want)
            del x, got, want
        assert bad == 0, (po, bad)


@pytest.mark.parametrize("shape", [(256, 256, 256), (78, 101, 145), (64, 203, 96), (512, 1000, 320)])
def test_mm_kahan_cuda_order(ref_cuda, be, shape):
    """The Kahan-compensated GEMMs against the reference's mm_kahan_impl / mm_kahan_fma_impl
    (quant_cuda/mm_kernel.h:457-676, selected by `compensated` at fp_kernel.cu:190-198); K = 203 and 145 are not
    multiples of the reference's 8-wide tile."""
    M, K, N = shape
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    for (ea, ma, em, mm_) in [(5, 2, 5, 2), (5, 10, 4, 3), (8, 7, 5, 2)]:
        want = torch.zeros(M, N, device="cuda")
        ref_cuda.float_quantize_nearest_mm(a, b, want, M, N, K, ma, ea, mm_, em, True, False, True)
        got = torch.empty(M, N, device="cuda")
        be.float_quantize_nearest_mm(a, b, got, M, N, K, ma, ea, mm_, em, True, False, True, order="cuda")
        assert bits_equal(got, want), (shape, ea, ma, em, mm_)
        want = torch.zeros(M, N, device="cuda")
        ref_cuda.float_quantize_nearest_mm_fma(a, b, want, M, N, K, ma, ea, True, False, True)
        got = torch.empty(M, N, device="cuda")
        be.float_quantize_nearest_mm_fma(a, b, got, M, N, K, ma, ea, True, False, True, order="cuda")
        assert bits_equal(got, want), ("fma", shape, ea, ma)


def test_bmm_kahan_cuda_order(ref_cuda, be):
    a = torch.randn(5, 96, 77, device="cuda") * 4
    b = torch.randn(5, 77, 64, device="cuda")
    for sat in (False, True):
        want = torch.zeros(5, 96, 64, device="cuda")
        ref_cuda.float_quantize_nearest_bmm(a, b, want, 96, 64, 77, 10, 5, 3, 4, True, sat, True)
        got = torch.empty(5, 96, 64, device="cuda")
        be.float_quantize_nearest_bmm(a, b, got, 96, 64, 77, 10, 5, 3, 4, True, sat, True, order="cuda")
        assert bits_equal(got, want), sat
        want = torch.zeros(5, 96, 64, device="cuda")
        ref_cuda.float_quantize_nearest_bmm_fma(a, b, want, 96, 64, 77, 2, 5, True, sat, True)
        got = torch.empty(5, 96, 64, device="cuda")
        be.float_quantize_nearest_bmm_fma(a, b, got, 96, 64, 77, 2, 5, True, sat, True, order="cuda")
        assert bits_equal(got, want), ("fma", sat)


@pytest.mark.parametrize("shape", [(256, 256, 256), (78, 101, 145), (512, 1000, 320)])
def test_mm_cuda_order(ref_cuda, be, shape):
    M, K, N = shape
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    for (ea, ma, em, mm_) in [(5, 2, 5, 2), (5, 10, 4, 3), (8, 7, 5, 2)]:
        want = torch.zeros(M, N, device="cuda")
        ref_cuda.float_quantize_nearest_mm(a, b, want, M, N, K, ma, ea, mm_, em, True, False, False)
        got = torch.empty(M, N, device="cuda")
        be.float_quantize_nearest_mm(a, b, got, M, N, K, ma, ea, mm_, em, True, False, False, order="cuda")
        assert bits_equal(got, want), (shape, ea, ma, em, mm_)
        want = torch.zeros(M, N, device="cuda")
        ref_cuda.float_quantize_nearest_mm_fma(a, b, want, M, N, K, ma, ea, True, False, False)
        got = torch.empty(M, N, device="cuda")
        be.float_quantize_nearest_mm_fma(a, b, got, M, N, K, ma, ea, True, False, False, order="cuda")
        assert bits_equal(got, want), ("fma", shape, ea, ma)


def test_bmm_cuda_order(ref_cuda, be):
    a = torch.randn(6, 128, 64, device="cuda")
    b = torch.randn(6, 64, 96, device="cuda")
    want = torch.zeros(6, 128, 96, device="cuda")
    ref_cuda.float_quantize_nearest_bmm(a, b, want, 128, 96, 64, 10, 5, 3, 4, True, False, False)
    got = torch.empty(6, 128, 96, device="cuda")
    be.float_quantize_nearest_bmm(a, b, got, 128, 96, 64, 10, 5, 3, 4, True, False, False, order="cuda")
    assert bits_equal(got, want)


def test_full_size_headline_vs_reference(ref_cuda, be):
    """4096^3, e5m2: the whole matrix equals the reference CUDA kernel's output."""
    S = 4096
    a = torch.randn(S, S, device="cuda")
    b = torch.randn(S, S, device="cuda")
    want = torch.zeros(S, S, device="cuda")
    ref_cuda.float_quantize_nearest_mm(a, b, want, S, S, S, 2, 5, 2, 5, True, False, False)
    got = torch.empty(S, S, device="cuda")
    be.float_quantize_nearest_mm(a, b, got, S, S, S, 2, 5, 2, 5, True, False, False, order="cuda")
    assert bits_equal(got, want)


def test_softmax_and_layernorm_cuda_order(ref_cuda):
    """Row reductions in the CUDA association, expf/logf from the same CUDA math library: bit for bit."""
    import mptorch_b200.quant as q

    x = torch.randn(6, 40, 1024, device="cuda") * 3
    g = torch.randn_like(x)
    for (e, m) in [(5, 10), (8, 7), (8, 23), (4, 3)]:
        for dim in (-1, 1):
            want = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_forward(x, want, dim, m, e, m, e, m, e, True, False)
            got = q.float_softmax_forward(x, dim, m, e, m, e, m, e)
            assert bits_equal(got, want), ("softmax", e, m, dim)
            want2 = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_lse_forward(x, want2, dim, m, e, m, e, True, False)
            got2 = q.float_softmax_lse_forward(x, dim, m, e, m, e)
            assert bits_equal(got2, want2), ("softmax lse", e, m, dim)
            want3 = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_backward(want, g, want3, dim, m, e, m, e, True, False)
            got3 = q.float_softmax_backward(want, g, dim, m, e, m, e)
            assert bits_equal(got3, want3), ("softmax bwd", e, m, dim)
    xl = torch.randn(4, 256, 768, device="cuda") * 2 + 0.3
    gl = torch.randn_like(xl)
    w = torch.randn(768, device="cuda")
    b = torch.randn(768, device="cuda")
    for (e, m) in [(5, 10), (8, 7), (8, 23)]:
        y = torch.zeros_like(xl)
        mean = torch.zeros(4, 256, device="cuda")
        rstd = torch.zeros(4, 256, device="cuda")
        ref_cuda.float_quantize_layernorm_forward(xl, w, b, y, mean, rstd, 1e-5, [-1], m, e, m, e, m, e, m, e, True, False)
        gy, gm, gr = q.float_layernorm_forward(xl, w, b, 1e-5, [-1], m, e, m, e, m, e, m, e)
        assert bits_equal(gy, y) and bits_equal(gm, mean) and bits_equal(gr, rstd), ("layernorm fwd", e, m)
        gi = torch.zeros_like(xl)
        gg = torch.zeros(768, device="cuda")
        gb = torch.zeros(768, device="cuda")
        ref_cuda.float_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, gi, gg, gb, [-1], m, e, m, e, m, e, True, False)
        ogi, ogg, ogb = q.float_layernorm_backward(xl, gl, w, b, mean, rstd, [-1], m, e, m, e, m, e)
        assert bits_equal(ogi, gi) and bits_equal(ogg, gg) and bits_equal(ogb, gb), ("layernorm bwd", e, m)


@pytest.mark.parametrize("shape", [(256, 256, 256), (78, 101, 145), (300, 2048, 136)])
def test_mm_with_formats_that_round_nothing(ref_cuda, be, shape):
    """fp32 as the add format (low-precision products accumulated in fp32), as the multiply format, or as both, against
    the reference's CUDA kernel.  With a multiply format that rounds nothing that kernel's `sum + a * b` is evaluated as
    one fused multiply-add by the reference's build; the CUDA order reproduces it.  The operands include magnitudes whose
    sums leave the range-checked path (1e30) and zeros of both signs."""
    M, K, N = shape
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    a[1, :] = 0.0
    a[2, ::3] = -0.0
    a[3, :8] = 1e30
    b[:8, 5] = 1e30
    for (ma, ea, mm_, em) in [(23, 8, 23, 8), (23, 8, 3, 4), (23, 8, 2, 5), (23, 8, 7, 8), (10, 5, 23, 8), (7, 8, 23, 8), (2, 5, 23, 8)]:
        for batched in (False, True):
            aa, bb = (a.view(1, M, K).repeat(2, 1, 1).contiguous(), b.view(1, K, N).repeat(2, 1, 1).contiguous()) if batched else (a, b)
            want = torch.zeros(*aa.shape[:-1], N, device="cuda")
            got = torch.empty_like(want)
            if batched:
                ref_cuda.float_quantize_nearest_bmm(aa, bb, want, M, N, K, ma, ea, mm_, em, True, False, False)
                be.float_quantize_nearest_bmm(aa, bb, got, M, N, K, ma, ea, mm_, em, True, False, False, order="cuda")
            else:
                ref_cuda.float_quantize_nearest_mm(aa, bb, want, M, N, K, ma, ea, mm_, em, True, False, False)
                be.float_quantize_nearest_mm(aa, bb, got, M, N, K, ma, ea, mm_, em, True, False, False, order="cuda")
            assert bits_equal(got, want), (shape, ma, ea, mm_, em, batched)
    want = torch.zeros(M, N, device="cuda")
    got = torch.empty_like(want)
    ref_cuda.float_quantize_nearest_mm_fma(a, b, want, M, N, K, 23, 8, True, False, False)
    be.float_quantize_nearest_mm_fma(a, b, got, M, N, K, 23, 8, True, False, False, order="cuda")
    assert bits_equal(got, want), ("fma", shape)


@pytest.mark.parametrize("shape", [(256, 256, 256), (78, 101, 145), (300, 2048, 136)])
def test_mm_formats_without_subnormals(ref_cuda, be, shape):
    """Float formats without subnormals (the default of the reference's FloatingPoint) on the range-checked path:
    products and sums that land below the smallest normal value are settled as the reference's
    clip_exponent_without_subnormals does (bit_helper.cu:166-199).  Operands scaled so that a large share of the
    products and many partial sums fall below 2^min_exp, rows that cancel to zero, zeros of both signs, and operands
    large enough to leave the range-checked path; plain and fused, batched and not."""
    M, K, N = shape
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randn(M, K, device="cuda", generator=g)
    b = torch.randn(K, N, device="cuda", generator=g)
    a[0] *= 2.0 ** -7
    a[1] *= 2.0 ** -12
    a[2, 1::2] = -a[2, 0::2][: a[2, 1::2].numel()]
    b[1::2, 3] = b[0::2, 3][: b[1::2, 3].numel()]
    a[3] = 0.0
    a[4, ::3] = -0.0
    for (ma, ea, mm_, em) in [(2, 5, 2, 5), (10, 5, 3, 4), (7, 8, 2, 5), (3, 4, 3, 4), (1, 3, 1, 3), (21, 8, 10, 5)]:
        for scale in (1.0, 2.0 ** -5, 300.0):
            aa = (a * scale).contiguous()
            want = torch.zeros(M, N, device="cuda")
            got = torch.empty_like(want)
            ref_cuda.float_quantize_nearest_mm(aa, b, want, M, N, K, ma, ea, mm_, em, False, False, False)
            be.float_quantize_nearest_mm(aa, b, got, M, N, K, ma, ea, mm_, em, False, False, False, order="cuda")
            assert bits_equal(got, want), (shape, ma, ea, mm_, em, scale, int((got.view(torch.int32) != want.view(torch.int32)).sum()))
            ref_cuda.float_quantize_nearest_mm_fma(aa, b, want, M, N, K, ma, ea, False, False, False)
            be.float_quantize_nearest_mm_fma(aa, b, got, M, N, K, ma, ea, False, False, False, order="cuda")
            assert bits_equal(got, want), ("fma", shape, ma, ea, scale)
        a3, b3 = a.view(1, M, K).repeat(3, 1, 1).contiguous(), b.view(1, K, N).repeat(3, 1, 1).contiguous()
        a3[1] *= 2.0 ** -6
        want = torch.zeros(3, M, N, device="cuda")
        got = torch.empty_like(want)
        ref_cuda.float_quantize_nearest_bmm(a3, b3, want, M, N, K, ma, ea, mm_, em, False, True, False)
        be.float_quantize_nearest_bmm(a3, b3, got, M, N, K, ma, ea, mm_, em, False, True, False, order="cuda")
        assert bits_equal(got, want), ("bmm saturate", shape, ma, ea, mm_, em)


def test_softmax_and_layernorm_in_formats_without_subnormals(ref_cuda, be):
    """The register-resident row kernels in their mode for formats without subnormals (settling rounding), against the
    reference's CUDA kernels: inputs scaled so that exponentials, squares and products land below the smallest normal
    value of the format, rows with fp32 denormals and infinities (which leave the trusted path), reduced dimension
    last (register-resident kernels) and in the middle (general kernels)."""
    import mptorch_b200.quant as q

    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(6, 40, 1024, device="cuda", generator=g) * 3
    x[0, 0] *= 8.0
    x[0, 1, :5] = 1e-41
    x[0, 2, 7] = float("-inf")
    gr = torch.randn(6, 40, 1024, device="cuda", generator=g)
    gr[1] *= 2.0 ** -10
    for (e, m) in [(5, 10), (4, 3), (8, 7), (5, 2)]:
        for dim in (-1, 1):
            want = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_forward(x, want, dim, m, e, m, e, m, e, False, False)
            got = torch.empty_like(x)
            be.float_quantize_nearest_softmax_forward(x, got, dim, m, e, m, e, m, e, False, False)
            assert bits_equal(got, want), ("softmax", e, m, dim)
            want2 = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_lse_forward(x, want2, dim, m, e, m, e, False, False)
            got2 = torch.empty_like(x)
            be.float_quantize_nearest_softmax_lse_forward(x, got2, dim, m, e, m, e, False, False)
            assert bits_equal(got2, want2), ("softmax lse", e, m, dim)
            want3 = torch.zeros_like(x)
            ref_cuda.float_quantize_nearest_softmax_backward(want, gr, want3, dim, m, e, m, e, False, False)
            got3 = torch.empty_like(x)
            be.float_quantize_nearest_softmax_backward(want, gr, got3, dim, m, e, m, e, False, False)
            assert bits_equal(got3, want3), ("softmax bwd", e, m, dim)
    xl = torch.randn(4, 256, 768, device="cuda", generator=g) * 2 + 0.3
    xl[0, :8] *= 2.0 ** -9
    xl[1, 3, :4] = 1e-40
    gl = torch.randn(4, 256, 768, device="cuda", generator=g)
    gl[2] *= 2.0 ** -8
    w = torch.randn(768, device="cuda", generator=g)
    b = torch.randn(768, device="cuda", generator=g)
    for (e, m) in [(5, 10), (8, 7), (6, 9)]:
        y, mean, rstd = torch.zeros_like(xl), torch.zeros(4, 256, device="cuda"), torch.zeros(4, 256, device="cuda")
        ref_cuda.float_quantize_layernorm_forward(xl, w, b, y, mean, rstd, 1e-5, [-1], m, e, m, e, m, e, m, e, False, False)
        gy, gm, grs = torch.empty_like(xl), torch.empty(4, 256, device="cuda"), torch.empty(4, 256, device="cuda")
        be.float_quantize_layernorm_forward(xl, w, b, gy, gm, grs, 1e-5, [-1], m, e, m, e, m, e, m, e, False, False)
        assert bits_equal(gy, y) and bits_equal(gm, mean) and bits_equal(grs, rstd), ("layernorm fwd", e, m)
        gi, gg, gb = torch.zeros_like(xl), torch.zeros(768, device="cuda"), torch.zeros(768, device="cuda")
        ref_cuda.float_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, gi, gg, gb, [-1], m, e, m, e, m, e, False, False)
        ogi, ogg, ogb = torch.empty_like(xl), torch.empty(768, device="cuda"), torch.empty(768, device="cuda")
        be.float_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, ogi, ogg, ogb, [-1], m, e, m, e, m, e, False, False)
        assert bits_equal(ogi, gi) and bits_equal(ogg, gg) and bits_equal(ogb, gb), ("layernorm bwd", e, m)


def test_large_products_leave_failed_range_checks_to_the_exact_kernel(ref_cuda, be):
    """Products of at least 2^33 MACs launch the exact kernel behind the range-checked one; it computes the batch
    entries whose operand statistics rule the range-checked path out and skips the others.  Batch of two 2048^3
    products: entry 0 is ordinary, entry 1 holds one infinity; then a single product with operands scaled by 200
    (sums overflow e5m2).  Against the reference's CUDA kernels."""
    S = 2048
    g = torch.Generator(device="cuda").manual_seed(6)
    a = torch.randn(2, S, S, device="cuda", generator=g)
    b = torch.randn(2, S, S, device="cuda", generator=g)
    a[1, 5, 7] = float("inf")
    want = torch.zeros(2, S, S, device="cuda")
    got = torch.full((2, S, S), float("nan"), device="cuda")
    ref_cuda.float_quantize_nearest_bmm(a, b, want, S, S, S, 10, 5, 3, 4, True, False, False)
    be.float_quantize_nearest_bmm(a, b, got, S, S, S, 10, 5, 3, 4, True, False, False, order="cuda")
    assert bits_equal(got[0], want[0]), "entry on the range-checked path"
    assert bits_equal(got[1], want[1]), "entry left to the exact kernel"
    a2 = (a[0] * 200).contiguous()
    w2 = torch.zeros(S, S, device="cuda")
    g2 = torch.full((S, S), float("nan"), device="cuda")
    ref_cuda.float_quantize_nearest_mm(a2, b[0], w2, S, S, S, 2, 5, 2, 5, True, False, False)
    be.float_quantize_nearest_mm(a2, b[0], g2, S, S, S, 2, 5, 2, 5, True, False, False, order="cuda")
    assert bits_equal(g2, w2)
