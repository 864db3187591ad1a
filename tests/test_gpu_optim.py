"""Multi-tensor quantization and the low-precision optimizer wrapper.

`float_quantize_multi` must give, per tensor, the bits of `float_quantize`; `QOptim` must leave a model in exactly
the state the reference's per-tensor wrapper (optim/optim_low.py:65-113, restated inline below) leaves it in."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    import mptorch_b200.quant as quant

    return quant


def bits_equal(a, b):
    a, b = a.contiguous(), b.contiguous()
    same = a.view(torch.int32) == b.view(torch.int32)
    return bool((same | (a.isnan() & b.isnan())).all())


SIZES = [0, 1, 3, 4, 5, 17, 255, 256, 1023, 4096, 4097, 16384, 100003, 768 * 768, 3 * 1024 * 1024 + 1]


@pytest.mark.parametrize("fmt", [(5, 2), (4, 3), (8, 7), (5, 10), (8, 23), (3, 0)])
@pytest.mark.parametrize("rounding", ["nearest", "truncate"])
def test_multi_equals_single(q, fmt, rounding):
    e, m = fmt
    g = torch.Generator(device="cuda").manual_seed(3)
    tensors = []
    for i, n in enumerate(SIZES * 4):                       # 60 tensors: more than one launch
        bits = torch.randint(-2**31, 2**31 - 1, (n,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
        t = bits.view(torch.float32) if i % 3 == 0 else torch.randn(n, device="cuda", generator=g) * 10.0 ** (i % 7 - 3)
        tensors.append(t)
    for sub in (True, False):
        for sat in (True, False):
            outs = q.float_quantize_multi(tensors, e, m, rounding, sub, sat)
            assert len(outs) == len(tensors)
            for t, o in zip(tensors, outs):
                assert o.shape == t.shape
                assert bits_equal(o, q.float_quantize(t, e, m, rounding, sub, sat)), (fmt, rounding, sub, sat, t.numel())


def test_multi_unaligned_views_and_inplace(q):
    base = torch.randn(10000, device="cuda")
    views = [base[1:1000], base[1001:1004], base[2000:6001]]          # 4-byte aligned only; views of one buffer
    want = [q.float_quantize(v, 4, 3, "nearest") for v in views]
    outs = q.float_quantize_multi(views, 4, 3, "nearest")
    assert all(bits_equal(a, b) for a, b in zip(outs, want))
    owned = [v.clone() for v in views]
    same = q.float_quantize_multi(owned, 4, 3, "nearest", inplace=True)
    assert all(s is o for s, o in zip(same, owned))
    assert all(bits_equal(a, b) for a, b in zip(owned, want))


def test_multi_stochastic_is_seeded_unbiased_and_on_grid(q):
    x = [torch.full((1 << 16,), 0.3, device="cuda"), torch.full((1 << 16,), 0.3, device="cuda"), torch.randn(1000, device="cuda")]
    a = q.float_quantize_multi(x, 4, 3, "stochastic", seed=11)
    b = q.float_quantize_multi(x, 4, 3, "stochastic", seed=11)
    c = q.float_quantize_multi(x, 4, 3, "stochastic", seed=12)
    assert all(bits_equal(u, v) for u, v in zip(a, b))
    assert not bits_equal(a[0], c[0])
    assert not bits_equal(a[0], a[1])                    # equal tensors at different list positions draw different words
    lo, hi = 0.28125, 0.3125                             # neighbours of 0.3 in e4m3
    assert set(a[0].unique().tolist()) <= {lo, hi}
    assert abs(a[0].mean().item() - 0.3) < 2e-4
    torch.manual_seed(5)
    d = q.float_quantize_multi(x, 4, 3, "stochastic")
    torch.manual_seed(5)
    e = q.float_quantize_multi(x, 4, 3, "stochastic")
    assert all(bits_equal(u, v) for u, v in zip(d, e))


class _RefQOptim:
    """The reference wrapper's step, one quantizer call per tensor (optim/optim_low.py:65-113)."""

    def __init__(self, optim, weight_quant=None, grad_quant=None, momentum_quant=None, acc_quant=None):
        self.optim, self.param_groups = optim, optim.param_groups
        self.weight_quant, self.grad_quant, self.momentum_quant, self.acc_quant = weight_quant, grad_quant, momentum_quant, acc_quant
        self.keys = ["momentum_buffer"] if isinstance(optim, torch.optim.SGD) else ["exp_avg", "exp_avg_sq"]
        if acc_quant is not None:
            self.weight_acc = {p: p.detach().clone() for g in self.param_groups for p in g["params"]}

    def step(self):
        if self.grad_quant is not None:
            for g in self.param_groups:
                for p in g["params"]:
                    if p.grad is not None:
                        p.grad.data = self.grad_quant(p.grad.data)
        if self.acc_quant is not None:
            for g in self.param_groups:
                for p in g["params"]:
                    p.data = self.weight_acc[p].data
        self.optim.step()
        if self.acc_quant is not None:
            for g in self.param_groups:
                for p in g["params"]:
                    p.data = self.weight_acc[p].data = self.acc_quant(p.data).data
        if self.weight_quant is not None:
            for g in self.param_groups:
                for p in g["params"]:
                    p.data = self.weight_quant(p.data).data
        if self.momentum_quant is not None:
            for g in self.param_groups:
                if isinstance(self.optim, torch.optim.SGD) and g["momentum"] == 0:
                    continue
                for p in g["params"]:
                    if p.grad is None:
                        continue
                    st = self.optim.state[p]
                    for k in self.keys:
                        st[k] = self.momentum_quant(st[k])


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(96, 200), torch.nn.GELU(), torch.nn.LayerNorm(200), torch.nn.Linear(200, 33),
                               torch.nn.Linear(33, 1, bias=False)).cuda()


@pytest.mark.parametrize("kind", ["sgd", "sgd_nomomentum", "adam", "adamw"])
def test_qoptim_equals_per_tensor_wrapper(q, kind):
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import QOptim

    wq = q.quantizer(forward_number=FloatingPoint(5, 10, True, True), forward_rounding="nearest")
    gq = q.quantizer(forward_number=FloatingPoint(5, 2, True, False), forward_rounding="nearest")
    mq = q.quantizer(forward_number=FloatingPoint(8, 7, True, True), forward_rounding="nearest")
    aq = q.quantizer(forward_number=FloatingPoint(6, 13, True, True), forward_rounding="nearest")
    plain = {"w": lambda t: q.float_quantize(t, 5, 10, "nearest", True, True), "g": lambda t: q.float_quantize(t, 5, 2, "nearest", True, False),
             "m": lambda t: q.float_quantize(t, 8, 7, "nearest", True, True), "a": lambda t: q.float_quantize(t, 6, 13, "nearest", True, True)}

    def make(model):
        ps = model.parameters()
        if kind == "sgd":
            return torch.optim.SGD(ps, lr=0.05, momentum=0.9)
        if kind == "sgd_nomomentum":
            return torch.optim.SGD(ps, lr=0.05)
        if kind == "adam":
            return torch.optim.Adam(ps, lr=1e-2)
        return torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.1)

    m1, m2 = _model(), _model()
    o1 = QOptim(make(m1), weight_quant=wq, grad_quant=gq, momentum_quant=mq, acc_quant=aq)
    o2 = _RefQOptim(make(m2), weight_quant=plain["w"], grad_quant=plain["g"], momentum_quant=plain["m"], acc_quant=plain["a"])
    g = torch.Generator(device="cuda").manual_seed(1)
    for step in range(4):
        x = torch.randn(64, 96, device="cuda", generator=g)
        for m, o in ((m1, o1), (m2, o2)):
            for p in m.parameters():
                p.grad = None
            m(x).square().mean().backward()
            if step == 2:
                list(m.parameters())[-1].grad = None          # a parameter without a gradient is skipped
            o.step()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            assert bits_equal(p1.data, p2.data), (kind, step)
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            s1, s2 = o1.optim.state.get(p1, {}), o2.optim.state.get(p2, {})
            for k in o1.momentum_keys:
                if k in s2 and s2[k] is not None:
                    assert bits_equal(s1[k], s2[k]), (kind, step, k)


def test_qoptim_passes_other_callables_through(q):
    from mptorch_b200.optim import QOptim

    calls = []

    def wq(t):
        calls.append(t.numel())
        return q.float_quantize(t, 4, 3, "nearest")

    m = _model()
    o = QOptim(torch.optim.SGD(m.parameters(), lr=0.1), weight_quant=wq)
    m(torch.randn(8, 96, device="cuda")).sum().backward()
    o.step()
    assert len(calls) == len(list(m.parameters()))
    for p in m.parameters():
        assert bits_equal(p.data, q.float_quantize(p.data, 4, 3, "nearest"))


# ------------------------------------------------------------------------------------------ QSGD / QAdamW
def _models(seed, n=3):
    g = torch.Generator().manual_seed(seed)
    shapes = [(301,), (64, 33), (7, 5, 3), (4096 + 5,), (1,)]
    return [[torch.nn.Parameter(torch.randn(s, generator=g).cuda()) for s in shapes] for _ in range(n)], shapes, g


def _same(a, b):
    return torch.equal(a.detach().contiguous().view(torch.int32), b.detach().contiguous().view(torch.int32))


SGD_CONFIGS = [
    dict(lr=0.05, momentum=0.9),
    dict(lr=0.05, momentum=0.9, compensated=True),
    dict(lr=0.1, momentum=0.8, dampening=0.25, weight_decay=0.01, compensated=True),
    dict(lr=0.1, momentum=0.8, nesterov=True, weight_decay=0.001),
    dict(lr=0.03, momentum=0.0, compensated=True),
    dict(lr=0.03, momentum=0.0),
]


@pytest.mark.parametrize("cfg", SGD_CONFIGS)
@pytest.mark.parametrize("fmts", [((8, 7), (8, 7)), ((5, 10), (5, 2)), (None, (4, 3)), ((5, 2), None), ((3, 0), (1, 3)), (None, None)])
def test_qsgd_fused_step_equals_per_tensor_steps(cfg, fmts):
    """One fused launch per step against the reference's per-tensor sequence of torch kernels and quantizer calls,
    on identical parameters and gradients, bit for bit, buffers included."""
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import QSGD, fma_quantizer

    mq, aq = [fma_quantizer(FloatingPoint(f[0], f[1], True, True)) if f else None for f in fmts]
    (pa, pb, _), shapes, g = _models(11)
    for x, y in zip(pa, pb):
        y.data.copy_(x.data)
    oa = QSGD(pa, momentum_quant=mq, acc_quant=aq, **cfg)                  # fused
    ob = QSGD(pb, momentum_quant=mq, acc_quant=aq, fused=False, **cfg)     # per tensor
    for step in range(4):
        for x, y in zip(pa, pb):
            gr = (torch.randn(x.shape, generator=g) * (0.3 + step)).cuda()
            x.grad, y.grad = gr.clone(), gr.clone()
        oa.step()
        ob.step()
        for i, (x, y) in enumerate(zip(pa, pb)):
            assert _same(x.data, y.data), ("param", step, i, cfg, fmts)
            assert _same(x.grad, y.grad), ("grad", step, i)
            for key in ("momentum_buffer", "compensated_buffer"):
                if key in ob.state[y]:
                    assert _same(oa.state[x][key], ob.state[y][key]), (key, step, i, cfg, fmts)


ADAM_CONFIGS = [
    dict(lr=0.01, betas=(0.9, 0.99)),
    dict(lr=0.01, betas=(0.9, 0.99), compensated=True),
    dict(lr=0.02, betas=(0.8, 0.95), amsgrad=True, eps=1e-6),
    dict(lr=0.02, betas=(0.8, 0.95), amsgrad=True, compensated=True),
]


@pytest.mark.parametrize("cfg", ADAM_CONFIGS)
@pytest.mark.parametrize("fmts", [((8, 7), (8, 7)), ((5, 10), (5, 2)), (None, (4, 3)), ((5, 10), None), (None, None)])
def test_qadamw_fused_step_equals_per_tensor_steps(cfg, fmts):
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import QAdamW, fma_quantizer

    mq, aq = [fma_quantizer(FloatingPoint(f[0], f[1], True, True)) if f else None for f in fmts]
    (pa, pb, _), shapes, g = _models(12)
    for x, y in zip(pa, pb):
        y.data.copy_(x.data)
    oa = QAdamW(pa, momentum_quant=mq, acc_quant=aq, **cfg)
    ob = QAdamW(pb, momentum_quant=mq, acc_quant=aq, fused=False, **cfg)
    for step in range(4):
        for x, y in zip(pa, pb):
            gr = (torch.randn(x.shape, generator=g) * (0.3 + step)).cuda()
            x.grad, y.grad = gr.clone(), gr.clone()
        oa.step()
        ob.step()
        for i, (x, y) in enumerate(zip(pa, pb)):
            assert _same(x.data, y.data), ("param", step, i, cfg, fmts)
            assert oa.state[x]["step"] == ob.state[y]["step"]
            for key in ("exp_avg", "exp_avg_sq", "max_exp_avg_sq", "compensated_buffer"):
                if key in ob.state[y]:
                    assert _same(oa.state[x][key], ob.state[y][key]), (key, step, i, cfg, fmts)


def _awkward(n, g, scale):
    """Values around every special case of a rounding to an 8-bit-exponent format: zeros of both signs, fp32
    denormals, the smallest normals, magnitudes next to the top of the range, infinities and NaN, among ordinary ones."""
    x = torch.randn(n, generator=g) * scale
    special = torch.tensor([0.0, -0.0, 1e-45, -3e-42, 1.1754942e-38, 1.1754944e-38, -1.2e-38, 3.3e38, -3.4e38, 3.4028235e38,
                            float("inf"), float("-inf"), float("nan"), 1e-30, -1e30, 2.5e-39])
    idx = torch.randperm(n, generator=g)[: 8 * special.numel()]
    x[idx] = special.repeat(8)
    return x


@pytest.mark.parametrize("opt", ["sgd", "sgd_comp", "adamw", "adamw_comp"])
@pytest.mark.parametrize("fmt", [(8, 7), (8, 3), (5, 10), (8, 7, False), (5, 10, False), (4, 3, False)])
def test_fused_steps_with_denormals_extremes_and_nonfinite_values(opt, fmt):
    """Whole 2048-element chunks (the vector path of the fused kernels) holding inputs that the straight-line rounding
    hands to the exact caster; the per-tensor sequence of torch kernels and quantizer calls is the reference."""
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import QAdamW, QSGD, fma_quantizer

    g = torch.Generator().manual_seed(21)
    q = fma_quantizer(FloatingPoint(fmt[0], fmt[1], fmt[2] if len(fmt) > 2 else True, True))      # third entry: subnormals
    n = 3 * 2048 + 17
    base = _awkward(n, g, 1.0)
    pa, pb = [torch.nn.Parameter(base.clone().cuda())], [torch.nn.Parameter(base.clone().cuda())]
    comp = opt.endswith("comp")
    if opt.startswith("sgd"):
        oa = QSGD(pa, lr=0.05, momentum=0.9, momentum_quant=q, acc_quant=q, compensated=comp)
        ob = QSGD(pb, lr=0.05, momentum=0.9, momentum_quant=q, acc_quant=q, compensated=comp, fused=False)
        keys = ("momentum_buffer", "compensated_buffer")
    else:
        oa = QAdamW(pa, lr=0.01, momentum_quant=q, acc_quant=q, compensated=comp)
        ob = QAdamW(pb, lr=0.01, momentum_quant=q, acc_quant=q, compensated=comp, fused=False)
        keys = ("exp_avg", "exp_avg_sq", "compensated_buffer")
    for step in range(3):
        gr = _awkward(n, g, 10.0 ** (step - 1)).cuda()
        pa[0].grad, pb[0].grad = gr.clone(), gr.clone()
        oa.step()
        ob.step()
        assert _same_or_nan(pa[0].data, pb[0].data), (opt, fmt, step)
        for key in keys:
            if key in ob.state[pb[0]]:
                assert _same_or_nan(oa.state[pa[0]][key], ob.state[pb[0]][key]), (key, opt, fmt, step)


def _same_or_nan(a, b):
    """Bit equality where either side is a number; a NaN must be a NaN on the other side (its payload is the
    arithmetic unit's business)."""
    a, b = a.detach().contiguous(), b.detach().contiguous()
    both_nan = a.isnan() & b.isnan()
    eq = a.view(torch.int32) == b.view(torch.int32)
    return bool((eq | both_nan).all())


@pytest.mark.parametrize("name", ["sgd_mom_acc", "sgd_mom_acc_comp", "sgd_mom_damp_comp_e5m2", "sgd_mom_only"])
def test_qsgd_fused_step_matches_reference_fixture(name):
    """The fused kernel against the outputs of the reference's own QSGD (CPU run, committed fixture): these cases use
    only separately rounded multiplies and adds, which a CPU and a GPU evaluate alike, so the bits must agree."""
    from test_optim_cpu import check_against_fixture

    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import fma_quantizer

    check_against_fixture(name, lambda fmt: fma_quantizer(FloatingPoint(fmt[0], fmt[1], True, True)) if fmt else None, device="cuda")


def test_optimizers_fall_back_for_other_callables():
    """Any other trivariate callable takes the per-tensor path and still works on CUDA tensors."""
    from mptorch_b200.optim import QSGD
    from mptorch_b200.quant import float_quantize

    p = torch.nn.Parameter(torch.randn(50).cuda())
    q = lambda x, y, z: float_quantize(x + y * z, 8, 7, "nearest")   # noqa: E731
    opt = QSGD([p], lr=0.1, momentum=0.9, momentum_quant=q, acc_quant=q, compensated=True)
    before = p.data.clone()
    p.grad = torch.randn(50).cuda()
    opt.step()
    assert not torch.equal(before, p.data) and torch.isfinite(p.data).all()
