"""QSGD / QAdamW on CPU tensors: the per-tensor path of mptorch_b200.optim (the reference's sequence of torch operations)
against fixtures produced by the reference's own optimizers (tests/golden/make_optim_golden.py), bit for bit.  The
quantizer callables are built on the CPU oracle, as the fixtures' were built on the reference CPU extension."""
import numpy as np
import pytest
import torch

from conftest import golden

from tests.golden.make_optim_golden import CASES, SHAPES, STEPS


def _oracle_quant(oracle, fmt):
    if fmt is None:
        return None
    e, m = fmt
    return lambda x, y, z: torch.from_numpy(oracle.float_quantize((x + y * z).contiguous().numpy(), m, e, "nearest", True, True)).reshape(x.shape)


def run_case(name, make_quant, device="cpu", **extra):
    """Replays a fixture case; yields (step, index, parameter, optimizer state) after every step."""
    from mptorch_b200.optim import QAdamW, QSGD

    fx = golden("optim_steps.npz")
    kind, kw, mfmt, afmt = CASES[name]
    params = [torch.nn.Parameter(torch.from_numpy(fx["%s/init/%d" % (name, i)].view(np.float32).copy()).to(device)) for i in range(len(SHAPES))]
    cls = QSGD if kind == "sgd" else QAdamW
    opt = cls(params, momentum_quant=make_quant(mfmt), acc_quant=make_quant(afmt), **kw, **extra)
    for step in range(STEPS):
        for i, p in enumerate(params):
            p.grad = torch.from_numpy(fx["%s/grad/%d/%d" % (name, step, i)].view(np.float32).copy()).to(device)
        opt.step()
        for i, p in enumerate(params):
            yield step, i, p, opt.state[p], fx


def check_against_fixture(name, make_quant, device="cpu", **extra):
    for step, i, p, state, fx in run_case(name, make_quant, device, **extra):
        want = fx["%s/param/%d/%d" % (name, step, i)]
        got = p.data.detach().cpu().contiguous().numpy().view(np.uint32)
        assert np.array_equal(got, want), (name, step, i, int((got != want).sum()))
        for key, val in state.items():
            if torch.is_tensor(val):
                w = fx["%s/state/%s/%d/%d" % (name, key, step, i)]
                g = val.detach().cpu().contiguous().numpy().view(np.uint32)
                assert np.array_equal(g, w), (name, key, step, i)


@pytest.mark.parametrize("name", sorted(CASES))
def test_per_tensor_path_matches_reference_optimizers(oracle, name):
    check_against_fixture(name, lambda fmt: _oracle_quant(oracle, fmt))


def test_fma_quantizer_is_recognised_only_for_nearest_float_formats():
    from mptorch_b200 import FloatingPoint
    from mptorch_b200.optim import _fusable_pair, fma_quantizer

    f = FloatingPoint(8, 7, True, True)
    q = fma_quantizer(f)
    assert _fusable_pair(q, q) == (f, f, True, True)
    assert _fusable_pair(None, q) == (None, f, True, True)
    assert _fusable_pair(None, None) == (None, None, True, True)      # plain fp32 steps fuse too
    assert _fusable_pair(lambda x, y, z: x, q) is None
    assert _fusable_pair(fma_quantizer(f, "stochastic"), q) is None
    assert _fusable_pair(fma_quantizer(FloatingPoint(8, 7, True, False)), q) is None
