"""The GEMM entry point that allocates nothing (mpt_float_mm_nearest_static) against the regular one.

It exists for callers that cannot allocate device memory and so cannot supply the GEMM's workspace: the operand
statistics then live in an array built into the library.  The two entry points must give identical bits.  The
check runs twice in a row with different data, because every call reuses the same built-in array: the first call
pushes it through the "huge values" state, the second must not see any of that.  This file sorts last so that a
run stopping at the first failure has already covered everything else.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(a, b, order, fmt_add=(2, 5), fmt_mul=(2, 5), compensated=0):
    from mptorch_b200 import _cabi

    batch, M, K = a.shape
    N = b.shape[2]
    dev = a.device
    c_ws = torch.full((batch, M, N), float("nan"), device=dev)
    c_st = torch.full((batch, M, N), float("nan"), device=dev)
    ws = _cabi.mm_workspace(dev, batch)
    args = (batch, M, N, K, fmt_add[0], fmt_add[1], fmt_mul[0], fmt_mul[1], 1, 0, compensated, order)
    _cabi.call("mpt_float_mm_nearest", _cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(c_ws), *args, _cabi.ptr(ws), ws.numel(),
               _cabi.stream_ptr(dev))
    _cabi.call("mpt_float_mm_nearest_static", _cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(c_st), *args, _cabi.stream_ptr(dev))
    torch.cuda.synchronize(dev)
    return c_ws, c_st


def test_static_scratch_entry_point_matches_workspace_entry_point():
    g = torch.Generator(device="cuda").manual_seed(2026)
    for order in (1, 0):
        # first call: one batch entry with huge values, so the array holds "exact path" statistics afterwards
        a = torch.randn(3, 70, 56, device="cuda", generator=g)
        b = torch.randn(3, 56, 44, device="cuda", generator=g)
        a[1] *= 1000.0
        c_ws, c_st = _run_both(a, b, order)
        assert torch.equal(c_ws.view(torch.int32), c_st.view(torch.int32))
        assert not torch.isnan(c_st[0]).any()
        # second call, straight after, ordinary values and another shape: must not inherit anything
        a2 = torch.randn(5, 33, 64, device="cuda", generator=g)
        b2 = torch.randn(5, 64, 129, device="cuda", generator=g)
        c_ws2, c_st2 = _run_both(a2, b2, order, (10, 5), (3, 4))
        assert torch.equal(c_ws2.view(torch.int32), c_st2.view(torch.int32))
        assert torch.isfinite(c_st2).all()


def test_static_scratch_full_batch_compensated_and_empty_sums():
    """The largest batch the built-in array holds (every record written and read), the Kahan-compensated variant,
    and the early returns for K = 0 and M = 0, all through the entry point that allocates nothing."""
    g = torch.Generator(device="cuda").manual_seed(2027)
    a = torch.randn(4096, 5, 9, device="cuda", generator=g)
    b = torch.randn(4096, 9, 6, device="cuda", generator=g)
    a[4095] *= 3000.0                                     # the last record must be its own
    c_ws, c_st = _run_both(a, b, 1)
    assert torch.equal(c_ws.view(torch.int32), c_st.view(torch.int32))
    a = torch.randn(2, 40, 72, device="cuda", generator=g)
    b = torch.randn(2, 72, 24, device="cuda", generator=g)
    for order in (1, 0):
        c_ws, c_st = _run_both(a, b, order, (10, 5), (3, 4), compensated=1)
        assert torch.equal(c_ws.view(torch.int32), c_st.view(torch.int32)) and torch.isfinite(c_st).all()
    c_ws, c_st = _run_both(torch.zeros(2, 7, 0, device="cuda"), torch.zeros(2, 0, 5, device="cuda"), 1)
    assert torch.equal(c_st, torch.zeros(2, 7, 5, device="cuda")) and torch.equal(c_ws, c_st)
    c_ws, c_st = _run_both(torch.zeros(2, 0, 3, device="cuda"), torch.zeros(2, 3, 5, device="cuda"), 1)
    assert c_st.numel() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_static_scratch_address_is_per_device():
    """The array's address is looked up once per device: a call on cuda:0 followed by one on cuda:1 must each use
    their own GPU's copy."""
    from mptorch_b200 import _cabi

    for d in (0, 1, 0):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            g = torch.Generator(device=dev).manual_seed(2028 + d)
            a = torch.randn(2, 30, 40, device=dev, generator=g)
            b = torch.randn(2, 40, 20, device=dev, generator=g)
            c_ws, c_st = _run_both(a, b, 1)
            assert torch.equal(c_ws.view(torch.int32), c_st.view(torch.int32)), d


def test_static_scratch_entry_point_rejects_oversized_batch():
    from mptorch_b200 import _cabi

    a = torch.zeros(4097, 1, 1, device="cuda")
    b = torch.zeros(4097, 1, 1, device="cuda")
    c = torch.zeros(4097, 1, 1, device="cuda")
    with pytest.raises(_cabi.MptError, match="exceeds the 4096 entries"):
        _cabi.call("mpt_float_mm_nearest_static", _cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(c), 4097, 1, 1, 1, 2, 5, 2, 5, 1, 0, 0,
                   1, _cabi.stream_ptr(c.device))
