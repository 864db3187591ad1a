"""The multi-rank host logic on CPU: two gloo ranks run the row-sharded GEMM decomposition (with the oracle standing
in for the GPU kernel) and the bucketed gradient all-reduce, and must reproduce the single-rank results exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mptorch_b200.parallel import GradientAllReducer, allreduce_gradients, panel_bounds, row_shard, sharded_float_mm


def test_row_shard_partitions_exactly():
    for M in (0, 1, 7, 8, 8192, 8193):
        for world in (1, 2, 3, 8):
            spans = [row_shard(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_shard(4, 2, 2)


def test_panel_bounds_cover_the_block():
    for block in (1, 2, 7, 8, 1024, 1025):
        for panels in (1, 2, 3, 4, 16, 5000):
            cuts = panel_bounds(block, panels)
            assert cuts[0] == 0 and cuts[-1] == block and all(a < b for a, b in zip(cuts, cuts[1:]))
            assert len(cuts) - 1 <= max(1, min(panels, block))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import loader

        g = torch.Generator().manual_seed(11)
        a = torch.randn(M, 24, generator=g)
        b = torch.randn(24, 10, generator=g)

        def mm_fn(x, y):   # the oracle stands in for the CUDA kernel: same per-row arithmetic
            return torch.from_numpy(loader.mm(x.numpy(), y.numpy(), 2, 5, 2, 5, True, False, False, "tile8"))

        lo, hi = row_shard(M, world, rank)
        c = sharded_float_mm(a[lo:hi].contiguous(), b, M, mm_fn)
        want = mm_fn(a, b)
        assert torch.equal(c.view(torch.int32), want.view(torch.int32)), "gathered result differs from the unsharded one"
        local = sharded_float_mm(a[lo:hi].contiguous(), b, M, mm_fn, gather=False)
        assert torch.equal(local, want[lo:hi])
        # row panels (the exchange of one panel runs under the next panel's kernel on a GPU): same bits for any panel
        # count, also when the ranks' row counts differ and the last panel is short on some ranks
        for panels in (2, 3, 5, 64):
            cp = sharded_float_mm(a[lo:hi].contiguous(), b, M, mm_fn, panels=panels)
            assert torch.equal(cp.view(torch.int32), want.view(torch.int32)), "panels=%d" % panels
        into = torch.full((M, 10), float("nan"))
        assert sharded_float_mm(a[lo:hi].contiguous(), b, M, mm_fn, panels=3, out=into) is into
        assert torch.equal(into.view(torch.int32), want.view(torch.int32))

        # gradient all-reduce: two buckets, averaged
        torch.manual_seed(100 + rank)
        params = [torch.nn.Parameter(torch.zeros(300)), torch.nn.Parameter(torch.zeros(7, 5)), torch.nn.Parameter(torch.zeros(3))]
        for p in params:
            p.grad = torch.randn_like(p)
        mine = [p.grad.clone() for p in params]
        calls = allreduce_gradients(params, bucket_bytes=1000, average=True)
        assert calls == 2
        gathered = [None] * world
        dist.all_gather_object(gathered, [m.numpy() for m in mine])
        for i, p in enumerate(params):
            mean = sum(torch.from_numpy(gathered[r][i]) for r in range(world)) / world
            assert torch.allclose(p.grad, mean, atol=1e-6)
        # the same reduction driven by autograd hooks while the backward pass runs
        torch.manual_seed(5)
        net = torch.nn.Sequential(torch.nn.Linear(6, 9), torch.nn.Tanh(), torch.nn.Linear(9, 4), torch.nn.Linear(4, 2))
        unused = torch.nn.Parameter(torch.zeros(3))          # never receives a gradient
        red = GradientAllReducer(list(net.parameters()) + [unused], bucket_bytes=200)
        assert len(red.buckets) >= 3
        for it in range(2):
            net.zero_grad(set_to_none=True)
            xin = torch.randn(5, 6, generator=torch.Generator().manual_seed(40 + 2 * rank + it))
            net(xin).pow(2).sum().backward()
            # every bucket that filled up has already been reduced inside backward()
            assert red.calls >= 1
            calls = red.finish()
            assert calls >= 3 and unused.grad is None
            # the gradients were reduced in place, so recompute every rank's own gradients for the comparison
            ref = []
            for r in range(world):
                net2 = torch.nn.Sequential(torch.nn.Linear(6, 9), torch.nn.Tanh(), torch.nn.Linear(9, 4), torch.nn.Linear(4, 2))
                net2.load_state_dict(net.state_dict())
                xr = torch.randn(5, 6, generator=torch.Generator().manual_seed(40 + 2 * r + it))
                net2(xr).pow(2).sum().backward()
                ref.append([p.grad for p in net2.parameters()])
            for i, p in enumerate(net.parameters()):
                mean = sum(ref[r][i] for r in range(world)) / world
                assert torch.allclose(p.grad, mean, atol=1e-6), (it, i)
        red.remove()
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [16, 13])
def test_two_rank_sharded_mm_and_gradient_allreduce(tmp_path, M):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), M, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))
