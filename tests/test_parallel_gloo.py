"""The multi-rank host logic on CPU: two gloo ranks run the row-sharded GEMM decomposition (with the oracle standing
in for the GPU kernel) and the bucketed gradient all-reduce, and must reproduce the single-rank results exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mptorch_b200.parallel import allreduce_gradients, row_shard, sharded_float_mm


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
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [16, 13])
def test_two_rank_sharded_mm_and_gradient_allreduce(tmp_path, M):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), M, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))
