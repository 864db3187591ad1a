"""Two NCCL ranks on two GPUs of one box (skipped when fewer are visible): the row-sharded GEMM with its panel-wise
all-gather, the host-operand form in which the ranks assemble B from slices, and the hook-driven gradient all-reduce
must reproduce the single-GPU results bit for bit (the GEMM) or to rounding (the averaged gradients)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

KW = dict(man_add=10, exp_add=5, man_mul=3, exp_mul=4, rounding="nearest", fma=False, subnormals=True, saturate=False)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import mptorch_b200.quant as q
        from mptorch_b200.parallel import GradientAllReducer, row_shard, sharded_float_mm, sharded_float_mm_streamed

        # the third case is long enough along K for the K-panel pipeline (a panel of B assembled per all-gather), the
        # fourth has a last panel that does not divide by the world size and takes the whole-B path
        for M, K, N in ((1024, 512, 640), (1001, 333, 520), (520, 2048, 264), (300, 1801, 136)):
            g = torch.Generator().manual_seed(7)
            a = torch.randn(M, K, generator=g)
            b = torch.randn(K, N, generator=g)
            want = q.float_mm(a.to(dev), b.to(dev), **KW)
            lo, hi = row_shard(M, world, rank)
            mine = a[lo:hi].contiguous().to(dev)
            for panels in (1, 3, 4):
                got = sharded_float_mm(mine, b.to(dev), M, lambda x, y: q.float_mm(x, y, **KW), panels=panels)
                assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (M, panels)
            ah, bh = a[lo:hi].contiguous().pin_memory(), b.pin_memory()
            out = sharded_float_mm_streamed(ah, bh, M, block_rows=200, **KW)
            assert torch.equal(out.view(torch.int32), want[lo:hi].cpu().view(torch.int32)), M

        torch.manual_seed(3)
        net = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 64), torch.nn.Linear(64, 8)).to(dev)
        red = GradientAllReducer(net.parameters(), bucket_bytes=40000)
        xs = [torch.randn(32, 64, generator=torch.Generator().manual_seed(50 + r)).to(dev) for r in range(world)]
        net(xs[rank]).pow(2).mean().backward()
        assert red.finish() >= 2
        got = [p.grad.clone() for p in net.parameters()]
        red.remove()
        mean = None
        for r in range(world):
            net.zero_grad(set_to_none=True)
            net(xs[r]).pow(2).mean().backward()
            gr = [p.grad.clone() for p in net.parameters()]
            mean = gr if mean is None else [m + x for m, x in zip(mean, gr)]
        for gg, m in zip(got, mean):
            assert torch.allclose(gg, m / world, rtol=1e-5, atol=1e-7)
        torch.cuda.synchronize(dev)
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_gemm_and_gradient_allreduce(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))
