"""Multi-GPU decomposition of the hot path (one process per GPU, ``torch.distributed``).

The reference has no distributed code; this is new.  ``float_mm`` shards by rows: rows of C are independent, every
rank runs the single-GPU kernel on its row block of A against the full B, and each output therefore sees exactly
the accumulation order of a single-GPU run.  The only exchange is the all-gather of the C row blocks.  The
data-parallel training step needs one more exchange, the gradient all-reduce; quantizer elements and softmax /
layernorm rows are independent and need none.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch
import torch.distributed as dist

__all__ = ["row_shard", "sharded_float_mm", "allreduce_gradients"]


def row_shard(M: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) rows of rank ``rank``: contiguous blocks, the first ``M % world`` ranks hold one row more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("invalid rank %d of %d" % (rank, world))
    base, extra = divmod(M, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sharded_float_mm(a_rows: torch.Tensor, b: torch.Tensor, M: int, mm_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                     group=None, gather: bool = True) -> torch.Tensor:
    """C = A x B with A given as this rank's row block (``row_shard(M, world, rank)``) and B replicated.

    ``mm_fn(a_rows, b)`` computes the local product (normally ``mptorch_b200.quant.float_mm`` with the formats
    bound).  With ``gather`` the full [M, N] result is assembled on every rank by one all-gather; otherwise the local
    row block is returned.  Uneven row counts are padded to the largest block for the collective and trimmed after.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lo, hi = row_shard(M, world, rank)
    if a_rows.shape[0] != hi - lo:
        raise ValueError("rank %d holds %d rows, expected %d" % (rank, a_rows.shape[0], hi - lo))
    c_rows = mm_fn(a_rows, b)
    if not gather or world == 1:
        return c_rows
    N = c_rows.shape[1]
    block = -(-M // world)                       # ceil: the largest row block
    if M % world == 0:
        out = torch.empty(M, N, dtype=c_rows.dtype, device=c_rows.device)
        dist.all_gather_into_tensor(out, c_rows.contiguous(), group=group)
        return out
    padded = torch.zeros(block, N, dtype=c_rows.dtype, device=c_rows.device)
    padded[: hi - lo] = c_rows
    buf = torch.empty(world * block, N, dtype=c_rows.dtype, device=c_rows.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    parts = []
    for r in range(world):
        rlo, rhi = row_shard(M, world, r)
        parts.append(buf[r * block: r * block + (rhi - rlo)])
    return torch.cat(parts, dim=0)


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, bucket_bytes: int = 32 << 20, average: bool = True) -> int:
    """Sum (or average) the ``.grad`` of ``params`` over the ranks with bucketed all-reduces; returns the number of
    collectives issued.  Buckets are sized for launch latency, not link count: a few tens of MB each."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0
    world = dist.get_world_size(group)
    grads = [p.grad for p in params if p.grad is not None]
    calls = 0
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size, calls
        if not bucket:
            return
        flat = torch.cat([g.reshape(-1) for g in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n
        calls += 1
        bucket, size = [], 0

    for g in grads:
        nbytes = g.numel() * g.element_size()
        if bucket and (size + nbytes > bucket_bytes or g.dtype != bucket[0].dtype):
            flush()
        bucket.append(g)
        size += nbytes
    flush()
    return calls
