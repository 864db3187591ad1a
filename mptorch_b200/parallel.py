"""Multi-GPU decomposition of the hot path (one process per GPU, ``torch.distributed``).

The reference has no distributed code; this is new.  ``float_mm`` shards by rows: rows of C are independent, every
rank runs the single-GPU kernel on its row block of A against the full B, and each output therefore sees exactly
the accumulation order of a single-GPU run.  The only exchange is the all-gather of the C row blocks, issued panel by
panel on a side stream so that it runs under the next panel's arithmetic.  With host-resident operands every rank
copies only its 1/world slice of B from host memory and the ranks assemble B over NVLink.  The data-parallel training
step needs one more exchange, the gradient all-reduce, launched bucket by bucket from autograd hooks while the
backward pass is still running; quantizer elements and softmax / layernorm rows are independent and need none.

Every collective is a plain NCCL call into local memory; no kernel reads another GPU's memory.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch
import torch.distributed as dist

__all__ = ["row_shard", "sharded_float_mm", "sharded_float_mm_streamed", "allreduce_gradients", "GradientAllReducer"]


def row_shard(M: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) rows of rank ``rank``: contiguous blocks, the first ``M % world`` ranks hold one row more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("invalid rank %d of %d" % (rank, world))
    base, extra = divmod(M, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _world(group):
    if not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def panel_bounds(block: int, panels: int) -> list[int]:
    """Row offsets that cut [0, block) into ``panels`` nearly equal panels (empty panels dropped)."""
    panels = max(1, min(int(panels), block)) if block else 1
    cuts = sorted({block * i // panels for i in range(panels + 1)})
    return cuts if len(cuts) > 1 else [0, block]


def sharded_float_mm(a_rows: torch.Tensor, b: torch.Tensor, M: int, mm_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                     group=None, gather: bool = True, panels: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """C = A x B with A given as this rank's row block (``row_shard(M, world, rank)``) and B replicated.

    ``mm_fn(a_rows, b)`` computes a local product (normally ``mptorch_b200.quant.float_mm`` with the formats bound).
    With ``gather`` the full [M, N] result is assembled on every rank (into ``out`` when given); otherwise the local
    row block is returned.  The local rows are cut into ``panels`` panels: panel i is gathered on a side stream while
    panel i + 1 is in the kernel, so only the last panel's exchange is exposed.  Rows of C are independent, so the
    bits do not depend on the panel count.  Ranks that hold one row fewer pad their last panel for the collective.
    """
    world, rank = _world(group)
    lo, hi = row_shard(M, world, rank)
    nloc = hi - lo
    if a_rows.shape[0] != nloc:
        raise ValueError("rank %d holds %d rows, expected %d" % (rank, a_rows.shape[0], nloc))
    if not gather or world == 1:
        c_rows = mm_fn(a_rows, b)
        if out is not None and gather:
            out.copy_(c_rows)
            return out
        return c_rows
    N = b.shape[-1]
    block = -(-M // world)                       # ceil: the largest row block
    starts = [row_shard(M, world, r)[0] for r in range(world)]
    counts = [row_shard(M, world, r)[1] - starts[r] for r in range(world)]
    if out is None:
        out = torch.empty(M, N, dtype=a_rows.dtype, device=a_rows.device)
    cuda = a_rows.is_cuda
    cuts = panel_bounds(block, panels)
    npan = len(cuts) - 1
    keep = []
    if cuda:
        # Each panel's kernel runs on a stream of its own, earlier panels at higher priority: the GPU fills the SMs that
        # a finishing panel leaves idle with the next panel's thread blocks, so cutting the launch into panels costs no
        # partial waves, and a panel's rows are complete (and on their way to the peers) while later panels compute.
        main = torch.cuda.current_stream(a_rows.device)
        side = torch.cuda.Stream(a_rows.device)
        low, high = _priority_range()
        compute = [torch.cuda.Stream(a_rows.device, priority=max(high, min(low, high + i))) for i in range(npan)] if npan > 1 else [main]
        side.wait_stream(main)                   # `out` may be recycled memory still in use on the main stream
        for cs in compute:
            if cs is not main:
                cs.wait_stream(main)
    for i, (plo, phi) in enumerate(zip(cuts[:-1], cuts[1:])):
        mine = a_rows[min(plo, nloc):min(phi, nloc)]
        even = all(c >= phi for c in counts)     # every rank holds the whole panel
        with (torch.cuda.stream(compute[i]) if cuda else _NullContext()):
            c_p = mm_fn(mine, b) if mine.shape[0] else torch.empty(0, N, dtype=a_rows.dtype, device=a_rows.device)
            if not even:
                padded = torch.zeros(phi - plo, N, dtype=c_p.dtype, device=c_p.device)
                padded[: c_p.shape[0]] = c_p
                c_p = padded
            if cuda:
                ready = torch.cuda.Event()
                ready.record(compute[i])
        with (torch.cuda.stream(side) if cuda else _NullContext()):
            if cuda:
                side.wait_event(ready)
            if even and npan == 1 and out.is_contiguous():
                # one panel and equal row blocks: the result is the ranks' blocks back to back, gathered in place
                dist.all_gather_into_tensor(out, c_p.contiguous(), group=group)
            elif even:
                dist.all_gather([out[starts[r] + plo: starts[r] + phi] for r in range(world)], c_p, group=group)
            else:
                pr = phi - plo
                buf = torch.empty(world * pr, N, dtype=c_p.dtype, device=c_p.device)
                dist.all_gather_into_tensor(buf, c_p, group=group)
                for r in range(world):
                    n = min(phi, counts[r]) - min(plo, counts[r])
                    if n > 0:
                        out[starts[r] + plo: starts[r] + plo + n].copy_(buf[r * pr: r * pr + n])
                keep.append(buf)
        if cuda:
            c_p.record_stream(side)
        keep.append(c_p)
    if cuda:
        main.wait_stream(side)
        for cs in compute:
            if cs is not main:
                main.wait_stream(cs)
        for t in keep:
            t.record_stream(main)
    return out


def _priority_range() -> tuple[int, int]:
    """(lowest, highest) CUDA stream priority of the current device; a numerically smaller value is a higher priority."""
    import ctypes

    from . import _cabi

    lo, hi = ctypes.c_int(0), ctypes.c_int(0)
    _cabi.call("mpt_stream_priority_range", ctypes.byref(lo), ctypes.byref(hi))
    return lo.value, hi.value


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def sharded_float_mm_streamed(a_rows: torch.Tensor, b: torch.Tensor, M: int, out: torch.Tensor | None = None, *, group=None,
                              device=None, block_rows: int = 1024, **formats) -> torch.Tensor:
    """``float_mm_streamed`` for a row-sharded A with every operand in HOST memory: ``a_rows`` is this rank's row block of
    A, ``b`` the whole of B (every rank holds the same host copy), ``out`` receives this rank's row block of C.

    Each rank copies only its 1/world slice of B's rows to its GPU; one NCCL all-gather over NVLink assembles B in
    every GPU's memory while the first block of A is still on its way from the host.  The host side of the box is read
    once for B instead of once per rank.  ``formats`` are the keyword arguments of ``float_mm``."""
    from .quant.quant_function import float_mm_streamed

    world, rank = _world(group)
    if world == 1:
        return float_mm_streamed(a_rows, b, out, device=device, block_rows=block_rows, **formats)
    if b.is_cuda or b.dtype != torch.float32 or not b.is_contiguous() or b.dim() != 2:
        raise RuntimeError("sharded_float_mm_streamed takes a contiguous float32 CPU matrix B")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    K, N = b.shape
    res = _streamed_by_panels(a_rows, b, out, dev, block_rows, group, world, rank, formats)
    if res is not None:
        return res
    klo, khi = row_shard(K, world, rank)
    kblock = -(-K // world)
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        s_b = torch.cuda.Stream(dev)
        gathered = torch.empty(world * kblock, N, device=dev)
        piece = torch.zeros(kblock, N, device=dev) if K % world else torch.empty(kblock, N, device=dev)
        s_b.wait_stream(main)
        with torch.cuda.stream(s_b):
            piece[: khi - klo].copy_(b[klo:khi], non_blocking=True)
            dist.all_gather_into_tensor(gathered, piece, group=group)
            if K % world == 0:
                bd = gathered
            else:                                  # drop the padding rows of the ranks that hold one row fewer
                bd = torch.cat([gathered[r * kblock: r * kblock + (row_shard(K, world, r)[1] - row_shard(K, world, r)[0])]
                                for r in range(world)], dim=0)
            b_ready = torch.cuda.Event()
            b_ready.record(s_b)
        res = float_mm_streamed(a_rows, bd, out, device=dev, block_rows=block_rows, b_ready=b_ready, **formats)
        for t in (gathered, piece, bd):
            t.record_stream(s_b)
    return res


def _streamed_by_panels(a_rows, b, out, dev, block_rows, group, world, rank, formats):
    """The K-panel pipeline of ``float_mm_streamed`` over the ranks (nearest rounding, K long enough, every panel a
    multiple of the world size): per panel a rank copies its columns of its rows of A and 1/world of the panel's rows
    of B from host memory, one all-gather assembles the panel of B on every GPU, and the kernel continues the rank's
    running sums.  None when the conditions do not hold (the caller then assembles B whole first)."""
    from .quant import quant_function as qf

    f = dict(man_add=23, exp_add=8, man_mul=23, exp_mul=8, rounding="nearest", fma=True, subnormals=True, saturate=True,
             compensated=False, rbits_add=0, rbits_mul=0)
    unknown = set(formats) - set(f)
    if unknown:
        raise TypeError("sharded_float_mm_streamed: unexpected arguments %s" % sorted(unknown))
    f.update(formats)
    Mr, K = a_rows.shape
    N = b.shape[1]
    panels = qf._k_panels(K) if (f["rounding"] == "nearest" and not f["compensated"] and Mr > 0 and N > 0) else None
    if panels is None or any((k1 - k0) % world for k0, k1 in panels):
        return None
    if a_rows.is_cuda or a_rows.dtype != torch.float32 or not a_rows.is_contiguous():
        raise RuntimeError("sharded_float_mm_streamed takes contiguous float32 CPU tensors")
    if out is None:
        out = torch.empty(Mr, N, dtype=torch.float32).pin_memory()
    assert out.shape == (Mr, N) and out.dtype == torch.float32 and not out.is_cuda and out.is_contiguous()
    widest = max(k1 - k0 for k0, k1 in panels)
    with torch.cuda.device(dev):
        stage = torch.empty(widest // world * N, device=dev)

        def load_b(k0, k1, bd):
            rows = (k1 - k0) // world
            mine = stage[: rows * N].view(rows, N)
            mine.copy_(b[k0 + rank * rows: k0 + (rank + 1) * rows], non_blocking=True)
            dist.all_gather_into_tensor(bd, mine, group=group)     # the copy stream waits for it

        fmt = ((f["man_add"], f["exp_add"], f["man_add"], f["exp_add"]) if f["fma"]
               else (f["man_add"], f["exp_add"], f["man_mul"], f["exp_mul"]))
        res = qf._mm_streamed_by_panels(a_rows, N, out, dev, max(1, int(block_rows)), panels, fmt, f["subnormals"], f["saturate"],
                                        f["fma"], load_b)
        stage.record_stream(torch.cuda.current_stream(dev))
    return res


# --------------------------------------------------------------------------------------------- gradients
def _flatten_reduce_scatter_back(bucket, group, world, average, nccl):
    flat = torch.cat([g.reshape(-1) for g in bucket]) if len(bucket) > 1 else bucket[0].reshape(-1)
    if average and nccl:
        dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=group)
    else:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
    if len(bucket) > 1:
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n


def _is_nccl(group) -> bool:
    try:
        return dist.get_backend(group) == "nccl"
    except Exception:
        return False


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, bucket_bytes: int = 32 << 20, average: bool = True) -> int:
    """Sum (or average) the ``.grad`` of ``params`` over the ranks with bucketed all-reduces, after the backward pass;
    returns the number of collectives issued.  Buckets are sized for launch latency, not link count: a few tens of MB
    each.  A gradient as large as a bucket is reduced in place, without the flatten and copy-back."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0
    world = dist.get_world_size(group)
    nccl = _is_nccl(group)
    grads = [p.grad for p in params if p.grad is not None]
    calls = 0
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size, calls
        if not bucket:
            return
        _flatten_reduce_scatter_back(bucket, group, world, average, nccl)
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


class GradientAllReducer:
    """Gradient all-reduce that runs UNDER the backward pass.

    Parameters are grouped into buckets in reverse registration order (roughly the order in which autograd finishes
    their gradients).  A hook on every parameter fires when its gradient has been accumulated; when the last gradient
    of a bucket arrives the bucket is flattened and all-reduced on a side stream, while the main stream carries on with
    the rest of the backward pass.  ``finish()`` (after ``loss.backward()``) reduces whatever is left (buckets whose
    parameters received no gradient this step are reduced over the gradients that did arrive) and makes the main stream
    wait for the side stream.  Gradients are averaged over the ranks unless ``average=False``.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, bucket_bytes: int = 8 << 20, average: bool = True):
        self.params = [p for p in params if p.requires_grad]
        self.group, self.average = group, average
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nccl = _is_nccl(group) if self.world > 1 else False
        self.buckets: list[list[torch.nn.Parameter]] = []
        cur, size = [], 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if cur and (size + nbytes > bucket_bytes or p.dtype != cur[0].dtype or p.device != cur[0].device):
                self.buckets.append(cur)
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            self.buckets.append(cur)
        self.bucket_of = {id(p): i for i, b in enumerate(self.buckets) for p in b}
        self.pending = [len(b) for b in self.buckets]
        self.arrived: list[set[int]] = [set() for _ in self.buckets]
        self.done = [False] * len(self.buckets)
        self.calls = 0
        self._side = {}
        self._handles = []
        if self.world > 1:
            for p in self.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        s = self._side.get(device)
        if s is None:
            s = self._side[device] = torch.cuda.Stream(device)
        return s

    def _on_grad(self, p):
        i = self.bucket_of[id(p)]
        if id(p) in self.arrived[i]:
            return
        self.arrived[i].add(id(p))
        self.pending[i] -= 1
        if self.pending[i] == 0:
            self._reduce(i)

    def _reduce(self, i):
        grads = [p.grad for p in self.buckets[i] if id(p) in self.arrived[i] and p.grad is not None]
        self.done[i] = True
        if not grads:
            return
        side = self._side_stream(grads[0].device)
        if side is None:
            _flatten_reduce_scatter_back(grads, self.group, self.world, self.average, self.nccl)
        else:
            main = torch.cuda.current_stream(grads[0].device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                _flatten_reduce_scatter_back(grads, self.group, self.world, self.average, self.nccl)
            for g in grads:
                g.record_stream(side)
        self.calls += 1

    def finish(self) -> int:
        """Reduce the buckets that are still open, wait (on the stream, not the host) for all of them, and re-arm for the
        next step.  Returns the number of collectives issued this step."""
        if self.world > 1:
            for i in range(len(self.buckets)):
                if not self.done[i]:
                    self._reduce(i)
            for dev, side in self._side.items():
                torch.cuda.current_stream(dev).wait_stream(side)
        calls = self.calls
        self.pending = [len(b) for b in self.buckets]
        self.arrived = [set() for _ in self.buckets]
        self.done = [False] * len(self.buckets)
        self.calls = 0
        return calls
