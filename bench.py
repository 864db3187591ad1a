#!/usr/bin/env python
"""Headline benchmark: per-MAC rounded float_mm, 8192 x 8192 x 8192, e5m2 multiply and add, round to
nearest (the headline metric "float_mm GMAC/s"), plus the elementwise quantizer's HBM throughput.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one float_mm over the whole problem.  With N > 1 (launched by torch.distributed.run, one rank
per GPU) the M rows of A and C are split across ranks, B is replicated, and every step ends with an
all-gather of the C row blocks, so the total work is fixed ("strong" scaling).  Prints ONE JSON line on
rank 0.  Inputs (512 MiB) are larger than L2, so no flush is needed between iterations.

`--impl reference` times the reference's own CPU implementation (oracle/_ref/quant_cpu, the unmodified
reference extension, when it has been built; otherwise the C restatement in oracle/) on the host cores on a
bounded row sample of the same problem.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZE = 8192
FMT = dict(man_add=2, exp_add=5, man_mul=2, exp_mul=5, subnormals=True, saturate=False)
# The roofline of the GEMM kernel is built from counters of an ncu capture of that kernel: issued thread-instructions
# per MAC (smsp__inst_executed.sum x 32 / MACs), the share of them on the half-rate ALU pipe, and the DRAM traffic of one
# launch at the bench size.  They live in profiles/mm_kernel_counters.json together with the command that produced them
# and the git blob hashes of the kernel sources they were taken at; when the sources have changed since, the bench line
# says so ("constants_stale") instead of silently reporting an old roofline.
COUNTERS_PATH = os.path.join(ROOT, "profiles", "mm_kernel_counters.json")
KERNEL_SOURCES = ("mptorch_b200/csrc/gemm_kernel.cuh", "mptorch_b200/csrc/cast.cuh")


def git_blob_hash(path: str) -> str:
    import hashlib

    data = open(path, "rb").read()
    return hashlib.sha1(b"blob %d\0" % len(data) + data).hexdigest()


def load_counters() -> dict:
    c = json.load(open(COUNTERS_PATH))
    now = {src: git_blob_hash(os.path.join(ROOT, src)) for src in KERNEL_SOURCES}
    c["constants_stale"] = any(c.get("source_blobs", {}).get(src) != h for src, h in now.items())
    return c


def record_counters(per_mac_csv: str, per_mac_size: int, traffic_csv: str | None, note: str) -> dict:
    """Rebuild profiles/mm_kernel_counters.json from ncu `--csv` logs of the GEMM kernel: `per_mac_csv` holds
    smsp__inst_executed.sum, sm__inst_executed_pipe_alu.sum, sm__inst_executed_pipe_fma.sum (and anything else asked for) of
    one mm_kernel launch at M = N = K = `per_mac_size`; `traffic_csv` dram__bytes_read.sum / dram__bytes_write.sum of one
    launch at 8192^3.  The hashes of the kernel sources as they are now are stored beside the numbers."""
    import csv

    def metrics(path):
        out = {}
        rows = [r for r in csv.reader(l for l in open(path) if l.startswith('"'))]
        head = rows[0]
        ik, im, iv, iu = head.index("Kernel Name"), head.index("Metric Name"), head.index("Metric Value"), head.index("Metric Unit")
        for r in rows[1:]:
            if "mm_kernel" in r[ik] and r[im] not in out:
                v = float(r[iv].replace(",", ""))
                unit = r[iu].lower()
                v *= {"kbyte": 1e3, "mbyte": 1e6, "gbyte": 1e9}.get(unit, 1.0)
                out[r[im]] = v
                out["kernel"] = r[ik]
        return out

    m = metrics(per_mac_csv)
    macs = float(per_mac_size) ** 3
    old = json.load(open(COUNTERS_PATH)) if os.path.exists(COUNTERS_PATH) else {}
    c = dict(old)
    c["kernel"] = m.pop("kernel", old.get("kernel"))
    c["captured_at"] = note
    c["metrics"] = {k: v for k, v in m.items()}
    c["metrics"]["macs"] = macs
    c["inst_per_mac"] = round(m["smsp__inst_executed.sum"] * 32 / macs, 3)
    c["alu_inst_per_mac"] = round(m["sm__inst_executed_pipe_alu.sum"] * 32 / macs, 3)
    if "sm__inst_executed_pipe_fma.sum" in m:
        # fp32 instructions of this kernel's fast path are all packed fp32x2 (FMUL2 / FADD2 / FFMA2)
        c["packed_fp_inst_per_mac"] = round(m["sm__inst_executed_pipe_fma.sum"] * 32 / macs, 3)
    if traffic_csv:
        t = metrics(traffic_csv)
        c["metrics"]["dram__bytes_read.sum_8192cubed"] = t["dram__bytes_read.sum"]
        c["metrics"]["dram__bytes_write.sum_8192cubed"] = t["dram__bytes_write.sum"]
        c["dram_bytes_per_launch_8192cubed"] = int(t["dram__bytes_read.sum"] + t["dram__bytes_write.sum"])
    c["source_blobs"] = {src: git_blob_hash(os.path.join(ROOT, src)) for src in KERNEL_SOURCES}
    json.dump(c, open(COUNTERS_PATH, "w"), indent=1)
    return c


METRIC = "float_mm GMAC/s (8192^3, e5m2 RN)"
WORKLOAD = "float_mm 8192x8192x8192, mul e5m2 / add e5m2, nearest, subnormals, no saturate"


def config_for(size: int) -> dict:
    """The same dictionary from both arms (the reference CPU arm and the GPU arm) for the same command line."""
    wl = WORKLOAD if size == SIZE else WORKLOAD.replace("8192x8192x8192", "%dx%dx%d" % (size, size, size))
    return {"workload": wl, "l2": "operands (512 MiB at 8192^3) exceed L2, no flush between iterations"}


# ----------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 7:
                    continue
                try:
                    sm.append(float(p[0])); mx.append(float(p[1])); power.append(float(p[2]))
                except ValueError:
                    continue
                for nm, v in zip(names, p[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # samples under load: the upper half by power draw
            order = sorted(range(len(sm)), key=lambda i: power[i])
            load = [sm[i] for i in order[len(order) // 2:]]
            out = {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm), "power_w_max": max(power)}
        return out


# ----------------------------------------------------------------------------------- CPU arm
def _cpu_worker(args):
    """Times the reference CPU float_mm on `rows` rows of the 8192-wide problem (one process, one core)."""
    rows, k, n, seed, use_ref = args
    import numpy as np
    import torch

    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(rows, k, generator=g)
    b = torch.randn(k, n, generator=g)
    if use_ref:
        from oracle.build_ref import load_ref

        ref = load_ref("quant_cpu")
        c = torch.zeros(rows, n)
        t0 = time.perf_counter()
        ref.float_quantize_nearest_mm(a, b, c, rows, n, k, FMT["man_add"], FMT["exp_add"], FMT["man_mul"],
                                      FMT["exp_mul"], True, False, False)
        return time.perf_counter() - t0
    os.environ["OMP_NUM_THREADS"] = "1"
    from oracle import loader

    an, bn = a.numpy(), b.numpy()
    t0 = time.perf_counter()
    loader.mm(an, bn, FMT["man_add"], FMT["exp_add"], FMT["man_mul"], FMT["exp_mul"], True, False, False, "seq")
    return time.perf_counter() - t0


def cpu_baseline(rows_per_core: int = 1, cores: int | None = None) -> dict:
    """All host cores, one process each (the reference CPU path is single threaded), each on its own rows."""
    import multiprocessing as mp

    from oracle.build_ref import load_ref

    cores = cores or os.cpu_count() or 1
    use_ref = load_ref("quant_cpu") is not None
    ctx = mp.get_context("spawn")
    t0 = time.perf_counter()
    with ctx.Pool(cores) as pool:
        times = pool.map(_cpu_worker, [(rows_per_core, SIZE, SIZE, 100 + i, use_ref) for i in range(cores)])
    wall = max(times)
    macs = cores * rows_per_core * SIZE * SIZE
    return {"value": macs / wall / 1e9, "unit": "GMAC/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": "%d rows of the 8192x8192x8192 problem per core (%d MACs total), sequential K order; "
                      "slowest core %.1f s" % (rows_per_core, macs, wall),
            "pool_wall_s": time.perf_counter() - t0}


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    res = []
    for _ in range(max(0, args.warmup)):
        cpu_baseline(1)
    for _ in range(max(1, args.steps)):
        res.append(cpu_baseline(1))
    # whole-run throughput over the K steps: total MACs / total time of the slowest core per step
    steps = len(res)
    best = dict(res[0])
    best["value"] = sum(r["value"] for r in res) / steps
    ms = statistics.mean(r["pool_wall_s"] for r in res) * 1e3
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": "GMAC/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": max(0, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (each multiply and add rounded to e5m2)", "data": "synthetic",
            "config": config_for(SIZE), "accum_order": "seq",
            "notes": "reference CPU extension (quant_cpu, sequential K order, single threaded) on one row of the problem per "
                     "host core, all cores at once; the MAC count per row is that of the GPU arm",
            "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": best["value"], "unit": "GMAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------------- HBM-bound kernels
def _ref_cuda():
    """The reference's own CUDA extension built for sm_100a (oracle/_ref/quant_cuda), or None when it is not there."""
    try:
        from oracle.build_ref import load_ref

        return load_ref("quant_cuda")
    except Exception:
        return None


def kernels_legs(dev, steps: int, warmup: int, scale: float = 1.0, with_reference: bool = True) -> dict:
    """Throughput of the HBM-bound kernels at the benchmark sizes: MX / NVFP4 on 16384 x 16384 (config 3), softmax rows of
    1024 and layernorm rows of 768 at the config 5 tensor sizes (`scale` shrinks the row counts).  Beside each figure that
    has a counterpart, the reference's own CUDA kernel (unmodified sources built for sm_100a) is timed on the same tensor."""
    import torch

    import mptorch_b200.quant as q

    g = torch.Generator(device=dev).manual_seed(7)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    out = {}
    ref = _ref_cuda() if with_reference else None

    def clock(fn):
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / steps

    def timed(name, fn, nbytes, ref_fn=None):
        ms = clock(fn)
        out[name] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm_peak, 3),
                     "algorithmic_bytes": nbytes}
        if ref is not None and ref_fn is not None:
            try:
                rms = clock(ref_fn)
                out[name]["reference_cuda_ms"] = round(rms, 4)
                out[name]["speedup_vs_reference_cuda"] = round(rms / ms, 2)
            except Exception as ex:
                out[name]["reference_cuda_error"] = repr(ex)[:120]

    n = int(16384 * scale)
    x = torch.randn(n, 16384, device=dev, generator=g) * (10.0 ** (torch.rand(n, 1, device=dev, generator=g) * 6 - 3))
    e = x.numel()
    timed("mxfp8_e4m3_block32", lambda: q.mx_quantize(x, "e4m3", 32), 8 * e)
    timed("mxfp4_e2m1_block32", lambda: q.mx_quantize(x, "e2m1", 32), 8 * e)
    gs = float(x.abs().max().item() / (448.0 * 6.0))
    timed("nvfp4_given_tensor_scale", lambda: q.nvfp4_quantize(x, gs), 8 * e)
    timed("nvfp4_computed_tensor_scale", lambda: q.nvfp4_quantize(x), 12 * e)
    del x
    rows = int(8 * 12 * 1024 * scale)
    att = torch.randn(rows, 1024, device=dev, generator=g) * 3
    gy = torch.randn(rows, 1024, device=dev, generator=g)
    ro = torch.zeros_like(att) if ref is not None else None
    e = att.numel()
    timed("softmax_fwd_e5m10_rows1024", lambda: q.float_softmax_forward(att, -1, 10, 5, 10, 5, 10, 5), 8 * e,
          lambda: ref.float_quantize_nearest_softmax_forward(att, ro, -1, 10, 5, 10, 5, 10, 5, True, False))
    timed("softmax_fwd_e8m7_rows1024", lambda: q.float_softmax_forward(att, -1, 7, 8, 7, 8, 7, 8), 8 * e,
          lambda: ref.float_quantize_nearest_softmax_forward(att, ro, -1, 7, 8, 7, 8, 7, 8, True, False))
    timed("softmax_lse_fwd_e5m10_rows1024", lambda: q.float_softmax_lse_forward(att, -1, 10, 5, 10, 5), 8 * e,
          lambda: ref.float_quantize_nearest_softmax_lse_forward(att, ro, -1, 10, 5, 10, 5, True, False))
    y = q.float_softmax_forward(att, -1, 10, 5, 10, 5, 10, 5)
    timed("softmax_bwd_e5m10_rows1024", lambda: q.float_softmax_backward(y, gy, -1, 10, 5, 10, 5), 12 * e,
          lambda: ref.float_quantize_nearest_softmax_backward(y, gy, ro, -1, 10, 5, 10, 5, True, False))
    del att, gy, y, ro
    rows = int(8192 * 8 * scale)      # 8 layernorm-sized tensors' worth of rows so the tensor exceeds L2
    xl = torch.randn(rows, 768, device=dev, generator=g)
    gl = torch.randn(rows, 768, device=dev, generator=g)
    w, b = torch.randn(768, device=dev, generator=g), torch.randn(768, device=dev, generator=g)
    e = xl.numel()
    if ref is not None:
        ry, rm, rr = torch.zeros_like(xl), torch.zeros(rows, device=dev), torch.zeros(rows, device=dev)
        rgi, rgg, rgb = torch.zeros_like(xl), torch.zeros(768, device=dev), torch.zeros(768, device=dev)
    timed("layernorm_fwd_e5m10_rows768", lambda: q.float_layernorm_forward(xl, w, b, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5), 8 * e,
          lambda: ref.float_quantize_layernorm_forward(xl, w, b, ry, rm, rr, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, True, False))
    timed("layernorm_fwd_e8m7_rows768", lambda: q.float_layernorm_forward(xl, w, b, 1e-5, [-1], 7, 8, 7, 8, 7, 8, 7, 8), 8 * e,
          lambda: ref.float_quantize_layernorm_forward(xl, w, b, ry, rm, rr, 1e-5, [-1], 7, 8, 7, 8, 7, 8, 7, 8, True, False))
    _, mean, rstd = q.float_layernorm_forward(xl, w, b, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5)
    timed("layernorm_bwd_e5m10_rows768", lambda: q.float_layernorm_backward(xl, gl, w, b, mean, rstd, [-1], 10, 5, 10, 5, 10, 5), 20 * e,
          lambda: ref.float_quantize_layernorm_backward(xl, gl, w, b, mean, rstd, rgi, rgg, rgb, [-1], 10, 5, 10, 5, 10, 5, True, False))
    # the same backward pass at the config 5 tensor size (8192 rows): the parameter gradients are a chain over the rows
    r5 = max(1, int(8192 * scale))
    timed("layernorm_bwd_e5m10_rows768_config5_size", lambda: q.float_layernorm_backward(xl[:r5], gl[:r5], w, b, mean[:r5], rstd[:r5], [-1], 10, 5, 10, 5, 10, 5),
          20 * r5 * 768,
          lambda: ref.float_quantize_layernorm_backward(xl[:r5], gl[:r5], w, b, mean[:r5], rstd[:r5], rgi[:r5], rgg, rgb, [-1], 10, 5, 10, 5, 10, 5, True, False))
    del xl, gl
    # QConv2d forward (ResNet-style 3x3 layer, 64 -> 64 channels, 56 x 56, batch 64): implicit GEMM vs unfold + GEMM
    import mptorch_b200.quant.modules as qmod
    from mptorch_b200 import FloatingPoint

    nb = max(1, int(64 * scale))
    fmt = q.QAffineFormats(fwd_mac=(FloatingPoint(5, 10, True, False), FloatingPoint(4, 3, True, False)),
                           bwd_mac=(FloatingPoint(5, 10, True, False), FloatingPoint(4, 3, True, False)))
    conv = q.QConv2d(64, 64, 3, fmt, padding=1).to(dev)
    xc = torch.randn(nb, 64, 56, 56, device=dev, generator=g)
    conv_macs = nb * 56 * 56 * 64 * 64 * 9
    with torch.no_grad():
        timed("qconv2d_fwd_implicit_gemm", lambda: conv(xc), 0)
        eligible = qmod.implicit_conv_eligible
        qmod.implicit_conv_eligible = lambda f, t: False
        try:
            timed("qconv2d_fwd_unfold_gemm", lambda: conv(xc), 0)
        finally:
            qmod.implicit_conv_eligible = eligible
    for k in ("qconv2d_fwd_implicit_gemm", "qconv2d_fwd_unfold_gemm"):
        out[k] = {"ms": out[k]["ms"], "gmacs": round(conv_macs / out[k]["ms"] / 1e6, 1)}
    # the same layer forward + backward: input gradient through the GEMM and F.fold, weight gradient as an implicit GEMM
    # (no unfolded input) against the unfold + GEMM composition
    import mptorch_b200.quant.functional as qfun

    xg = xc.clone().requires_grad_(True)
    gy = torch.randn(nb, 64, 56, 56, device=dev, generator=g)

    def conv_step():
        xg.grad = None
        conv.weight.grad = None
        conv(xg).backward(gy)

    timed("qconv2d_fwd_bwd_implicit_wgrad", conv_step, 0)
    wgrad_ok = qfun.implicit_wgrad_eligible
    qfun.implicit_wgrad_eligible = lambda f: False
    try:
        timed("qconv2d_fwd_bwd_unfold_wgrad", conv_step, 0)
    finally:
        qfun.implicit_wgrad_eligible = wgrad_ok
    for k in ("qconv2d_fwd_bwd_implicit_wgrad", "qconv2d_fwd_bwd_unfold_wgrad"):
        out[k] = {"ms": out[k]["ms"], "gmacs": round(3 * conv_macs / out[k]["ms"] / 1e6, 1)}
    del xc, conv, xg, gy
    # fused optimizer steps over the parameter tensors of a GPT-2-small (embeddings + one block, 46.5 M parameters):
    # QSGD with momentum and QAdamW, momentum / moments and weights in e8m7 with the Kahan compensation buffer
    from mptorch_b200.optim import QAdamW, QSGD, fma_quantizer

    shapes = [(50257, 768), (1024, 768), (768,), (768,), (2304, 768), (2304,), (768, 768), (768,), (768,), (768,), (3072, 768), (3072,),
              (768, 3072), (768,)]
    if scale < 1.0:
        shapes[0] = (max(1024, int(50257 * scale)), 768)
    params = [torch.nn.Parameter(torch.randn(*s, device=dev, generator=g)) for s in shapes]
    for p_ in params:
        p_.grad = torch.randn(p_.shape, device=dev, generator=g) * 0.01
    npar = sum(p_.numel() for p_ in params)
    accq = fma_quantizer(FloatingPoint(8, 7, True, True))
    sgd = QSGD(params, lr=1e-3, momentum=0.9, momentum_quant=accq, acc_quant=accq, compensated=True)
    sgd.step()                                   # creates the momentum buffers
    timed("qsgd_fused_step_e8m7_compensated", sgd.step, 32 * npar)          # weight, gradient, momentum, compensation read; all but the gradient written
    adam = QAdamW(params, lr=1e-3, momentum_quant=accq, acc_quant=accq, compensated=True)
    adam.step()
    timed("qadamw_fused_step_e8m7_compensated", adam.step, 36 * npar)
    return {"hbm_peak_gbs": hbm_peak, "unit": "GB/s at algorithmic bytes", "kernels": out}


def run_kernels(args) -> int:
    import torch

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    res = kernels_legs(dev, args.steps, args.warmup, args.size / 8192.0)
    print(json.dumps({"metric": "HBM-bound kernels, GB/s at algorithmic bytes", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, **res}))
    return 0


# ----------------------------------------------------------------------------------- config 4: GEMM sweep
C4_PAIRS = {"mul e4m3 / add e5m10": (10, 5, 3, 4), "mul e5m2 / add e8m7": (7, 8, 2, 5), "mul e5m2 / add e5m2": (2, 5, 2, 5)}


def c4_sweep(dev, sizes=(2048, 4096, 8192), variants=True) -> dict:
    """float_mm at M = N = K in `sizes` for the three format pairs of benchmark config 4, both accumulation orders, the
    fused multiply-add form, and (at 4096) the Kahan-compensated and stochastic variants.  CUDA events around a loop of
    calls through the reference-named backend functions; operands of 2048^3 (48 MiB) fit L2, the larger ones do not."""
    import torch

    from mptorch_b200 import backend as be

    g = torch.Generator(device=dev).manual_seed(4)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps

    rows = []
    for S in sizes:
        a = torch.randn(S, S, device=dev, generator=g)
        b = torch.randn(S, S, device=dev, generator=g)
        c = torch.empty(S, S, device=dev)
        reps = 20 if S <= 2048 else (6 if S <= 4096 else 3)

        def rec(name, order, form, ms):
            rows.append({"size": S, "formats": name, "order": order, "form": form, "ms": round(ms, 3),
                         "tmacs": round(float(S) ** 3 / ms / 1e9, 3)})

        for name, (ma, ea, mm, em) in C4_PAIRS.items():
            for order in ("cuda", "seq"):
                rec(name, order, "mul+add", timed(lambda: be.float_quantize_nearest_mm(a, b, c, S, S, S, ma, ea, mm, em, True, False, False, order=order), reps))
            rec(name, "cuda", "fma (add format)", timed(lambda: be.float_quantize_nearest_mm_fma(a, b, c, S, S, S, ma, ea, True, False, False, order="cuda"), reps))
        if variants and (S == 4096 or len(sizes) == 1):
            for name, (ma, ea, mm, em) in C4_PAIRS.items():
                rec(name, "cuda", "kahan", timed(lambda: be.float_quantize_nearest_mm(a, b, c, S, S, S, ma, ea, mm, em, True, False, True, order="cuda"), 3))
                rec(name, "cuda", "stochastic", timed(lambda: be.float_quantize_stochastic_mm(a, b, c, S, S, S, ma, ea, 23 - ma, mm, em, 23 - mm, True, False, seed=5), 3))
            rec("fma e5m10", "cuda", "kahan fma", timed(lambda: be.float_quantize_nearest_mm_fma(a, b, c, S, S, S, 10, 5, True, False, True, order="cuda"), 3))
            rec("fma e5m10", "cuda", "stochastic fma", timed(lambda: be.float_quantize_stochastic_mm_fma(a, b, c, S, S, S, 10, 5, 13, True, False, seed=5), 3))
        if variants and S == min(sizes):
            # formats outside the three pairs, each with the reference's own CUDA kernel on the same operands: fp32
            # accumulation (a format that rounds nothing), and formats only the exact casters cover
            ref = _ref_cuda()
            r = torch.empty(S, S, device=dev)

            def both(name, form, ours, theirs):
                ms = timed(ours, 5)
                row = {"size": S, "formats": name, "order": "cuda", "form": form, "ms": round(ms, 3), "tmacs": round(float(S) ** 3 / ms / 1e9, 3)}
                if ref is not None:
                    try:
                        rms = timed(theirs, 3)
                        row["reference_cuda_ms"] = round(rms, 3)
                        row["same_bits_as_reference_cuda"] = bool(((c.view(torch.int32) == r.view(torch.int32)) | (c.isnan() & r.isnan())).all())
                    except Exception as ex:
                        row["reference_cuda_error"] = repr(ex)[:120]
                rows.append(row)

            both("mul e4m3 / add fp32", "mul+add", lambda: be.float_quantize_nearest_mm(a, b, c, S, S, S, 23, 8, 3, 4, True, False, False, order="cuda"),
                 lambda: ref.float_quantize_nearest_mm(a, b, r, S, S, S, 23, 8, 3, 4, True, False, False))
            both("mul fp32 / add fp32", "mul+add", lambda: be.float_quantize_nearest_mm(a, b, c, S, S, S, 23, 8, 23, 8, True, False, False, order="cuda"),
                 lambda: ref.float_quantize_nearest_mm(a, b, r, S, S, S, 23, 8, 23, 8, True, False, False))
            both("mul e5m2 / add e5m2, no subnormals", "mul+add (settling rounding)",
                 lambda: be.float_quantize_nearest_mm(a, b, c, S, S, S, 2, 5, 2, 5, False, False, False, order="cuda"),
                 lambda: ref.float_quantize_nearest_mm(a, b, r, S, S, S, 2, 5, 2, 5, False, False, False))
            both("supernormal e8m7, 1 binade each side", "mul+add (exact casters)",
                 lambda: be.superfp_quantize_nearest_mm(a, b, c, S, S, S, 7, 8, 7, 8, 1, 1, 1, 1, True, order="cuda"),
                 lambda: ref.superfp_quantize_nearest_mm(a, b, r, S, S, S, 7, 8, 7, 8, 1, 1, 1, 1, True))
            both("supernormal e8m7, 1 binade each side", "fma (exact casters)",
                 lambda: be.superfp_quantize_nearest_mm_fma(a, b, c, S, S, S, 7, 8, 1, 1, True, order="cuda"),
                 lambda: ref.superfp_quantize_nearest_mm_fma(a, b, r, S, S, S, 7, 8, 1, 1, True))
            del r
        del a, b, c
    return {"rows": rows}


def formats_sweep(dev) -> dict:
    """The paths outside the three benchmark format pairs, each beside the reference's own CUDA kernel (unmodified
    sources built for sm_100a) on the same tensors, with a bit comparison: float formats WITHOUT subnormals (the
    reference's FloatingPoint default) through the quantizer, the GEMM (plain, compensated, stochastic), softmax,
    layernorm and the convolution layer; products whose operands rule the range-checked path out; and the block
    training step in formats without subnormals."""
    import torch

    import mptorch_b200.quant as q
    import mptorch_b200.quant.modules as qmod
    from mptorch_b200 import FloatingPoint
    from mptorch_b200 import backend as be
    from mptorch_b200.gpt2_block import BlockConfig, QTinyGPT, default_formats

    ref = _ref_cuda()
    g = torch.Generator(device=dev).manual_seed(1)

    def clock(fn, n=3):
        fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / n

    def same(x, y):
        return bool(((x.view(torch.int32) == y.view(torch.int32)) | (x.isnan() & y.isnan())).all())

    rows = []

    def row(name, ours, theirs=None, o=None, r=None):
        rec = {"path": name, "ms": round(clock(ours), 4)}
        if ref is not None and theirs is not None:
            rec["reference_cuda_ms"] = round(clock(theirs), 4)
            if o is not None:
                rec["same_bits_as_reference_cuda"] = same(o, r)
        rows.append(rec)

    x = torch.randn(1 << 26, device=dev, generator=g) * 3
    row("float_quantize nearest e4m3 without subnormals, 2^26 elements", lambda: be.float_quantize_nearest(x, 3, 4, False, True),
        lambda: ref.float_quantize_nearest(x, 3, 4, False, True), be.float_quantize_nearest(x, 3, 4, False, True),
        ref.float_quantize_nearest(x, 3, 4, False, True) if ref is not None else None)
    del x
    S = 2048
    a = torch.randn(S, S, device=dev, generator=g)
    b = torch.randn(S, S, device=dev, generator=g)
    c, r = torch.empty(S, S, device=dev), torch.empty(S, S, device=dev)

    def mm(name, aa, ma, ea, mm_, em, sub, sat, comp):
        row("float_mm 2048^3 " + name,
            lambda: be.float_quantize_nearest_mm(aa, b, c, S, S, S, ma, ea, mm_, em, sub, sat, comp, order="cuda"),
            lambda: ref.float_quantize_nearest_mm(aa, b, r, S, S, S, ma, ea, mm_, em, sub, sat, comp), c, r)

    mm("e5m2 / e5m2 without subnormals", a, 2, 5, 2, 5, False, False, False)
    mm("e5m10 / e4m3 without subnormals", a, 10, 5, 3, 4, False, False, False)
    mm("e5m10 / e4m3 without subnormals, compensated", a, 10, 5, 3, 4, False, False, True)
    mm("fp32 add / e4m3 mul, compensated", a, 23, 8, 3, 4, True, False, True)
    mm("e3m4 / e3m4 (range checks fail: exact kernel)", a, 4, 3, 4, 3, True, True, False)
    mm("e5m2 / e5m2, operands x 200 (sums overflow: exact kernel)", a * 200, 2, 5, 2, 5, True, False, False)
    a_inf = a.clone()
    a_inf[0, 0] = float("inf")
    mm("e5m10 / e4m3, one infinity in A (exact kernel)", a_inf, 10, 5, 3, 4, True, False, False)
    for sub in (True, False):
        row("float_mm stochastic 2048^3 e5m10 / e4m3 subnormals=%s" % sub,
            lambda: be.float_quantize_stochastic_mm(a, b, c, S, S, S, 10, 5, 13, 3, 4, 20, sub, False, seed=5),
            lambda: ref.float_quantize_stochastic_mm(a, b, r, S, S, S, 10, 5, 13, 3, 4, 20, sub, False))
    del a, b, c, r, a_inf
    att = torch.randn(12288, 1024, device=dev, generator=g)
    so, sr = torch.empty_like(att), torch.empty_like(att)
    row("softmax forward 12288 x 1024 e5m10 without subnormals",
        lambda: be.float_quantize_nearest_softmax_forward(att, so, -1, 10, 5, 10, 5, 10, 5, False, False),
        lambda: ref.float_quantize_nearest_softmax_forward(att, sr, -1, 10, 5, 10, 5, 10, 5, False, False), so, sr)
    del att, so, sr
    xl = torch.randn(16384, 768, device=dev, generator=g)
    w, bb = torch.randn(768, device=dev, generator=g), torch.randn(768, device=dev, generator=g)
    y1, m1, r1 = torch.empty_like(xl), torch.empty(16384, device=dev), torch.empty(16384, device=dev)
    y2, m2, r2 = torch.empty_like(xl), torch.empty(16384, device=dev), torch.empty(16384, device=dev)
    row("layernorm forward 16384 x 768 e5m10 without subnormals",
        lambda: be.float_quantize_layernorm_forward(xl, w, bb, y1, m1, r1, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, False, False),
        lambda: ref.float_quantize_layernorm_forward(xl, w, bb, y2, m2, r2, 1e-5, [-1], 10, 5, 10, 5, 10, 5, 10, 5, False, False), y1, y2)
    del xl, y1, y2
    for sub in (True, False):
        fmt = q.QAffineFormats(fwd_mac=(FloatingPoint(5, 10, sub, False), FloatingPoint(4, 3, sub, False)),
                               bwd_mac=(FloatingPoint(5, 10, sub, False), FloatingPoint(4, 3, sub, False)))
        conv = q.QConv2d(64, 64, 3, fmt, padding=1).to(dev)
        xc = torch.randn(64, 64, 56, 56, device=dev, generator=g)
        with torch.no_grad():
            row("QConv2d forward 64 x 64 x 56 x 56, 3 x 3, implicit GEMM, subnormals=%s" % sub, lambda: conv(xc))
            eligible = qmod.implicit_conv_eligible
            qmod.implicit_conv_eligible = lambda f, t: False
            try:
                row("QConv2d forward, unfold + GEMM, subnormals=%s" % sub, lambda: conv(xc))
            finally:
                qmod.implicit_conv_eligible = eligible
        del conv, xc
    for sub in (True, False):
        torch.manual_seed(0)
        model = QTinyGPT(BlockConfig(), default_formats(FloatingPoint(5, 10, sub, False), FloatingPoint(4, 3, sub, False))).to(dev)
        idx = torch.randint(0, 50257, (8, 1024), device=dev)

        def step():
            model.zero_grad(set_to_none=True)
            model(idx).float().pow(2).mean().backward()

        row("GPT-2-small block forward + backward (no update), subnormals=%s" % sub, step)
        del model
    return {"rows": rows}


def run_formats(args) -> int:
    import torch

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    out = formats_sweep(dev)
    for r in out["rows"]:
        sys.stderr.write("%-76s %9.3f ms%s\n" % (r["path"], r["ms"], ("   reference CUDA %9.3f ms%s" % (
            r["reference_cuda_ms"], ("  same bits %s" % r["same_bits_as_reference_cuda"]) if "same_bits_as_reference_cuda" in r else ""))
            if "reference_cuda_ms" in r else ""))
    print(json.dumps({"metric": "paths outside the benchmark format pairs, ms beside the reference's CUDA kernels", "unit": "ms", "n_gpus": 1, **out}))
    return 0


def run_c4(args) -> int:
    import torch

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    sizes = (2048, 4096, 8192) if args.size == SIZE else (args.size,)
    out = c4_sweep(dev, sizes)
    for r in out["rows"]:
        sys.stderr.write("%5d  %-38s %-4s %-24s %9.3f ms %7.3f TMAC/s%s\n" % (r["size"], r["formats"], r["order"], r["form"], r["ms"], r["tmacs"],
                                                                              ("   reference CUDA %.3f ms, same bits %s" % (r["reference_cuda_ms"], r["same_bits_as_reference_cuda"]))
                                                                              if "reference_cuda_ms" in r else ""))
    print(json.dumps({"metric": "float_mm sweep (benchmark config 4), simulated TMAC/s", "unit": "TMAC/s", "n_gpus": 1, **out}))
    return 0


# ----------------------------------------------------------------------------------- config 5: training step
def block_step(dev, world: int, rank: int, steps: int, warmup: int, overlap: bool = True) -> dict | None:
    """One quantized GPT-2-small block (d=768, 12 heads, MLP 3072, seq 1024, batch 8 per GPU), forward + backward,
    gradients averaged over the ranks with bucketed NCCL all-reduces launched from autograd hooks while the backward
    pass runs (`overlap`; otherwise after it).  Weak scaling: the per-GPU batch is fixed.  The process group must
    exist already when world > 1.  Returns the record on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist

    from mptorch_b200 import FloatingPoint
    from mptorch_b200.gpt2_block import BlockConfig, QTinyGPT
    from mptorch_b200.optim import QSGD, fma_quantizer
    from mptorch_b200.parallel import GradientAllReducer, allreduce_gradients

    B, T = 8, 1024
    torch.manual_seed(0)                                   # identical random-init weights on every rank
    model = QTinyGPT(BlockConfig(seq_len=T)).to(dev)
    g = torch.Generator().manual_seed(1000 + rank)
    idx_host = torch.randint(0, 50257, (B, T), generator=g).pin_memory()     # synthetic uniform token ids
    reducer = GradientAllReducer(model.parameters()) if (overlap and world > 1) else None
    # the weight update of the step: SGD with momentum, momentum and weights kept in e8m7 with a Kahan compensation
    # buffer (the reference's QSGD), as one fused launch per 40 tensors
    acc_q = fma_quantizer(FloatingPoint(8, 7, True, True))
    opt = QSGD(model.parameters(), lr=1e-3, momentum=0.9, momentum_quant=acc_q, acc_quant=acc_q, compensated=True)
    opt_ev = []

    def step(timed=False):
        idx = idx_host.to(dev, non_blocking=True)
        model.zero_grad(set_to_none=True)
        loss = model(idx).float().pow(2).mean()
        loss.backward()
        if reducer is not None:
            reducer.finish()
        else:
            allreduce_gradients(model.parameters())
        if timed:
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            o0.record()
            opt.step()
            o1.record()
            opt_ev.append((o0, o1))
        else:
            opt.step()
        return loss

    warmup = max(warmup, 3)
    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step(timed=True)
        loss_host = loss.item()                            # device -> host read of the step's result
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / steps
    if reducer is not None:
        reducer.remove()
    opt_ms = statistics.mean(a.elapsed_time(b) for a, b in opt_ev)
    # the same update through the reference's per-tensor sequence of torch kernels and quantizer launches, once, for scale
    opt.fused = False
    torch.cuda.synchronize(dev)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    opt.step()
    p1.record()
    torch.cuda.synchronize(dev)
    opt_per_tensor_ms = p0.elapsed_time(p1)
    n_params = sum(p.numel() for p in model.parameters())
    macs = model.macs_per_step(B, T) * world
    del model, opt
    if rank != 0:
        return None
    v = macs / ms / 1e6
    return {"metric": "GPT-2-small block training step, simulated GMAC/s", "value": v, "unit": "GMAC/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (MACs rounded: add e5m10, mul e4m3)", "data": "synthetic",
            "config": {"workload": "QLinear/QLayerNorm/QSoftmax block d=768 h=12 mlp=3072 seq=1024 batch=8 per GPU, fwd+bwd, "
                                   "DP gradient all-reduce %s, QSGD update (momentum 0.9, e8m7 momentum and weights, Kahan-compensated)"
                                   % ("under the backward pass" if reducer is not None or world == 1 else "after the backward pass"),
                       "loss": loss_host},
            "optimizer": {"fused_step_ms": round(opt_ms, 4), "per_tensor_step_ms": round(opt_per_tensor_ms, 4), "parameters": n_params,
                          "gbs": round(32.0 * n_params / opt_ms / 1e6, 1),
                          "note": "QSGD.step inside the timed step: one launch for all parameter tensors; 32 B per parameter "
                                  "(weight, gradient, momentum, compensation read; weight, momentum, compensation written)"},
            "e2e": {"value": v, "unit": "GMAC/s", "h2d_bytes_per_step": B * T * 8, "d2h_bytes_per_step": 4, "ms_per_step": ms}}


def run_block(args) -> int:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = block_step(dev, world, rank, args.steps, args.warmup, overlap=not args.no_overlap)
    if rec is not None:
        print(json.dumps(rec))
    if world > 1:
        dist.destroy_process_group()
    return 0


# ----------------------------------------------------------------------------------- GPU arm
def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=SIZE, help="M=N=K (the headline is 8192)")
    ap.add_argument("--order", default="cuda", choices=["cuda", "seq"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline legs only: skip the kernel, sweep and training-step legs")
    ap.add_argument("--no-overlap", action="store_true", help="collectives after the compute they follow instead of under it")
    ap.add_argument("--panels", type=int, default=1,
                    help="row panels per rank whose all-gather runs under the next panel's kernel (1: one launch and one "
                         "all-gather, the fastest form measured at 2, 4 and 8 GPUs)")
    ap.add_argument("--quant-log2n", type=int, default=28, help="log2 of the quantizer leg's element count")
    ap.add_argument("--workload", default="mm", choices=["mm", "block", "kernels", "c4", "formats"],
                    help="mm: the headline float_mm (default); block: benchmark config 5, one GPT-2-small-shaped block, "
                         "fwd+bwd with (add e5m10, mul e4m3) MACs, data parallel with a gradient all-reduce")
    ap.add_argument("--record-counters", nargs="+", metavar="CSV",
                    help="no benchmark: rebuild profiles/mm_kernel_counters.json from ncu --csv logs "
                         "(PER_MAC_CSV SIZE [TRAFFIC_CSV_8192]) and stamp it with the kernel sources' git blob hashes")
    args = ap.parse_args()
    if args.record_counters:
        rc = args.record_counters
        c = record_counters(rc[0], int(rc[1]), rc[2] if len(rc) > 2 else None,
                            "float_mm %s^3 mul e5m2 / add e5m2 (per-MAC counters), 8192^3 (DRAM traffic)" % rc[1])
        print(json.dumps(c))
        return 0
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "block":
        return run_block(args)
    if args.workload == "kernels":
        return run_kernels(args)
    if args.workload == "c4":
        return run_c4(args)
    if args.workload == "formats":
        return run_formats(args)

    import torch
    import torch.distributed as dist

    from mptorch_b200 import backend as be
    from mptorch_b200.parallel import sharded_float_mm, sharded_float_mm_streamed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    S = args.size
    assert S % world == 0
    rows = S // world
    warmup = max(args.warmup, 3)
    panels = 1 if (world == 1 or args.no_overlap) else max(1, args.panels)

    g = torch.Generator(device=dev).manual_seed(1234)
    a_full = torch.randn(S, S, device=dev, generator=g)      # same on every rank
    b = torch.randn(S, S, device=dev, generator=g)
    a = a_full[rank * rows:(rank + 1) * rows].contiguous()
    del a_full
    c_full = torch.empty(S, S, device=dev)
    launches = [0]

    def mm_rows(x, y):
        """This rank's kernel on a block of its rows: the reference-named backend entry (C ABI underneath)."""
        out = torch.empty(x.shape[0], S, device=dev)
        be.float_quantize_nearest_mm(x, y, out, x.shape[0], S, S, FMT["man_add"], FMT["exp_add"], FMT["man_mul"],
                                     FMT["exp_mul"], True, False, False, order=args.order)
        # stats_init_kernel, two stats_kernel, mm_kernel, and for products of at least 2^33 MACs the exact_mm_kernel
        # launch that follows it (which finds nothing to do on these operands)
        launches[0] += 4 + (1 if x.shape[0] * S * S >= 2 ** 33 else 0)
        return out

    def step():
        # one float_mm over the whole problem: the local row block in `panels` panels, each panel's C rows all-gathered
        # on a side stream under the next panel's kernel
        if world == 1:
            be.float_quantize_nearest_mm(a, b, c_full, S, S, S, FMT["man_add"], FMT["exp_add"], FMT["man_mul"],
                                         FMT["exp_mul"], True, False, False, order=args.order)
            launches[0] += 4 + (1 if S ** 3 >= 2 ** 33 else 0)
        else:
            sharded_float_mm(a, b, S, mm_rows, panels=panels, out=c_full)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    launches_timed = launches[0]
    # the kernel alone (no exchange), for the roofline: this rank's whole row block in one launch, CUDA events around it
    c_rows = torch.empty(rows, S, device=dev)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(max(1, min(args.steps, 5)))]
    for x, y in kev:
        x.record()
        be.float_quantize_nearest_mm(a, b, c_rows, rows, S, S, FMT["man_add"], FMT["exp_add"], FMT["man_mul"],
                                     FMT["exp_mul"], True, False, False, order=args.order)
        y.record()
    barrier()
    kern_ms = statistics.mean(x.elapsed_time(y) for x, y in kev)
    clocks = sampler.stop() if rank == 0 else None
    del c_rows
    t = torch.tensor([total_ms, kern_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kern_ms = t.tolist()
    ms_per_step = total_ms / args.steps
    macs = float(S) ** 3

    # ---- end to end through the public API with host buffers: each rank's A rows and its 1/world slice of B travel host ->
    # device (the ranks assemble B with one all-gather over NVLink), the rank's C rows travel back
    ah = torch.empty(rows, S).pin_memory(); ah.copy_(a)
    bh = torch.empty(S, S).pin_memory(); bh.copy_(b)
    ch = torch.empty(rows, S).pin_memory()
    e2e_steps = max(1, min(args.steps, 3))
    kw = dict(man_add=2, exp_add=5, man_mul=2, exp_mul=5, rounding="nearest", fma=False, subnormals=True, saturate=False)

    def e2e_step():
        if args.no_overlap and world > 1:
            from mptorch_b200.quant import float_mm_streamed

            float_mm_streamed(ah, bh, out=ch, device=dev, block_rows=1024, **kw)      # every rank copies all of B
        else:
            sharded_float_mm_streamed(ah, bh, S, out=ch, device=dev, block_rows=1024, **kw)

    e2e_step()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(e2e_steps):
        e2e_step()
    s1.record()
    barrier()
    t = torch.tensor([s0.elapsed_time(s1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = t.item() / e2e_steps
    b_h2d_rows = S if (args.no_overlap or world == 1) else S // world
    # the rows that came back through host memory against the same rows of the device-resident product of the timed steps
    same = torch.tensor([int(torch.equal(ch.view(torch.int32), c_full[rank * rows:(rank + 1) * rows].cpu().view(torch.int32)))], device=dev)
    if world > 1:
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
    e2e_same_bits = bool(same.item())
    del ah, bh, ch, a, b, c_full
    torch.cuda.empty_cache()

    extras = not args.no_extras
    ref = _ref_cuda() if (rank == 0 and not args.no_cpu_baseline) else None

    def clock(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(reps):
            fn()
        q1.record()
        torch.cuda.synchronize(dev)
        return q0.elapsed_time(q1) / reps

    # ---- elementwise quantizers, HBM bound: 2^28 elements of the benchmark config 2 mixture
    # (90% N(0,1), 5% N(0,1e-6), 5% U(-1e5,1e5)); e4m3 with subnormals and saturation; binary8 P=3
    quant, quant_all = None, {}
    if rank == 0:
        n = 1 << args.quant_log2n
        u = torch.rand(n, device=dev, generator=g)
        x = torch.randn(n, device=dev, generator=g)
        x = torch.where(u < 0.90, x, torch.where(u < 0.95, x * 1e-3, (torch.rand(n, device=dev, generator=g) * 2 - 1) * 1e5))
        del u
        rnd = torch.randint_like(x, 2147483647, dtype=torch.int32)
        legs = {
            "nearest": (lambda: be.float_quantize_nearest(x, 3, 4, True, True), 8,
                        (lambda: ref.float_quantize_nearest(x, 3, 4, True, True)) if ref is not None else None),
            "truncate": (lambda: be.float_quantize_truncate(x, 3, 4, True, True), 8, None),
            "stochastic_given_words": (lambda: be.float_quantize_stochastic(x, 3, 4, 20, True, True, rand=rnd), 12,
                                       (lambda: ref.float_quantize_stochastic(x, 3, 4, 20, True, True)) if ref is not None else None),
            "stochastic_philox": (lambda: be.float_quantize_stochastic(x, 3, 4, 20, True, True, seed=1), 8, None),
            "binary8_p3_nearest": (lambda: be.binary8_quantize_nearest(x, 3, True, 1, True), 8,
                                   (lambda: ref.binary8_quantize_nearest(x, 3, True, ref.OverflowPolicy.SATURATE_MAXFLOAT, True)) if ref is not None else None),
        }
        for name, (fn, bytes_per, ref_fn) in legs.items():
            qms = clock(fn, 10)
            quant_all[name] = {"gbs": bytes_per * n / qms / 1e6, "ms": qms, "bytes_per_element": bytes_per}
            if ref_fn is not None:
                try:
                    # the reference call includes what it always does around its kernel (zeros_like, its own random words)
                    quant_all[name]["reference_cuda_ms"] = clock(ref_fn, 5)
                except Exception as ex:
                    quant_all[name]["reference_cuda_error"] = repr(ex)[:120]
        quant = quant_all["nearest"]
        del x, rnd
        torch.cuda.empty_cache()

    # ---- same-GPU baseline: the reference's own CUDA kernel (unmodified sources built for sm_100a into oracle/_ref),
    # same formats and accumulation order, at 2048^3 (its 8x8-thread blocks are slow; the rate is size independent)
    ref_gpu = None
    if ref is not None:
        try:
            R = 2048
            ra = torch.randn(R, R, device=dev, generator=g)
            rb = torch.randn(R, R, device=dev, generator=g)
            rcout = torch.zeros(R, R, device=dev)
            rms = clock(lambda: ref.float_quantize_nearest_mm(ra, rb, rcout, R, R, R, 2, 5, 2, 5, True, False, False), 3)
            ours = torch.empty(R, R, device=dev)
            be.float_quantize_nearest_mm(ra, rb, ours, R, R, R, 2, 5, 2, 5, True, False, False, order="cuda")
            ref_gpu = {"value": float(R) ** 3 / rms / 1e6, "unit": "GMAC/s", "size": R, "ms": rms,
                       "kernel": "reference quant_cuda mm_impl (float_quantize_nearest_mm), same GPU",
                       "bit_identical_to_ours": bool(torch.equal(ours.view(torch.int32), rcout.view(torch.int32)))}
            del ra, rb, rcout, ours
        except Exception as ex:
            ref_gpu = {"value": None, "error": repr(ex)[:200]}

    # ---- the other benchmark configurations, so that one driver-run line carries them: config 3 and the reductions
    # (HBM-bound kernels), config 4 (the GEMM sweep with its variants), config 5 (the training step, every N)
    kernels = sweep = formats = None
    if extras and rank == 0 and world == 1:
        try:
            kernels = kernels_legs(dev, 10, 3, 1.0, with_reference=ref is not None)
        except Exception as ex:
            kernels = {"error": repr(ex)[:300]}
        torch.cuda.empty_cache()
        try:
            sweep = c4_sweep(dev)
        except Exception as ex:
            sweep = {"error": repr(ex)[:300]}
        torch.cuda.empty_cache()
        try:
            formats = formats_sweep(dev)          # formats without subnormals and failed range checks, reference beside
        except Exception as ex:
            formats = {"error": repr(ex)[:300]}
        torch.cuda.empty_cache()
    block = None
    if extras:
        try:
            block = block_step(dev, world, rank, 3, 3, overlap=not args.no_overlap)
        except Exception as ex:
            block = {"error": repr(ex)[:300]}
            if world > 1:
                raise

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        clk = (clocks or {}).get("sm_mhz") or peaks.get("sm_max_mhz") or 1965.0
        cnt = load_counters()
        i_mac, alu_mac = cnt["inst_per_mac"], cnt["alu_inst_per_mac"]
        slots_mac = 2 * cnt["packed_fp_inst_per_mac"] + alu_mac
        issue_peak = sms * 128 * clk * 1e6 / i_mac / 1e9          # GMAC/s per GPU at the sampled clock
        achieved = macs / world / kern_ms / 1e6                   # GMAC/s of one GPU's kernel
        line = {
            "metric": METRIC, "value": macs / ms_per_step / 1e6, "unit": "GMAC/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (each multiply and add rounded to e5m2)", "data": "synthetic",
            "config": config_for(S), "accum_order": args.order,
            "notes": "M rows sharded over %d GPU(s)%s" % (world, (", C all-gathered in %d row panel(s) per rank" % panels) if world > 1 else ""),
            "clocks": clocks,
            "e2e": {"value": macs / e2e_ms / 1e6, "unit": "GMAC/s", "h2d_bytes_per_step": 4 * (rows * S + b_h2d_rows * S),
                    "d2h_bytes_per_step": 4 * rows * S, "ms_per_step": e2e_ms, "same_bits_as_device_result": e2e_same_bits,
                    "b_operand": "each rank copies 1/%d of every K panel of B from host memory; one NCCL all-gather per panel assembles it under the kernels of the panels before" % world if b_h2d_rows != S
                    else "A and B copied from host memory in K panels under the kernels of the panels before; C returns in row blocks under the last panel"},
            "gpu_launches": launches_timed,
            "roofline": {"bound": "issue", "achieved": achieved, "peak": issue_peak, "unit": "GMAC/s",
                         "frac": achieved / issue_peak,
                         "traffic": cnt.get("dram_bytes_per_launch_8192cubed") if (S == 8192 and world == 1) else None,
                         "traffic_source": "ncu capture recorded in profiles/mm_kernel_counters.json",
                         "algorithmic_bytes": 3 * 4 * S * S // world + (world - 1) * 4 * S * S // world,
                         "alu_pipe_peak": sms * 64 * clk * 1e6 / alu_mac / 1e9,
                         "datapath_peak": sms * 128 * clk * 1e6 / slots_mac / 1e9,
                         "datapath_frac": achieved / (sms * 128 * clk * 1e6 / slots_mac / 1e9),
                         "constants_stale": cnt["constants_stale"], "constants_from": cnt.get("captured_at"),
                         "note": "CUDA-core issue roofline: %d SMs x 128 lanes x %.0f MHz / %.2f instructions per MAC; "
                                 "alu_pipe_peak = %d SMs x 64 ALU lanes x clock / %.2f ALU instructions per MAC; "
                                 "datapath_peak = SMs x 128 fp32/int32 lane slots x clock / %.2f slots per MAC "
                                 "(a packed fp32x2 instruction takes two)" % (sms, clk, i_mac, sms, alu_mac, slots_mac)},
            "roofline_quantize": {"bound": "hbm", "achieved": quant["gbs"], "peak": hbm_peak, "unit": "GB/s",
                                  "frac": quant["gbs"] / hbm_peak, "traffic": None, "peak_source": peak_src,
                                  "kernel": "float_quantize_nearest e4m3, 2^%d elements, 8 B/element" % args.quant_log2n,
                                  "all_kernels_gbs": {k: round(v["gbs"], 1) for k, v in quant_all.items()},
                                  "reference_cuda_ms": {k: round(v["reference_cuda_ms"], 4) for k, v in quant_all.items() if "reference_cuda_ms" in v},
                                  "ms": {k: round(v["ms"], 4) for k, v in quant_all.items()}},
        }
        if ref_gpu is not None:
            line["reference_cuda_same_gpu"] = ref_gpu
        if kernels is not None:
            line["roofline_kernels"] = kernels
        if sweep is not None:
            line["c4_sweep"] = sweep
        if formats is not None:
            line["formats_sweep"] = formats
        if block is not None:
            line["block_step"] = block
        if world == 1 and not args.no_cpu_baseline:
            try:
                cb = cpu_baseline(1)
                line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as ex:  # the baseline is a reported figure, never a reason to lose the bench line
                line["cpu_baseline"] = {"value": None, "unit": "GMAC/s", "cores": 0, "kind": "port", "sample": "failed: %r" % (ex,)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
