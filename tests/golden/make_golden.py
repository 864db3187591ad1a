"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference tree is mounted (it is not needed afterwards):

    python oracle/build_ref.py            # builds oracle/_ref/quant_cpu from the reference sources
    python tests/golden/make_golden.py    # writes tests/golden/*.npz

Every array written here is an output of the reference's own compiled CPU
extension (``quant_cpu``) on seeded inputs; inputs are stored beside the
outputs (as uint32 bit patterns for the casters) so the fixtures are
self-contained.  The tests compare the C oracle, and through it the CUDA
kernels, against these files.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.build_ref import load_ref  # noqa: E402

INT_MAX = 2147483647


def caster_inputs(n_random: int, seed: int) -> np.ndarray:
    """fp32 bit patterns: specials, every exponent with a few mantissas, and uniform random bits."""
    rng = np.random.default_rng(seed)
    spec = [0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x7F800001,
            0x00000001, 0x80000001, 0x007FFFFF, 0x00400000, 0x00800000, 0x7F7FFFFF, 0xFF7FFFFF]
    mans = [0x000000, 0x000001, 0x3FFFFF, 0x400000, 0x400001, 0x7FFFFF, 0x200000, 0x600000, 0x100000, 0x500000]
    grid = [(s << 31) | (e << 23) | m for e in range(0, 256, 1) for m in mans for s in (0, 1)]
    rnd = rng.integers(0, 2**32, size=n_random, dtype=np.uint64).astype(np.uint32)
    return np.concatenate([np.array(spec, dtype=np.uint32), np.array(grid, dtype=np.uint32), rnd])


def bits_to_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.float32).copy())


def out_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().numpy().view(np.uint32).copy()


def main() -> int:
    ref = load_ref("quant_cpu")
    if ref is None:
        print("oracle/_ref/quant_cpu is not built; run oracle/build_ref.py first")
        return 1
    pol = {0: ref.OverflowPolicy.SATURATE_INFTY, 1: ref.OverflowPolicy.SATURATE_MAXFLOAT,
           2: ref.OverflowPolicy.SATURATE_MAXFLOAT2}

    # ---- casters --------------------------------------------------------------------------
    bits = caster_inputs(3000, 20251125)
    x = bits_to_tensor(bits)
    d = {"in_bits": bits}
    for (e, m) in [(5, 2), (4, 3), (5, 10), (8, 7), (8, 1), (2, 23), (3, 0), (6, 9), (8, 23), (2, 1), (7, 16), (8, 0)]:
        for sub in (0, 1):
            for sat in (0, 1):
                d[f"fp_e{e}m{m}_sub{sub}_sat{sat}"] = out_bits(ref.float_quantize_nearest(x, m, e, bool(sub), bool(sat)))
    for P in range(1, 8):
        for sg in (0, 1):
            for po in (0, 1, 2):
                for sub in (0, 1):
                    key = f"b8_P{P}_sg{sg}_po{po}_sub{sub}"
                    d[key + "_nearest"] = out_bits(ref.binary8_quantize_nearest(x, P, bool(sg), pol[po], bool(sub)))
                    d[key + "_truncate"] = out_bits(ref.binary8_quantize_truncate(x, P, bool(sg), pol[po], bool(sub)))
    # stochastic binary8: the reference draws randint_like(a, INT_MAX, int32) from the torch CPU generator
    torch.manual_seed(777)
    rnd = torch.randint_like(x, INT_MAX, dtype=torch.int32)
    d["b8_rand"] = rnd.numpy().copy()
    for P in (1, 3, 4, 6):
        for sg in (0, 1):
            for prng in (0, 4, 23 - (P - 1)):
                torch.manual_seed(777)
                d[f"b8_P{P}_sg{sg}_po1_sub1_stochastic_prng{prng}"] = out_bits(
                    ref.binary8_quantize_stochastic(x, P, prng, bool(sg), pol[1], True))
    for (e, m, bl, bu) in [(4, 3, 1, 1), (4, 3, 2, 1), (5, 2, 1, 2), (3, 4, 1, 1), (6, 1, 2, 2), (4, 2, 3, 1), (7, 5, 1, 1)]:
        for sat in (0, 1):
            d[f"sfp_e{e}m{m}_l{bl}_u{bu}_sat{sat}"] = out_bits(ref.superfp_quantize_nearest(x, m, e, bl, bu, bool(sat)))
    np.savez_compressed(os.path.join(HERE, "casters.npz"), **d)

    # ---- GEMM, sequential K order (the reference CPU path) ----------------------------------
    g = {}
    torch.manual_seed(4242)
    for tag, (M, K, N) in {"s": (17, 29, 23), "k8": (9, 32, 12), "c1": (64, 256, 48)}.items():
        a = torch.randn(M, K)
        b = torch.randn(K, N)
        g[f"{tag}_a"], g[f"{tag}_b"] = a.numpy().copy(), b.numpy().copy()
        for (ea, ma, em, mm_) in [(5, 2, 5, 2), (5, 10, 4, 3), (8, 7, 5, 2), (4, 3, 4, 3)]:
            for sat in (0, 1):
                c = torch.zeros(M, N)
                ref.float_quantize_nearest_mm(a, b, c, M, N, K, ma, ea, mm_, em, True, bool(sat), False)
                g[f"{tag}_mm_add_e{ea}m{ma}_mul_e{em}m{mm_}_sat{sat}"] = out_bits(c)
            c = torch.zeros(M, N)
            ref.float_quantize_nearest_mm_fma(a, b, c, M, N, K, ma, ea, True, False, False)
            g[f"{tag}_fma_e{ea}m{ma}"] = out_bits(c)
    # batched
    a = torch.randn(3, 10, 21)
    b = torch.randn(3, 21, 7)
    c = torch.zeros(3, 10, 7)
    ref.float_quantize_nearest_bmm(a, b, c, 10, 7, 21, 2, 5, 2, 5, True, False, False)
    g["bmm_a"], g["bmm_b"], g["bmm_e5m2"] = a.numpy().copy(), b.numpy().copy(), out_bits(c)
    # large-magnitude inputs: overflow to inf / saturation inside the accumulation
    a = torch.randn(8, 40) * 300.0
    b = torch.randn(40, 8) * 300.0
    g["big_a"], g["big_b"] = a.numpy().copy(), b.numpy().copy()
    for sat in (0, 1):
        c = torch.zeros(8, 8)
        ref.float_quantize_nearest_mm(a, b, c, 8, 8, 40, 2, 5, 2, 5, True, bool(sat), False)
        g[f"big_mm_e5m2_sat{sat}"] = out_bits(c)
    np.savez_compressed(os.path.join(HERE, "mm_seq.npz"), **g)

    # ---- softmax / layernorm, sequential order (reference CPU path) -------------------------
    r = {}
    torch.manual_seed(99)
    xs = torch.randn(4, 37, 5) * 3.0
    gs = torch.randn(4, 37, 5)
    r["sm_x"], r["sm_g"] = xs.numpy().copy(), gs.numpy().copy()
    for dim in (0, 1, 2):
        for (e, m) in [(5, 10), (8, 7), (4, 3)]:
            o = torch.zeros_like(xs)
            ref.float_quantize_nearest_softmax_forward(xs, o, dim, m, e, m, e, m, e, True, False)
            r[f"sm_fwd_dim{dim}_e{e}m{m}"] = out_bits(o)
            o2 = torch.zeros_like(xs)
            ref.float_quantize_nearest_softmax_lse_forward(xs, o2, dim, m, e, m, e, True, False)
            r[f"sm_lse_dim{dim}_e{e}m{m}"] = out_bits(o2)
            o3 = torch.zeros_like(xs)
            ref.float_quantize_nearest_softmax_backward(o, gs, o3, dim, m, e, m, e, True, False)
            r[f"sm_bwd_dim{dim}_e{e}m{m}"] = out_bits(o3)
    xl = torch.randn(6, 5, 48) * 2.0 + 0.5
    gl = torch.randn(6, 5, 48)
    w = torch.randn(48)
    bb = torch.randn(48)
    r["ln_x"], r["ln_g"], r["ln_w"], r["ln_b"] = xl.numpy().copy(), gl.numpy().copy(), w.numpy().copy(), bb.numpy().copy()
    for (e, m) in [(5, 10), (8, 7), (8, 23)]:
        y = torch.zeros_like(xl)
        mean = torch.zeros(6, 5)
        rstd = torch.zeros(6, 5)
        ref.float_quantize_layernorm_forward(xl, w, bb, y, mean, rstd, 1e-5, [-1], m, e, m, e, m, e, m, e, True, False)
        r[f"ln_fwd_y_e{e}m{m}"], r[f"ln_fwd_mean_e{e}m{m}"], r[f"ln_fwd_rstd_e{e}m{m}"] = out_bits(y), out_bits(mean), out_bits(rstd)
        gi = torch.zeros_like(xl)
        gg = torch.zeros(48)
        gb = torch.zeros(48)
        ref.float_quantize_layernorm_backward(xl, gl, w, bb, mean, rstd, gi, gg, gb, [-1], m, e, m, e, m, e, True, False)
        r[f"ln_bwd_gi_e{e}m{m}"], r[f"ln_bwd_gg_e{e}m{m}"], r[f"ln_bwd_gb_e{e}m{m}"] = out_bits(gi), out_bits(gg), out_bits(gb)
    np.savez_compressed(os.path.join(HERE, "reductions_seq.npz"), **r)
    for f in ("casters.npz", "mm_seq.npz", "reductions_seq.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
