"""Generate tests/golden/optim_steps.npz from the UNMODIFIED reference optimizers.

Run where the reference tree is mounted (MPT_REFERENCE_ROOT, default: a sibling directory `reference`) after
`python oracle/build_ref.py`:

    python tests/golden/make_optim_golden.py

The reference's mptorch/optim/sgd.py and adamw.py import nothing but torch, so they are loaded file by file; their
quantizer callables are q(x, y, z) = float_quantize_nearest(x + y * z) with the reference's own compiled CPU extension
(quant_cpu) behind them.  Each case runs a few steps on seeded CPU tensors; the fixture keeps the initial parameters,
the per-step gradients and the parameters (and the optimizer's buffers) after every step, as uint32 bit patterns.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.build_ref import load_ref  # noqa: E402

SHAPES = [(37,), (8, 5), (3, 4, 2)]
STEPS = 4

# name -> (optimizer, constructor arguments, momentum format (exp, man) or None, accumulator format or None)
CASES = {
    "sgd_mom_acc": ("sgd", dict(lr=0.05, momentum=0.9), (5, 10), (8, 7)),
    "sgd_mom_acc_comp": ("sgd", dict(lr=0.05, momentum=0.9, compensated=True), (8, 7), (8, 7)),
    "sgd_mom_damp_comp_e5m2": ("sgd", dict(lr=0.1, momentum=0.8, dampening=0.25, compensated=True), (5, 2), (5, 2)),
    "sgd_mom_only": ("sgd", dict(lr=0.05, momentum=0.9), (5, 10), None),
    "adamw_mom_acc": ("adamw", dict(lr=0.01, betas=(0.9, 0.99)), (8, 7), (8, 7)),
    "adamw_mom_acc_comp": ("adamw", dict(lr=0.01, betas=(0.9, 0.99), compensated=True), (8, 7), (5, 10)),
    "adamw_amsgrad": ("adamw", dict(lr=0.02, betas=(0.8, 0.95), amsgrad=True), (5, 10), (5, 10)),
}


def load_module(root, rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t):
    return t.detach().contiguous().numpy().view(np.uint32).copy()


def main() -> int:
    root = os.environ.get("MPT_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    ref = load_ref("quant_cpu")
    if ref is None or not os.path.isdir(root):
        print("needs the reference tree and oracle/_ref/quant_cpu")
        return 1
    sgd = load_module(root, "mptorch/optim/sgd.py", "_ref_sgd").QSGD
    adamw = load_module(root, "mptorch/optim/adamw.py", "_ref_adamw").QAdamW

    def quant(fmt):
        if fmt is None:
            return None
        e, m = fmt
        return lambda x, y, z: ref.float_quantize_nearest((x + y * z).contiguous(), m, e, True, True)

    out = {}
    for name, (kind, kw, mfmt, afmt) in CASES.items():
        g = torch.Generator().manual_seed(sum(ord(c) for c in name))
        params = [torch.nn.Parameter(torch.randn(s, generator=g)) for s in SHAPES]
        for i, p in enumerate(params):
            out["%s/init/%d" % (name, i)] = bits(p.data)
        cls = sgd if kind == "sgd" else adamw
        opt = cls(params, momentum_quant=quant(mfmt), acc_quant=quant(afmt), **kw)
        for step in range(STEPS):
            for i, p in enumerate(params):
                p.grad = torch.randn(p.shape, generator=g) * (0.5 + step)
                out["%s/grad/%d/%d" % (name, step, i)] = bits(p.grad)
            opt.step()
            for i, p in enumerate(params):
                out["%s/param/%d/%d" % (name, step, i)] = bits(p.data)
                for key, val in opt.state[p].items():
                    if torch.is_tensor(val):
                        out["%s/state/%s/%d/%d" % (name, key, step, i)] = bits(val)
    np.savez_compressed(os.path.join(HERE, "optim_steps.npz"), **out)
    print("wrote optim_steps.npz with %d arrays" % len(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
