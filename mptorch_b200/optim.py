"""Low-precision optimizer wrapper: the reference's ``mptorch.optim.QOptim`` (optim/optim_low.py:8-122) with the
per-tensor quantizer loops fused.

Semantics per step, as in the reference: quantize gradients; swap the accumulator copies in; run the wrapped
optimizer; quantize and store the accumulators; quantize the weights; quantize the momentum buffers.  Each of those
quantizations visits every parameter tensor.  The reference calls its quantizer once per tensor (hundreds of small
launches per step for a transformer); here a quantizer made by ``mptorch_b200.quant.quantizer`` with a
``FloatingPoint`` format is recognised and applied to the whole list with ``float_quantize_multi`` (one launch per
48 tensors).  Any other callable is applied per tensor exactly as the reference does.

Stochastic quantizers are fused only when ``fused_stochastic=True``: the fused kernel draws Philox words, whereas
the per-tensor path draws ``randint_like`` from the torch generator like the reference, and the two streams differ.
"""
from __future__ import annotations

import torch
from torch.optim import SGD, Adam, AdamW, Optimizer

from .number import FloatingPoint
from .quant import float_quantize_multi

__all__ = ["QOptim", "OptimLP"]


def _fusable(q, fused_stochastic):
    num = getattr(q, "forward_number", None)
    rnd = getattr(q, "forward_rounding", None)
    if not isinstance(num, FloatingPoint) or rnd not in ("nearest", "stochastic"):
        return None
    if rnd == "stochastic" and not fused_stochastic:
        return None
    return num, rnd


class QOptim(Optimizer):
    """reference: optim/optim_low.py:8-122 (same constructor arguments and step order)."""

    def __init__(self, optim, weight_quant=None, grad_quant=None, momentum_quant=None, acc_quant=None, fused_stochastic=False):
        assert isinstance(optim, (SGD, Adam, AdamW))
        super().__init__(optim.param_groups, optim.defaults)
        self.param_groups = optim.param_groups       # shared with the wrapped optimizer, not copied
        self.optim = optim
        self.weight_quant, self.grad_quant = weight_quant, grad_quant
        self.momentum_quant, self.acc_quant = momentum_quant, acc_quant
        self.fused_stochastic = fused_stochastic
        self.momentum_keys = ["momentum_buffer"] if isinstance(optim, SGD) else ["exp_avg", "exp_avg_sq"]
        if acc_quant is not None:
            self.weight_acc = {}
            for group in self.param_groups:
                for p in group["params"]:
                    self.weight_acc[p] = p.detach().clone()

    # -- one quantizer over many tensors: returns the quantized tensors, fused when possible
    def _apply(self, q, tensors):
        if not tensors:
            return []
        spec = _fusable(q, self.fused_stochastic)
        if spec is not None and all(t.is_cuda and t.dtype == torch.float32 for t in tensors):
            num, rnd = spec
            return float_quantize_multi(tensors, num.exp, num.man, rnd, num.subnormals, num.saturate)
        return [q(t) for t in tensors]

    def step(self, closure=None):
        if self.grad_quant is not None:
            ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
            for p, gq in zip(ps, self._apply(self.grad_quant, [p.grad.data for p in ps])):
                p.grad.data = gq

        if self.acc_quant is not None:
            for group in self.param_groups:
                for p in group["params"]:
                    p.data = self.weight_acc[p].data

        loss = self.optim.step()

        if self.acc_quant is not None:
            ps = [p for g in self.param_groups for p in g["params"]]
            for p, aq in zip(ps, self._apply(self.acc_quant, [p.data for p in ps])):
                p.data = self.weight_acc[p].data = aq.data

        if self.weight_quant is not None:
            ps = [p for g in self.param_groups for p in g["params"]]
            for p, wq in zip(ps, self._apply(self.weight_quant, [p.data for p in ps])):
                p.data = wq.data

        if self.momentum_quant is not None:
            slots = []
            for group in self.param_groups:
                if isinstance(self.optim, SGD) and group["momentum"] == 0:
                    continue
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    state = self.optim.state[p]
                    for key in self.momentum_keys:
                        slots.append((state, key))
            for (state, key), mq in zip(slots, self._apply(self.momentum_quant, [s[k] for s, k in slots])):
                state[key] = mq
        return loss

    def __repr__(self):
        return "Quantized Optimizer: {}".format(self.optim.__repr__())

    __str__ = __repr__


OptimLP = QOptim
