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

import ctypes as _C
import math
from typing import Callable

import numpy as _np

from . import _cabi
from .number import FloatingPoint
from .quant import float_quantize, float_quantize_multi

__all__ = ["QOptim", "OptimLP", "QSGD", "QAdamW", "fma_quantizer"]


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


# ------------------------------------------------------------------------------------------ QSGD / QAdamW
class fma_quantizer:
    """The trivariate quantizer the reference's QSGD / QAdamW take for ``momentum_quant`` and ``acc_quant``:
    ``q(x, y, z) = Q(x + y * z)`` with Q = ``float_quantize`` to ``number`` (reference optim/sgd.py:17-21, and the
    ``acc_q`` of examples/mlp/mptorch_mlp_csupdate.py:165-171).  Calling it runs the product, the sum and the
    quantizer as three kernels, like a hand-written lambda would.  An optimizer that receives instances of this class
    (nearest rounding) for its quantizers recognises them and runs its whole step as one multi-tensor kernel
    (``mpt_qsgd_step`` / ``mpt_qadamw_step``) with the same bits."""

    def __init__(self, number: FloatingPoint, rounding: str = "nearest"):
        assert isinstance(number, FloatingPoint), "fma_quantizer takes a FloatingPoint format"
        assert rounding in ("nearest", "stochastic")
        self.number, self.rounding = number, rounding

    def __call__(self, x, y, z):
        n = self.number
        return float_quantize(x + y * z, n.exp, n.man, self.rounding, n.subnormals, n.saturate)


def _f32(x: float) -> float:
    """A Python scalar as torch hands it to an fp32 kernel: rounded to float32."""
    return float(_np.float32(x))


class _OptimTensor(_C.Structure):
    """``mpt_optim_tensor`` of include/mptorch_b200.h."""
    _fields_ = [("param", _C.c_void_p), ("grad", _C.c_void_p), ("buf0", _C.c_void_p), ("buf1", _C.c_void_p),
                ("buf2", _C.c_void_p), ("buf3", _C.c_void_p), ("n", _C.c_int64), ("flags", _C.c_int32)]


def _fusable_pair(mq, aq):
    """(momentum format or None, accumulator format or None, subnormals, saturate) when the whole step can run as the
    fused kernel: each quantizer is absent or a nearest ``fma_quantizer``, and the two agree on the format flags."""
    for q in (mq, aq):
        if q is not None and not (isinstance(q, fma_quantizer) and q.rounding == "nearest"):
            return None
    nums = [q.number for q in (mq, aq) if q is not None]
    if not nums:
        return (None, None, True, True)       # plain fp32 arithmetic: the same kernel with both quantizers off
    if any((n.subnormals, n.saturate) != (nums[0].subnormals, nums[0].saturate) for n in nums):
        return None
    return (mq.number if mq is not None else None, aq.number if aq is not None else None, nums[0].subnormals, nums[0].saturate)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _cuda_f32(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()) for t in ts)


class QSGD(SGD):
    """SGD with quantized momentum and weight updates and an optional Kahan compensation buffer
    (reference optim/sgd.py:30-163: same constructor, same state keys, same order of operations).

    ``momentum_quant`` and ``acc_quant`` are trivariate callables ``q(x, y, z) = Q(x + y * z)`` or None.  Any callable
    works through the per-tensor path, which issues the reference's torch operations one by one.  With ``fma_quantizer``
    instances (nearest rounding) and contiguous float32 CUDA parameters the step of a parameter group is ONE kernel
    launch per 40 tensors, bit-identical to the per-tensor path; ``fused=False`` turns that off."""

    def __init__(self, params, lr=1e-3, momentum=0, dampening=0, weight_decay=0, nesterov=False, momentum_quant=None,
                 acc_quant=None, compensated=False, fused=True):
        super().__init__(params=params, lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)
        self.momentum_quant, self.acc_quant, self.fused = momentum_quant, acc_quant, fused
        if compensated:
            for group in self.param_groups:
                for p in group["params"]:
                    self.state[p]["compensated_buffer"] = torch.zeros_like(p.data, device=p.data.device)

    def _step_fused(self, group, spec) -> bool:
        mnum, anum, sub, sat = spec
        ps = [p for p in group["params"] if p.grad is not None]
        momentum = group["momentum"]
        rows = []
        for p in ps:
            st = self.state[p]
            comp = st.get("compensated_buffer")
            if not _cuda_f32(p.data, p.grad.data, comp) or p.grad.is_sparse:
                return False
            first = momentum != 0 and "momentum_buffer" not in st
            if first:
                st["momentum_buffer"] = torch.empty_like(p.data)
            buf = st.get("momentum_buffer") if momentum != 0 else None
            if not _cuda_f32(buf):
                return False
            rows.append((p, buf, comp, first))
        if not rows:
            return True
        # one launch needs one answer to "compensated?"; parameters added later without a buffer go separately
        for want_comp in (True, False):
            sel = [r for r in rows if (r[2] is not None) == want_comp]
            if not sel:
                continue
            tab = (_OptimTensor * len(sel))()
            for i, (p, buf, comp, first) in enumerate(sel):
                tab[i] = _OptimTensor(p.data.data_ptr(), p.grad.data.data_ptr(), _ptr(buf), _ptr(comp), None, None, p.data.numel(), 1 if first else 0)
            dev = sel[0][0].device
            with torch.cuda.device(dev):
                _cabi.call("mpt_qsgd_step", tab, len(sel), _f32(group["lr"]), _f32(momentum), _f32(1.0 - group["dampening"]),
                           _f32(group["weight_decay"]), int(bool(group["nesterov"])), int(want_comp),
                           int(mnum is not None), mnum.man if mnum else 23, mnum.exp if mnum else 8,
                           int(anum is not None), anum.man if anum else 23, anum.exp if anum else 8, int(sub), int(sat),
                           _cabi.stream_ptr(dev))
        return True

    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        spec = _fusable_pair(self.momentum_quant, self.acc_quant) if self.fused else None
        with torch.no_grad():
            for group in self.param_groups:
                if spec is not None and self._step_fused(group, spec):
                    continue
                self._step_group(group)
        return loss

    def _step_group(self, group):
        """The reference's per-parameter sequence of torch operations (sgd.py:70-162)."""
        weight_decay, momentum, dampening = group["weight_decay"], group["momentum"], group["dampening"]
        nesterov, lr = group["nesterov"], group["lr"]
        for p in group["params"]:
            if p.grad is None:
                continue
            d_p = p.grad.data
            param_state = self.state[p]
            if weight_decay != 0:
                d_p.add_(p.data, alpha=weight_decay)
            if momentum != 0:
                if "momentum_buffer" not in param_state:
                    if self.momentum_quant is not None:
                        buf = param_state["momentum_buffer"] = self.momentum_quant(
                            torch.clone(d_p).detach(), torch.zeros_like(d_p), torch.zeros_like(d_p))
                    else:
                        buf = param_state["momentum_buffer"] = torch.clone(d_p).detach()
                else:
                    buf = param_state["momentum_buffer"]
                    if self.momentum_quant is not None:
                        buf = param_state["momentum_buffer"] = self.momentum_quant(
                            buf.mul_(momentum), d_p, (1.0 - dampening) * torch.ones_like(d_p))
                    else:
                        buf.mul_(momentum).add_(d_p, alpha=(1.0 - dampening))
                d_p = d_p.add(buf, alpha=momentum) if nesterov else buf
            comp = param_state.get("compensated_buffer")
            if self.acc_quant is not None:
                if comp is None:
                    p.data = self.acc_quant(p.data, d_p, -lr * torch.ones_like(p.data))
                else:
                    y = -self.acc_quant(comp, d_p, lr * torch.ones_like(d_p))
                    s = self.acc_quant(p.data, y, torch.ones_like(p.data))
                    param_state["compensated_buffer"] = self.acc_quant(self.acc_quant(s, p.data, -torch.ones_like(s)), y, -torch.ones_like(y))
                    p.data = s
            elif comp is None:
                p.add_(d_p, alpha=-lr)
            else:
                u = -lr * d_p
                y = u - comp
                s = p.data + y
                param_state["compensated_buffer"] = (s - p.data) - y
                p.data = s


class QAdamW(AdamW):
    """AdamW-shaped optimizer with quantized moment and weight updates and an optional Kahan compensation buffer
    (reference optim/adamw.py:12-167: same constructor, state keys and order of operations, including two properties
    of that code that are kept on purpose: ``weight_decay`` is accepted and never applied, and with ``compensated`` the
    moments and the step count are re-initialised at every step, because the state is never empty).

    Quantizers and the fused path are as for ``QSGD``; tensors that share a step count share a launch."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False, acc_quant=None,
                 momentum_quant=None, compensated=False, fused=True):
        super().__init__(params=params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
        self.acc_quant, self.momentum_quant, self.fused = acc_quant, momentum_quant, fused
        if compensated:
            for group in self.param_groups:
                for p in group["params"]:
                    self.state[p]["compensated_buffer"] = torch.zeros_like(p.data, device=p.data.device)

    @staticmethod
    def _init_state(param_state, p, amsgrad):
        if len(param_state) == 0 or "compensated_buffer" in param_state:
            param_state["step"] = 0
            param_state["exp_avg"] = torch.zeros_like(p.data, device=p.data.device)
            param_state["exp_avg_sq"] = torch.zeros_like(p.data, device=p.data.device)
            if amsgrad:
                param_state["max_exp_avg_sq"] = torch.zeros_like(p.data, device=p.data.device)

    def _step_fused(self, group, spec) -> bool:
        mnum, anum, sub, sat = spec
        amsgrad = group["amsgrad"]
        beta1, beta2 = group["betas"]
        ps = [p for p in group["params"] if p.grad is not None]
        for p in ps:
            st = self.state[p]
            if p.grad.is_sparse:
                raise RuntimeError("AdamW does not support sparse gradients")
            if not _cuda_f32(p.data, p.grad.data, st.get("compensated_buffer")):
                return False
        by_key = {}
        for p in ps:
            st = self.state[p]
            self._init_state(st, p, amsgrad)
            st["step"] += 1
            by_key.setdefault((st["step"], "compensated_buffer" in st), []).append(p)
        for (step, comp), sel in by_key.items():
            bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
            tab = (_OptimTensor * len(sel))()
            for i, p in enumerate(sel):
                st = self.state[p]
                tab[i] = _OptimTensor(p.data.data_ptr(), p.grad.data.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                                      _ptr(st.get("compensated_buffer")), _ptr(st.get("max_exp_avg_sq")) if amsgrad else None,
                                      p.data.numel(), 0)
            dev = sel[0].device
            # a CUDA tensor divided by a Python scalar is multiplied by the reciprocal, taken in double and rounded to fp32
            inv = _f32(1.0 / math.sqrt(bc2))
            with torch.cuda.device(dev):
                _cabi.call("mpt_qadamw_step", tab, len(sel), _f32(beta1), _f32(beta2), _f32(1.0 - beta1), _f32(1.0 - beta2), inv,
                           _f32(group["eps"]), _f32(group["lr"] / bc1), int(bool(amsgrad)), int(comp),
                           int(mnum is not None), mnum.man if mnum else 23, mnum.exp if mnum else 8,
                           int(anum is not None), anum.man if anum else 23, anum.exp if anum else 8, int(sub), int(sat),
                           _cabi.stream_ptr(dev))
        return True

    def step(self, closure: Callable = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        spec = _fusable_pair(self.momentum_quant, self.acc_quant) if self.fused else None
        with torch.no_grad():
            for group in self.param_groups:
                if spec is not None and self._step_fused(group, spec):
                    continue
                self._step_group(group)
        return loss

    def _step_group(self, group):
        """The reference's per-parameter sequence of torch operations (adamw.py:52-167)."""
        for p in group["params"]:
            amsgrad = group["amsgrad"]
            if p.grad is None:
                continue
            d_p = p.grad.data
            if d_p.is_sparse:
                raise RuntimeError("AdamW does not support sparse gradients")
            param_state = self.state[p]
            self._init_state(param_state, p, amsgrad)
            exp_avg, exp_avg_sq = param_state["exp_avg"], param_state["exp_avg_sq"]
            if amsgrad:
                max_exp_avg_sq = param_state["max_exp_avg_sq"]
            beta1, beta2 = group["betas"]
            param_state["step"] += 1
            if self.momentum_quant is not None:
                param_state["exp_avg"] = exp_avg = self.momentum_quant(exp_avg.mul_(beta1), d_p, (1.0 - beta1) * torch.ones_like(d_p))
                param_state["exp_avg_sq"] = exp_avg_sq = self.momentum_quant(exp_avg_sq.mul_(beta2), d_p ** 2, (1.0 - beta2) * torch.ones_like(d_p))
            else:
                exp_avg.mul_(beta1).add_(d_p, alpha=1.0 - beta1)
                exp_avg_sq.mul_(beta2).addcmul_(d_p, d_p, value=1.0 - beta2)
            bias_correction1 = 1.0 - beta1 ** param_state["step"]
            bias_correction2 = 1.0 - beta2 ** param_state["step"]
            step_size = group["lr"] / bias_correction1
            if amsgrad:
                torch.max(max_exp_avg_sq, exp_avg_sq, out=max_exp_avg_sq)
                denom = (max_exp_avg_sq.sqrt() / math.sqrt(bias_correction2)).add_(group["eps"])
            else:
                denom = (exp_avg_sq.sqrt() / math.sqrt(bias_correction2)).add_(group["eps"])
            comp = param_state.get("compensated_buffer")
            if self.acc_quant is not None:
                if comp is None:
                    p.data.addcdiv_(exp_avg, denom, value=-step_size)
                    p.data = self.acc_quant(p.data, torch.zeros_like(p.data), torch.zeros_like(p.data))
                else:
                    u = self.acc_quant(exp_avg / denom, torch.zeros_like(exp_avg), torch.zeros_like(exp_avg))
                    y = -self.acc_quant(comp, u, step_size * torch.ones_like(u))
                    s = self.acc_quant(p.data, y, torch.ones_like(p.data))
                    param_state["compensated_buffer"] = self.acc_quant(self.acc_quant(s, p.data, -torch.ones_like(s)), y, -torch.ones_like(y))
                    p.data = s
            elif comp is None:
                p.data.addcdiv_(exp_avg, denom, value=-step_size)
            else:
                u = -step_size * exp_avg / denom
                y = u - comp
                s = p.data + y
                param_state["compensated_buffer"] = (s - p.data) - y
                p.data = s
