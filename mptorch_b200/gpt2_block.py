"""A GPT-2-small-shaped transformer block built from the quantized layers: the caller-side workload of
benchmark config 5 (d=768, 12 heads, MLP 3072), wired like the reference's example
``examples/gpt/mptorch_shakespeare_softmax_gpt.py:246-337`` (pre-LN block: QLayerNorm -> attention with QLinear
projections, qmatmul for QK^T and PV, QSoftmax -> QLayerNorm -> QLinear MLP with GELU).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .number import FloatingPoint
from .quant import QAffineFormats, QLayerNorm, QLayerNormFormats, QLinear, QSoftmax, QSoftmaxFormats
from .quant.functional import qmatmul

__all__ = ["BlockConfig", "QBlock", "QTinyGPT", "default_formats"]


class BlockConfig:
    def __init__(self, d_model=768, n_head=12, d_mlp=3072, vocab=50257, seq_len=1024):
        self.d_model, self.n_head, self.d_mlp, self.vocab, self.seq_len = d_model, n_head, d_mlp, vocab, seq_len


def default_formats(add=FloatingPoint(5, 10, True, False), mul=FloatingPoint(4, 3, True, False)):
    """fwd_mac = bwd_mac = (add e5m10, mul e4m3) for the GEMMs (tuple order is (add, mul)); softmax and layernorm in
    the add format."""
    affine = QAffineFormats(fwd_mac=(add, mul), bwd_mac=(add, mul), fwd_rnd="nearest", bwd_rnd="nearest")
    softmax = QSoftmaxFormats(fwd_off=add, fwd_exp=add, fwd_acc=add, bwd_add=add, bwd_mul=add)
    lnorm = QLayerNormFormats(fwd_acc=add, fwd_mul=add, fwd_div=add, fwd_sqrt=add, bwd_acc=add, bwd_mul=add, bwd_div=add)
    return affine, softmax, lnorm


class QBlock(nn.Module):
    def __init__(self, cfg: BlockConfig, formats=None):
        super().__init__()
        affine, softmax, lnorm = formats or default_formats()
        self.cfg, self.affine = cfg, affine
        d = cfg.d_model
        self.ln1 = QLayerNorm(d, lnorm)
        self.qkv = QLinear(d, 3 * d, affine)
        self.proj = QLinear(d, d, affine)
        self.softmax = QSoftmax(-1, softmax)
        self.ln2 = QLayerNorm(d, lnorm)
        self.fc = QLinear(d, cfg.d_mlp, affine)
        self.out = QLinear(cfg.d_mlp, d, affine)
        for m in (self.qkv, self.proj, self.fc, self.out):
            nn.init.normal_(m.weight, std=0.02)
            nn.init.zeros_(m.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, d = x.shape
        h = self.cfg.n_head
        q, k, v = self.qkv(self.ln1(x)).split(d, dim=2)
        q = q.view(B, T, h, d // h).transpose(1, 2).contiguous()
        k = k.view(B, T, h, d // h).transpose(1, 2).contiguous()
        v = v.view(B, T, h, d // h).transpose(1, 2).contiguous()
        att = qmatmul(q, k.transpose(-2, -1), self.affine) * (1.0 / math.sqrt(d // h))
        mask = torch.ones(T, T, device=x.device, dtype=torch.bool).tril()
        att = self.softmax(att.masked_fill(~mask, float("-inf")))
        y = qmatmul(att, v, self.affine).transpose(1, 2).contiguous().view(B, T, d)
        x = x + self.proj(y)
        return x + self.out(torch.nn.functional.gelu(self.fc(self.ln2(x))))


class QTinyGPT(nn.Module):
    """Token embedding -> one quantized block -> plain fp32 head (the head and the loss stay in fp32)."""

    def __init__(self, cfg: BlockConfig, formats=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.block = QBlock(cfg, formats)
        nn.init.normal_(self.wte.weight, std=0.02)
        nn.init.normal_(self.wpe.weight, std=0.02)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        T = idx.shape[1]
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        return self.block(x)

    def macs_per_step(self, batch: int, seq: int) -> int:
        """Simulated MACs of one forward+backward pass (backward = 2x forward for every GEMM)."""
        c = self.cfg
        rows = batch * seq
        fwd = rows * c.d_model * (3 * c.d_model + c.d_model + 2 * c.d_mlp) + 2 * batch * c.n_head * seq * seq * (c.d_model // c.n_head)
        return 3 * fwd
