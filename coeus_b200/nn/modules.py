"""``torch.nn.Module`` layers over :mod:`coeus_b200.nn.functional`.  Shapes and parameter names
follow the reference's transformer structs (``MultiHeadAttention`` with q/k/v/o weights,
``FeedForward`` with up/down, ``LayerNorm`` scale/bias; plugins/model-transformer/src/lib.rs:131-383)
with q, k and v fused into one matrix."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import functional as F


def _dtype(device) -> torch.dtype:
    return torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32


class Linear(nn.Module):
    """``y = act(x @ W + b)`` with ``W [in, out]``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 activation: str = "none", device="cuda", init_std: float = 0.02) -> None:
        super().__init__()
        dt = _dtype(device)
        self.weight = nn.Parameter(torch.empty(in_features, out_features, device=device,
                                               dtype=dt).normal_(0, init_std))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dt)) if bias else None
        self.activation = activation

    def forward(self, x):
        return F.linear(x, self.weight, self.bias, self.activation)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device="cuda") -> None:
        super().__init__()
        dt = _dtype(device)
        self.scale = nn.Parameter(torch.ones(dim, device=device, dtype=dt))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dt))
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x, self.scale, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, device="cuda") -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim, device=device, dtype=_dtype(device)))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, self.scale, self.eps)


class Embedding(nn.Module):
    def __init__(self, vocab: int, dim: int, device="cuda", init_std: float = 0.02) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, device=device,
                                               dtype=_dtype(device)).normal_(0, init_std))

    def forward(self, ids, pe: Optional[torch.Tensor] = None):
        return F.embedding(ids, self.weight, pe)


class CausalSelfAttention(nn.Module):
    """Fused QKV projection, optional RoPE, flash attention, output projection."""

    def __init__(self, dim: int, num_heads: int, bias: bool = False, rope: bool = False,
                 rope_theta: float = 10000.0, device="cuda") -> None:
        super().__init__()
        self.nh, self.dh = num_heads, dim // num_heads
        self.rope, self.theta = rope, rope_theta
        self.qkv = Linear(dim, 3 * dim, bias, device=device)
        self.o = Linear(dim, dim, bias, device=device)

    def forward(self, x, B: int, S: int):
        qkv = self.qkv(x)
        if self.rope:
            qkv = F.rope(qkv, 2 * self.nh, self.dh, S, 0, self.theta)
        return self.o(F.attention(qkv, B, S, self.nh, self.dh, True))


class MLP(nn.Module):
    """``down(gelu(up(x)))`` or, with ``swiglu=True``, ``down(silu(gate) * up)``."""

    def __init__(self, dim: int, inter: int, bias: bool = False, swiglu: bool = False,
                 device="cuda") -> None:
        super().__init__()
        self.swiglu = swiglu
        self.up = Linear(dim, 2 * inter if swiglu else inter, bias and not swiglu,
                         activation="none" if swiglu else "gelu", device=device)
        self.down = Linear(inter, dim, bias and not swiglu, device=device)

    def forward(self, x):
        h = self.up(x)
        return self.down(F.swiglu(h) if self.swiglu else h)


class Block(nn.Module):
    """Pre-norm decoder block (the reference's ``TransformerLayer``, lib.rs:425-500)."""

    def __init__(self, dim: int, num_heads: int, inter: int, rms: bool = False, bias: bool = True,
                 swiglu: bool = False, rope: bool = False, device="cuda") -> None:
        super().__init__()
        Norm = RMSNorm if rms else LayerNorm
        self.norm1, self.norm2 = Norm(dim, device=device), Norm(dim, device=device)
        self.attn = CausalSelfAttention(dim, num_heads, bias, rope, device=device)
        self.mlp = MLP(dim, inter, bias, swiglu, device=device)

    def forward(self, x, B: int, S: int):
        x = x + self.attn(self.norm1(x), B, S)
        return x + self.mlp(self.norm2(x))


class CrossEntropyLoss(nn.Module):
    def forward(self, logits, targets):
        return F.cross_entropy(logits, targets)
