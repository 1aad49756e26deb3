"""``torch.autograd.Function`` wrappers around the hand-written kernels, so that the ops compose
with PyTorch autograd (custom models, research code) while the flagship decoder keeps its explicit
forward/backward over flat buffers.

Conventions: activations are 2-D ``[tokens, features]`` bf16 on the GPU (any float dtype on CPU,
where the ops run their PyTorch restatement); parameters are ``torch.nn.Parameter`` in the
activation dtype; weight gradients are produced in fp32 by the kernels and cast to the parameter
dtype.  The reference has neither autograd nor layers beyond its transformer plugin's private
structs (plugins/model-transformer/src/lib.rs:131-383); ``Linear`` keeps its ``[in, out]`` weight
layout (lib.rs:50-74)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import norm as N


def _flat(x: torch.Tensor):
    return x.reshape(-1, x.shape[-1]), x.shape


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act):
        x2, shape = _flat(x)
        x2 = x2.contiguous()
        need_u = act == "gelu" and (x.requires_grad or w.requires_grad)
        u = torch.empty((x2.shape[0], w.shape[1]), dtype=x2.dtype, device=x2.device) if need_u else None
        y = G.linear_fwd(x2, w, bias, epi=act, aux_out=u)
        ctx.save_for_backward(x2, w, u)
        ctx.has_bias, ctx.act, ctx.shape = bias is not None, act, shape
        return y.reshape(*shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w, u = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        if ctx.act == "gelu":
            dy2 = E.gelu_bwd(u, dy2)
        gw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        G.linear_wgrad(x2, dy2, gw)
        gb = None
        if ctx.has_bias:
            gb = torch.zeros(w.shape[1], dtype=torch.float32, device=w.device)
            E.colsum_into(dy2, gb)
            gb = gb.to(w.dtype)
        dx = G.linear_dgrad(dy2, w).reshape(ctx.shape)
        return dx, gw.to(w.dtype), gb, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           activation: str = "none") -> torch.Tensor:
    """``act(x @ w + bias)`` with ``w [in, out]``; ``activation``: ``none`` | ``gelu`` (fused)."""
    return _Linear.apply(x, w, bias, activation)


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        x2, shape = _flat(x)
        x2 = x2.contiguous()
        y, mean, rstd = N.norm_fwd(x2, gamma, beta, eps, rms)
        ctx.save_for_backward(x2, gamma, mean, rstd)
        ctx.rms, ctx.shape, ctx.has_beta = rms, shape, beta is not None
        return y.reshape(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, gamma, mean, rstd = ctx.saved_tensors
        dg = torch.zeros(gamma.shape, dtype=torch.float32, device=gamma.device)
        db = torch.zeros_like(dg) if ctx.has_beta else None
        dx = N.norm_bwd(dy.reshape(x2.shape).contiguous(), x2, gamma, mean, rstd, dg, db, None,
                        ctx.rms)
        return (dx.reshape(ctx.shape), dg.to(gamma.dtype),
                db.to(gamma.dtype) if db is not None else None, None, None)


def layer_norm(x, gamma, beta, eps: float = 1e-5):
    return _Norm.apply(x, gamma, beta, eps, False)


def rms_norm(x, gamma, eps: float = 1e-6):
    return _Norm.apply(x, gamma, None, eps, True)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, nh, dh, causal):
        H = nh * dh
        q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
        o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal)
        ctx.save_for_backward(qkv, o, lse)
        ctx.dims = (B, S, nh, dh, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        B, S, nh, dh, causal = ctx.dims
        H = nh * dh
        dqkv = torch.empty_like(qkv)
        A.attention_bwd(do.contiguous(), qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:], o, lse, B, S,
                        nh, dh, causal=causal, dqkv=dqkv)
        return dqkv, None, None, None, None, None


def attention(qkv: torch.Tensor, B: int, S: int, nh: int, dh: int, causal: bool = True):
    """Flash attention over a fused ``[B*S, 3*nh*dh]`` projection output -> ``[B*S, nh*dh]``."""
    return _Attention.apply(qkv.contiguous(), B, S, nh, dh, causal)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, nheads, dh, S, pos_offset, theta):
        ctx.args = (nheads, dh, S, pos_offset, theta)
        return E.rope_(x.clone(), nheads, dh, S, pos_offset=pos_offset, theta=theta)

    @staticmethod
    def backward(ctx, dy):
        nheads, dh, S, pos_offset, theta = ctx.args
        return (E.rope_(dy.clone(), nheads, dh, S, pos_offset=pos_offset, theta=theta,
                        inverse=True), None, None, None, None, None)


def rope(x, nheads: int, dh: int, S: int, pos_offset: int = 0, theta: float = 10000.0):
    """Rotary embedding of the first ``nheads * dh`` columns of ``x [B*S, >=nheads*dh]``."""
    return _Rope.apply(x, nheads, dh, S, pos_offset, theta)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return E.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return E.swiglu_bwd(gu, dy.contiguous())


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dimension."""
    x2, shape = _flat(gate_up)
    return _SwiGLU.apply(x2.contiguous()).reshape(*shape[:-1], shape[-1] // 2)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return E.gelu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return E.gelu_bwd(x, dy.contiguous())


def gelu(x: torch.Tensor) -> torch.Tensor:
    """Tanh-approximated GELU (the reference's ``math::gelu``, lib.rs:94-99)."""
    x2, shape = _flat(x)
    return _Gelu.apply(x2.contiguous()).reshape(shape)


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, pe, S):
        ctx.save_for_backward(ids)
        ctx.shape = table.shape
        return E.embed_fwd(ids.reshape(-1), table, pe, S)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        g = torch.zeros(ctx.shape, dtype=torch.float32, device=dy.device)
        E.embed_bwd(ids.reshape(-1), dy.contiguous(), g)
        return None, g.to(dy.dtype), None, None


def embedding(ids: torch.Tensor, table: torch.Tensor, pe: Optional[torch.Tensor] = None,
              S: Optional[int] = None) -> torch.Tensor:
    """Rows of ``table`` for ``ids [B, S]`` (+ the sinusoidal table ``pe``) -> ``[B*S, H]``."""
    return _Embedding.apply(ids, table, pe, S if S is not None else ids.shape[-1])


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        T = logits.shape[0]
        g = logits.clone()
        loss_tok = E.cross_entropy_fwd_bwd(g, targets.reshape(-1), 1.0 / T)
        ctx.save_for_backward(g)
        return loss_tok.sum() / T

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return (g.float() * dloss).to(g.dtype), None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean token cross-entropy of ``logits [T, V]``; negative targets are ignored."""
    return _CrossEntropy.apply(logits.contiguous(), targets)


def softmax(x: torch.Tensor) -> torch.Tensor:
    """Row softmax in fp32 (no gradient; the reference's ``math::softmax``, lib.rs:80-88)."""
    return E.softmax_rows(x)
