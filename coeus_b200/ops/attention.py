"""Flash-style attention on tcgen05 (``csrc/attention_fwd.cu``: two query tiles per CTA with the
probabilities kept in tensor memory; ``csrc/attention_bwd.cu``).

Tensors are token-major: ``q``, ``k``, ``v`` are ``[B*S, nh*dh]`` views (they may be column
slices of one fused ``[B*S, 3*nh*dh]`` projection output), ``o`` is ``[B*S, nh*dh]``.  The
``S x S`` score matrix of the reference (plugins/model-transformer/src/lib.rs:237-277) is never
materialised.  CPU tensors use a float32 PyTorch restatement.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch

from . import _lib

# ``COEUS_ATTN_POLY=1`` makes the forward kernel evaluate a quarter of its exponentials as a
# polynomial on the FMA pipe instead of the special-function unit (measured slower on B200 at
# dh 64 and 128 with the present instruction mix, hence off by default).
FWD_POLY = int(os.environ.get("COEUS_ATTN_POLY", "0"))


def _ref_fwd(q, k, v, B, S, nh, dh, scale, causal):
    qf = q.float().reshape(B, S, nh, dh).transpose(1, 2)
    nkv = k.shape[1] // dh
    kf = k.float().reshape(B, S, nkv, dh).transpose(1, 2)
    vf = v.float().reshape(B, S, nkv, dh).transpose(1, 2)
    if nkv != nh:          # grouped-query attention: query head h reads K/V head h // group
        kf = kf.repeat_interleave(nh // nkv, 1)
        vf = vf.repeat_interleave(nh // nkv, 1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.softmax(s, -1)
    o = (p @ vf).transpose(1, 2).reshape(B * S, nh * dh)
    return o, lse, p, (qf, kf, vf)


def flash_dropout_ok(q: torch.Tensor, S: int, dh: int) -> bool:
    """Whether the flash kernels can apply dropout themselves for this call (else the
    materialised path :func:`attention_dropout_fwd` / ``_bwd`` is the one to use)."""
    return q.is_cuda and S % 4 == 0 and dh in (64, 128)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, B: int, S: int, nh: int,
                  dh: int, *, causal: bool = True, scale: Optional[float] = None,
                  dropout: Optional[Tuple[int, int]] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(o [B*S, nh*dh], lse [B, nh, S] fp32)``.  ``k`` and ``v`` may hold fewer heads
    than ``q`` (``[B*S, nkv*dh]``, ``nkv`` dividing ``nh``): grouped-query attention, query head
    ``h`` reading K/V head ``h // (nh // nkv)`` inside the kernel.  ``dropout = (thr, key)``
    drops the probabilities inside the kernel (mask of :func:`..elementwise.dropout_mask` over the
    ``[B*nh*S, S]`` probability matrix; nothing is stored, the backward pass recomputes it)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    nkv = k.shape[1] // dh
    thr, key = dropout if dropout is not None else (0, 0)
    if thr and not flash_dropout_ok(q, S, dh):
        return attention_dropout_fwd(q, k, v, B, S, nh, dh, thr, key, causal=causal, scale=scale)
    if not q.is_cuda:
        o, lse, _, _ = _ref_fwd(q, k, v, B, S, nh, dh, scale, causal)
        return o.to(q.dtype), lse
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(1) == 1
    o = torch.empty((B * S, nh * dh), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
    st = _lib.status_buffer(q.device)
    rc = _lib.lib().cb_attn_fwd_dropout(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), B, S, nh, nkv, dh,
        q.stride(0), k.stride(0), v.stride(0), o.stride(0), ctypes.c_float(scale),
        int(causal), FWD_POLY, int(thr), ctypes.c_uint(key & 0xFFFFFFFF), _lib.ptr(st), 0,
        _lib.stream_ptr())
    _lib.check_rc(rc, "cb_attn_fwd")
    return o, lse


def attention_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  o: torch.Tensor, lse: torch.Tensor, B: int, S: int, nh: int, dh: int, *,
                  causal: bool = True, scale: Optional[float] = None,
                  dqkv: Optional[torch.Tensor] = None,
                  dropout: Optional[Tuple[int, int]] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(dq, dk, dv)`` as column slices of one fused ``[B*S, 3*nh*dh]`` bf16 buffer
    (``dqkv`` if given), ready to be the input of the QKV projection's backward GEMMs.
    ``dropout``: the ``(thr, key)`` the forward pass was given."""
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    H = nh * dh
    thr, key = dropout if dropout is not None else (0, 0)
    if thr and not flash_dropout_ok(q, S, dh):
        return attention_dropout_bwd(do, q, k, v, o, lse, B, S, nh, dh, thr, key, causal=causal,
                                     scale=scale, dqkv=dqkv)
    if not q.is_cuda:
        _, lse_own, p, (qf, kf, vf) = _ref_fwd(q, k, v, B, S, nh, dh, scale, causal)
        # probabilities relative to the normaliser that was passed in (it covers more keys than
        # these when the call is one block pair of ring attention), as the kernel computes them
        p = p * torch.exp(lse_own - lse.float())[..., None]
        dof = do.float().reshape(B, S, nh, dh).transpose(1, 2)
        of = o.float().reshape(B, S, nh, dh).transpose(1, 2)
        dv = p.transpose(-1, -2) @ dof
        dp = dof @ vf.transpose(-1, -2)
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = ds @ kf
        dk = ds.transpose(-1, -2) @ qf
        out = dqkv if dqkv is not None else torch.empty((B * S, 3 * H), dtype=q.dtype)
        for i, t in enumerate((dq, dk, dv)):
            out[:, i * H:(i + 1) * H] = t.transpose(1, 2).reshape(B * S, H).to(out.dtype)
        return out[:, :H], out[:, H:2 * H], out[:, 2 * H:]
    out = dqkv if dqkv is not None else torch.empty((B * S, 3 * H), dtype=torch.bfloat16,
                                                    device=q.device)
    dq_acc = torch.zeros((B * S, H), dtype=torch.float32, device=q.device)
    delta = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
    st = _lib.status_buffer(q.device)
    rc = _lib.lib().cb_attn_bwd_dropout(
        _lib.ptr(do), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse),
        _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(out), B, S, nh, dh, do.stride(0), q.stride(0),
        k.stride(0), v.stride(0), o.stride(0), out.stride(0), ctypes.c_float(scale), int(causal),
        int(thr), ctypes.c_uint(key & 0xFFFFFFFF), _lib.ptr(st), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_attn_bwd", launches=3)
    return out[:, :H], out[:, H:2 * H], out[:, 2 * H:]


# ------------------------------------------------------------------------------ dropout path
# Attention with dropout on the probabilities by materialising the score matrix with tensor ops
# (on either device): the oracle of the flash kernels' own dropout and the path of the cases they
# do not cover (CPU tensors, a sequence length that is not a multiple of four).  The mask is the
# counter-based one of
# :func:`coeus_b200.ops.elementwise.dropout_mask` over the ``[B*nh*S, S]`` probability matrix, so
# nothing is stored between the passes and CPU and GPU agree.
def attention_dropout_fwd(q, k, v, B, S, nh, dh, thr, key, *, causal=True, scale=None):
    """``(o, lse)`` like :func:`attention_fwd`, with ``P`` dropped before ``P @ V``."""
    from .elementwise import dropout_mask
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    _, lse, p, (_, _, vf) = _ref_fwd(q, k, v, B, S, nh, dh, scale, causal)
    keep = dropout_mask(B * nh * S, S, thr, key, q.device).view(B, nh, S, S)
    pd = torch.where(keep, p * (256.0 / (256 - thr)), torch.zeros((), device=q.device))
    o = (pd @ vf).transpose(1, 2).reshape(B * S, nh * dh)
    return o.to(q.dtype), lse


def attention_dropout_bwd(do, q, k, v, o, lse, B, S, nh, dh, thr, key, *, causal=True, scale=None,
                          dqkv=None):
    """``(dq, dk, dv)`` of :func:`attention_dropout_fwd` (views of one ``[B*S, H + 2*Hkv]``
    buffer)."""
    from .elementwise import dropout_mask
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    H, Hkv = nh * dh, k.shape[1]
    nkv = Hkv // dh
    _, _, p, (qf, kf, vf) = _ref_fwd(q, k, v, B, S, nh, dh, scale, causal)
    sc = 256.0 / (256 - thr)
    keep = dropout_mask(B * nh * S, S, thr, key, q.device).view(B, nh, S, S)
    zero = torch.zeros((), device=q.device)
    pd = torch.where(keep, p * sc, zero)
    dof = do.float().reshape(B, S, nh, dh).transpose(1, 2)
    of = o.float().reshape(B, S, nh, dh).transpose(1, 2)
    dv = pd.transpose(-1, -2) @ dof
    dp = torch.where(keep, (dof @ vf.transpose(-1, -2)) * sc, zero)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    if nkv != nh:        # gradients of a shared K/V head: the sum over its query heads
        g = nh // nkv
        dk = dk.reshape(B, nkv, g, S, dh).sum(2)
        dv = dv.reshape(B, nkv, g, S, dh).sum(2)
    out = dqkv if dqkv is not None else torch.empty((B * S, H + 2 * Hkv), dtype=q.dtype,
                                                    device=q.device)
    out[:, :H] = dq.transpose(1, 2).reshape(B * S, H).to(out.dtype)
    out[:, H:H + Hkv] = dk.transpose(1, 2).reshape(B * S, Hkv).to(out.dtype)
    out[:, H + Hkv:H + 2 * Hkv] = dv.transpose(1, 2).reshape(B * S, Hkv).to(out.dtype)
    return out[:, :H], out[:, H:H + Hkv], out[:, H + Hkv:H + 2 * Hkv]
