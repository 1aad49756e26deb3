"""bf16 GEMM with fused epilogues on the tcgen05 tensor cores (``csrc/gemm.cu``).

``gemm`` is the general entry; ``linear_fwd`` / ``linear_dgrad`` / ``linear_wgrad`` are the
three products of a linear layer whose weight is stored ``[in, out]`` row-major, the layout
``math::matmul`` uses in the reference (plugins/model-transformer/src/lib.rs:50-74).

CPU tensors take a float32 PyTorch restatement of the same math (the oracle the GPU tests
compare against); CUDA tensors always run the hand-written kernel.
"""
from __future__ import annotations

import ctypes
import os
import math
from typing import Optional

import torch

from . import _lib

EPI = {"none": 0, "gelu": 1, "dgelu": 2}
_OUT_BF16, _OUT_F32, _OUT_F32_ATOMIC = 0, 1, 2


def _gelu_ref(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)))


def _gelu_grad_ref(x: torch.Tensor) -> torch.Tensor:
    x2 = x * x
    u = 0.7978845608028654 * x * (1.0 + 0.044715 * x2)
    t = torch.tanh(u)
    du = 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * x2)
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * du


_PAIRS = os.environ.get("COEUS_GEMM_PAIRS", "1") != "0"


def use_cta_pairs(on: bool) -> None:
    """Run the 256-wide plain GEMMs on clusters of two CTAs (``tcgen05`` ``cta_group::2``): one
    256 x 256 tile per pair, each CTA staging its 128 rows of A and half of the B rows, which
    halves the B traffic into every SM (measured +5 % on the layer shapes, +15 % on the LM head).
    On by default; ``COEUS_GEMM_PAIRS=0`` or ``use_cta_pairs(False)`` selects single CTAs."""
    global _PAIRS
    _PAIRS = bool(on)


def _pick_bn(M: int, N: int) -> int:
    """N tile of the GEMM: 256 whenever N allows it (a 128-wide tile halves the arithmetic
    intensity per shared-memory byte and measured ~30 % slower per FLOP, which outweighs the
    better wave quantisation it sometimes gives).  The value 512 stands for "256 wide on CTA
    pairs" and is chosen when the matrix has at least one full 256-row tile."""
    if N <= 128:
        return 128
    return 512 if _PAIRS and M >= 256 else 256


def _pick_ksplit(tiles: int, kblocks: int, sms: int = 148, max_split: int = 16,
                 epilogue_kblocks: int = 25) -> int:
    """Split of the contraction dimension for the weight-gradient GEMM.  A work unit (one tile of
    one split) costs its k-blocks plus an atomic fp32 epilogue worth about ``epilogue_kblocks``
    k-blocks (measured on 256 x 256 tiles: 9.1 us against 0.36 us per k-block; a split multiplies
    the epilogues, and with one unit per CTA nothing hides them), and the launch takes
    ``ceil(units / sms)`` rounds of units: the split with the smallest product wins, each split
    keeping at least 8 k-blocks."""
    best, best_cost = 1, None
    for ks in range(1, max_split + 1):
        if ks > 1 and kblocks // ks < 8:
            break
        rounds = -(-(tiles * ks) // sms)
        cost = rounds * (-(-kblocks // ks) + epilogue_kblocks)
        if best_cost is None or cost < best_cost:
            best, best_cost = ks, cost
    return best


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         resid: Optional[torch.Tensor] = None, epi: str = "none",
         aux_in: Optional[torch.Tensor] = None, aux_out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, alpha: float = 1.0,
         ksplit: int = 1, bn: Optional[int] = None, max_ctas: int = 0,
         _discard: bool = False, dropout: Optional[tuple] = None) -> torch.Tensor:
    """``out[M,N] = epilogue(alpha * A @ B^T)`` with A logical ``[M,K]`` and B logical ``[N,K]``.

    ``dropout=(thr, key)`` drops elements of the epilogue value (after bias and activation,
    before ``resid`` is added) with the mask of :func:`coeus_b200.ops.elementwise.dropout_mask`
    and scales the kept ones by ``256 / (256 - thr)`` (bf16 output, ``N % 32 == 0``).

    ``a_mn`` / ``b_mn`` say that the tensor passed is the transpose in memory (``[K,M]`` /
    ``[K,N]`` row-major).  ``accumulate=True`` adds into an fp32 ``out`` with atomic adds,
    which is what allows ``ksplit > 1``.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    if accumulate:
        out_dtype = torch.float32
        if out is None:
            raise ValueError("gemm: accumulate=True needs an fp32 `out`")
    if out is None:
        if not a.is_cuda and a.dtype != torch.bfloat16 and out_dtype == torch.bfloat16:
            out_dtype = a.dtype  # the CPU oracle keeps the precision it is given
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if not a.is_cuda:
        A = (a.t() if a_mn else a).float()
        B = (b.t() if b_mn else b).float()
        v = alpha * (A @ B.t())
        if bias is not None:
            v = v + bias.float()
        if epi == "gelu":
            if aux_out is not None:
                aux_out.copy_(v.to(aux_out.dtype))
            v = _gelu_ref(v)
        elif epi == "dgelu":
            v = v * _gelu_grad_ref(aux_in.float())
        if dropout is not None and dropout[0] > 0:
            from .elementwise import dropout_mask
            keep = dropout_mask(M, N, dropout[0], dropout[1], v.device)
            v = torch.where(keep, v * (256.0 / (256 - dropout[0])), torch.zeros((), device=v.device))
        if resid is not None:
            v = v + resid.float()
        if accumulate:
            out.add_(v.to(out.dtype))
        else:
            out.copy_(v.to(out.dtype))
        return out

    for t in (a, b):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise ValueError("gemm: operands must be bf16 with unit inner stride")
    if out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("gemm: bad output tensor")
    out_mode = _OUT_F32_ATOMIC if accumulate else (
        _OUT_F32 if out.dtype == torch.float32 else _OUT_BF16)
    if _discard:   # profiling aid: run the main loop, drop the result
        out_mode = 3
    if bn is None:
        bn = _pick_bn(M, N)
    aux = aux_in if aux_in is not None else aux_out
    st = _lib.status_buffer(a.device)
    if dropout is not None and dropout[0] > 0:
        if aux is not None or out_mode != _OUT_BF16 or ksplit != 1 or N % 32:
            raise ValueError("gemm: dropout needs a plain bf16 output with N % 32 == 0")
        rc = _lib.lib().cb_gemm_bf16_dropout(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
            out.stride(0), int(a_mn), int(b_mn), _lib.ptr(bias), _lib.ptr(resid),
            resid.stride(0) if resid is not None else 0, EPI[epi], ctypes.c_float(alpha), bn,
            int(dropout[0]), ctypes.c_uint(dropout[1] & 0xFFFFFFFF), _lib.ptr(st), max_ctas,
            _lib.stream_ptr())
        _lib.check_rc(rc, "cb_gemm_bf16_dropout")
        return out
    rc = _lib.lib().cb_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
        out.stride(0), int(a_mn), int(b_mn), _lib.ptr(bias), _lib.ptr(resid),
        resid.stride(0) if resid is not None else 0, _lib.ptr(aux_in), _lib.ptr(aux_out),
        aux.stride(0) if aux is not None else 0, EPI[epi], out_mode, ctypes.c_float(alpha),
        ksplit, bn, _lib.ptr(st), max_ctas, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_gemm_bf16")
    return out


def gemm_grouped(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
                 out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                 accumulate: bool = False, alpha: float = 1.0, ksplit: int = 1,
                 max_ctas: int = 0) -> torch.Tensor:
    """``out[g] = alpha * A[g] @ B[g]^T`` for every group ``g`` in ONE launch (the experts of a
    mixture-of-experts layer).  ``a`` is ``[G, M, K]`` (``a_mn``: ``[G, K, M]``), ``b`` is
    ``[G, N, K]`` (``b_mn``: ``[G, K, N]``), ``out`` ``[G, M, N]``; groups must lie one after the
    other in memory (``stride(0) == shape[1] * stride(1)``).  The kernel is the persistent
    tcgen05 GEMM with a per-tile group offset on the operand coordinates; it needs ``M`` to be
    a multiple of 128 and ``K`` of 64 so that no tile straddles two groups -- other shapes run
    one launch per group."""
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0]
    Gn = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn else (a.shape[1], a.shape[2])
    N, Kb = (b.shape[2], b.shape[1]) if b_mn else (b.shape[1], b.shape[2])
    if K != Kb:
        raise ValueError(f"gemm_grouped: contraction mismatch {K} vs {Kb}")
    if accumulate:
        out_dtype = torch.float32
        if out is None:
            raise ValueError("gemm_grouped: accumulate=True needs an fp32 `out`")
    if out is None:
        if not a.is_cuda and a.dtype != torch.bfloat16 and out_dtype == torch.bfloat16:
            out_dtype = a.dtype
        out = torch.empty((Gn, M, N), dtype=out_dtype, device=a.device)
    stacked = all(t.stride(2) == 1 and t.stride(0) == t.shape[1] * t.stride(1)
                  for t in (a, b, out))
    if not a.is_cuda or not stacked or M % 128 or K % 64 or Gn == 1:
        for g in range(Gn):
            gemm(a[g], b[g], a_mn=a_mn, b_mn=b_mn, out=out[g], out_dtype=out_dtype,
                 accumulate=accumulate, alpha=alpha, ksplit=ksplit, max_ctas=max_ctas)
        return out
    for t in (a, b):
        if t.dtype != torch.bfloat16:
            raise ValueError("gemm_grouped: operands must be bf16")
    out_mode = _OUT_F32_ATOMIC if accumulate else (
        _OUT_F32 if out.dtype == torch.float32 else _OUT_BF16)
    bn = _pick_bn(M, N)
    st = _lib.status_buffer(a.device)
    rc = _lib.lib().cb_gemm_bf16_grouped(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), Gn, M, N, K, a.stride(1), b.stride(1),
        out.stride(1), int(a_mn), int(b_mn), out_mode, ctypes.c_float(alpha), ksplit, bn,
        _lib.ptr(st), max_ctas, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_gemm_bf16_grouped")
    return out


def linear_wgrad_grouped(x: torch.Tensor, dy: torch.Tensor, grad_w: torch.Tensor, *,
                         max_ctas: int = 0) -> torch.Tensor:
    """``grad_w[g][in,out] += x[g][T,in]^T @ dy[g][T,out]`` for all groups in one launch."""
    Gn, T, Min, Nout = x.shape[0], x.shape[1], x.shape[2], dy.shape[2]
    if _pick_bn(Min, Nout) == 512 and Min % 256 == 0:     # CTA pairs: 256-row tiles, 74 units
        ksplit = _pick_ksplit(Gn * (Min // 256) * ((Nout + 255) // 256), (T + 63) // 64, sms=74)
    else:
        ksplit = _pick_ksplit(Gn * ((Min + 127) // 128) * ((Nout + 255) // 256), (T + 63) // 64)
    return gemm_grouped(x, dy, a_mn=True, b_mn=True, out=grad_w, accumulate=True, ksplit=ksplit,
                        max_ctas=max_ctas)


def linear_fwd(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
               resid: Optional[torch.Tensor] = None, epi: str = "none",
               aux_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               out_dtype: torch.dtype = torch.bfloat16, max_ctas: int = 0,
               dropout: Optional[tuple] = None) -> torch.Tensor:
    """``y[T,out] = dropout(epilogue(x[T,in] @ w[in,out] + bias)) (+ resid)``."""
    return gemm(x, w, b_mn=True, bias=bias, resid=resid, epi=epi, aux_out=aux_out, out=out,
                out_dtype=out_dtype, max_ctas=max_ctas, dropout=dropout)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, *, epi: str = "none",
                 aux_in: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """``dx[T,in] = dy[T,out] @ w[in,out]^T`` (optionally times GELU'(aux_in), plus resid)."""
    return gemm(dy, w, epi=epi, aux_in=aux_in, resid=resid, out=out, max_ctas=max_ctas)


def linear_wgrad(x: torch.Tensor, dy: torch.Tensor, grad_w: torch.Tensor, *,
                 ksplit: Optional[int] = None, max_ctas: int = 0) -> torch.Tensor:
    """``grad_w[in,out] += x[T,in]^T @ dy[T,out]`` accumulated in fp32."""
    T = x.shape[0]
    if ksplit is None:
        bn = _pick_bn(x.shape[1], dy.shape[1])
        if bn == 512:     # CTA pairs: 256-row tiles scheduled over half as many units
            tiles = ((x.shape[1] + 255) // 256) * ((dy.shape[1] + 255) // 256)
            ksplit = _pick_ksplit(tiles, (T + 63) // 64, sms=74)
        else:
            tiles = ((x.shape[1] + 127) // 128) * ((dy.shape[1] + bn - 1) // bn)
            ksplit = _pick_ksplit(tiles, (T + 63) // 64)
    return gemm(x, dy, a_mn=True, b_mn=True, out=grad_w, accumulate=True, ksplit=ksplit,
                max_ctas=max_ctas)
