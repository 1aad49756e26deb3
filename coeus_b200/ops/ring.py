"""Helpers of context-parallel attention (``csrc/ring.cu``): merging partial attention results,
fp32 accumulation of bf16 gradient slices, reduction into a peer's buffer, fp32 -> bf16 rows.
The reference materialises one S x S score matrix per head on one device
(plugins/model-transformer/src/lib.rs:237-277) and has nothing of the kind."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def merge_partial(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_p: torch.Tensor,
                  lse_p: torch.Tensor, B: int, S: int, nh: int, dh: int, first: bool) -> None:
    """In place: ``(o_acc fp32 [B*S, nh*dh], lse_acc [B, nh, S])`` absorbs ``(o_p, lse_p)``."""
    if not o_acc.is_cuda:
        op = o_p.float().reshape(B, S, nh, dh)
        if first:
            o_acc.copy_(op.reshape(B * S, nh * dh))
            lse_acc.copy_(lse_p)
            return
        ln = torch.logaddexp(lse_acc, lse_p)
        wa = torch.exp(lse_acc - ln).transpose(1, 2)[..., None]      # [B, S, nh, 1]
        wp = torch.exp(lse_p - ln).transpose(1, 2)[..., None]
        o_acc.copy_((o_acc.reshape(B, S, nh, dh) * wa + op * wp).reshape(B * S, nh * dh))
        lse_acc.copy_(ln)
        return
    assert o_acc.dtype == torch.float32 and o_acc.is_contiguous() and o_p.stride(1) == 1
    rc = _lib.lib().cb_attn_merge(_lib.ptr(o_acc), _lib.ptr(lse_acc), _lib.ptr(o_p), o_p.stride(0),
                                  _lib.ptr(lse_p), B, S, nh, dh, int(first), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_attn_merge")


def accum_rows(acc: torch.Tensor, x: torch.Tensor) -> None:
    """``acc (fp32) += x`` for 2-D row-strided views of equal shape."""
    if not acc.is_cuda:
        acc += x.float()
        return
    assert acc.dtype == torch.float32 and x.dtype == torch.bfloat16
    assert acc.stride(1) == 1 and x.stride(1) == 1 and acc.shape == x.shape
    rc = _lib.lib().cb_accum_rows(_lib.ptr(acc), acc.stride(0), _lib.ptr(x), x.stride(0),
                                  x.shape[0], x.shape[1], _lib.stream_ptr())
    _lib.check_rc(rc, "cb_accum_rows")


def peer_add_f32(dst_ptr: int, src: torch.Tensor) -> None:
    """``*dst_ptr[0:n] += src`` where ``dst_ptr`` is a (possibly peer-mapped) device address."""
    assert src.is_cuda and src.dtype == torch.float32 and src.is_contiguous()
    rc = _lib.lib().cb_peer_add_f32(ctypes.c_void_p(dst_ptr), _lib.ptr(src),
                                    ctypes.c_size_t(src.numel()), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_peer_add_f32")


def cast_rows(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0) -> None:
    """``dst (bf16 rows) = src (fp32 rows) * scale`` for row-strided 2-D views."""
    if not src.is_cuda:
        dst.copy_((src * scale).to(dst.dtype))
        return
    assert src.dtype == torch.float32 and dst.dtype == torch.bfloat16 and src.shape == dst.shape
    rc = _lib.lib().cb_cast_rows(_lib.ptr(src), src.stride(0), _lib.ptr(dst), dst.stride(0),
                                 src.shape[0], src.shape[1], ctypes.c_float(scale),
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "cb_cast_rows")
