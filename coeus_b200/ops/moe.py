"""Mixture-of-experts routing and token permutation (``csrc/moe.cu``); CPU tensors take the
PyTorch restatement of the same rules (top-k with ties to the lowest expert index, slots handed
out in token order, pairs beyond the capacity dropped)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def route(logits: torch.Tensor, k: int, capacity: int
          ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``logits [T, E]`` fp32 -> ``(expert [T,k] int32, weight [T,k] fp32 (sums to 1 per token),
    probs [T,E] fp32, slot [T,k] int32 (-1 = dropped), counts [E] int32)``."""
    T, E = logits.shape
    if not logits.is_cuda:
        probs = torch.softmax(logits.float(), -1)
        # stable top-k with ties to the lowest index
        order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :k]
        w = probs.gather(1, order)
        w = w / w.sum(-1, keepdim=True)
        expert = order.to(torch.int32)
        slot = torch.full((T, k), -1, dtype=torch.int32)
        counts = torch.zeros(E, dtype=torch.int32)
        flat = expert.reshape(-1)
        for e in range(E):
            idx = (flat == e).nonzero()[:, 0]
            pos = torch.arange(idx.numel(), dtype=torch.int32)
            keep = pos < capacity
            slot.view(-1)[idx[keep]] = pos[keep]
            counts[e] = min(idx.numel(), capacity)
        return expert, w, probs, slot, counts
    logits = logits.float().contiguous()
    dev = logits.device
    expert = torch.empty((T, k), dtype=torch.int32, device=dev)
    weight = torch.empty((T, k), dtype=torch.float32, device=dev)
    probs = torch.empty((T, E), dtype=torch.float32, device=dev)
    slot = torch.empty((T, k), dtype=torch.int32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    rc = _lib.lib().cb_moe_route(_lib.ptr(logits), T, E, k, capacity, _lib.ptr(expert),
                                 _lib.ptr(weight), _lib.ptr(probs), _lib.ptr(slot),
                                 _lib.ptr(counts), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_moe_route", launches=2)
    return expert, weight, probs, slot, counts


def gather_rows(src: torch.Tensor, expert: torch.Tensor, slot: torch.Tensor, dst: torch.Tensor,
                capacity: int, scale: Optional[torch.Tensor] = None) -> None:
    """``dst[e*C + slot] = src[token] * scale[token,k]`` for every kept (token, k) pair; ``dst``
    is ``[E*C, H]``."""
    T, K = expert.shape
    H = src.shape[1]
    if not src.is_cuda:
        keep = slot.reshape(-1) >= 0
        rows = (expert.reshape(-1).long() * capacity + slot.reshape(-1).long())[keep]
        tok = torch.arange(T).repeat_interleave(K)[keep]
        vals = src[tok].float()
        if scale is not None:
            vals = vals * scale.reshape(-1)[keep][:, None]
        dst[rows] = vals.to(dst.dtype)
        return
    rc = _lib.lib().cb_moe_gather_rows(_lib.ptr(src), src.stride(0), _lib.ptr(expert),
                                       _lib.ptr(slot), _lib.ptr(scale), _lib.ptr(dst), T, K, H,
                                       capacity, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_moe_gather_rows")


def combine_rows(ret: torch.Tensor, expert: torch.Tensor, slot: torch.Tensor, capacity: int,
                 w: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None
                 ) -> torch.Tensor:
    """``out[token] = resid[token] + sum_k w[token,k] * ret[e_k*C + slot_k]``."""
    T, K = expert.shape
    H = ret.shape[1]
    if not ret.is_cuda:
        out = resid.float().clone() if resid is not None else torch.zeros((T, H))
        for k in range(K):
            keep = slot[:, k] >= 0
            rows = expert[:, k].long() * capacity + slot[:, k].long().clamp(min=0)
            v = ret[rows].float() * keep[:, None]
            if w is not None:
                v = v * w[:, k][:, None]
            out += v
        return out.to(ret.dtype)
    out = torch.empty((T, H), dtype=ret.dtype, device=ret.device)
    rc = _lib.lib().cb_moe_combine_rows(_lib.ptr(ret), _lib.ptr(expert), _lib.ptr(slot), _lib.ptr(w),
                                        _lib.ptr(resid), _lib.ptr(out), T, K, H, capacity,
                                        _lib.stream_ptr())
    _lib.check_rc(rc, "cb_moe_combine_rows")
    return out


def pair_dot(a: torch.Tensor, ret: torch.Tensor, expert: torch.Tensor, slot: torch.Tensor,
             capacity: int) -> torch.Tensor:
    """``dots[token,k] = <a[token], ret[e_k*C + slot_k]>`` (0 for dropped pairs), fp32."""
    T, K = expert.shape
    H = a.shape[1]
    if not a.is_cuda:
        keep = slot >= 0
        rows = expert.long() * capacity + slot.long().clamp(min=0)
        return (a.float()[:, None, :] * ret[rows].float()).sum(-1) * keep
    dots = torch.empty((T, K), dtype=torch.float32, device=a.device)
    rc = _lib.lib().cb_moe_pair_dot(_lib.ptr(a), _lib.ptr(ret), _lib.ptr(expert), _lib.ptr(slot),
                                    _lib.ptr(dots), T, K, H, capacity, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_moe_pair_dot")
    return dots
