"""Decode-time ops (``csrc/decode_attn.cu``): attention of one query token per sequence over a
paged KV cache, appending K/V to the pages, and arg-max over the vocabulary."""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib

PAGE = 64


def kv_write(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             page_table: torch.Tensor, pos0: torch.Tensor, tokens_per_seq: int, nh: int,
             dh: int) -> None:
    """Store ``k``/``v`` (``[B*tokens_per_seq, nh*dh]`` views) at positions
    ``pos0[b] + (t % tokens_per_seq)`` of each sequence's pages."""
    T = k.shape[0]
    max_pages = page_table.shape[1]
    if not k.is_cuda:
        kc = k_cache.view(-1, PAGE, nh * dh)
        vc = v_cache.view(-1, PAGE, nh * dh)
        for t in range(T):
            b = t // tokens_per_seq
            pos = int(pos0[b]) + t % tokens_per_seq
            page = int(page_table[b, pos // PAGE])
            kc[page, pos % PAGE] = k[t, :nh * dh].to(kc.dtype)
            vc[page, pos % PAGE] = v[t, :nh * dh].to(vc.dtype)
        return
    st = _lib.status_buffer(k.device)
    rc = _lib.lib().cb_kv_write(_lib.ptr(k), _lib.ptr(v), k.stride(0), v.stride(0),
                                _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(page_table),
                                max_pages, _lib.ptr(pos0), T, tokens_per_seq, nh, dh, _lib.ptr(st),
                                _lib.stream_ptr())
    _lib.check_rc(rc, "cb_kv_write")


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     page_table: torch.Tensor, ctx_len: torch.Tensor, nh: int, dh: int,
                     scale: Optional[float] = None, splits: int = 0,
                     nkv: Optional[int] = None) -> torch.Tensor:
    """``q`` is a ``[B, nh*dh]`` view; returns ``[B, nh*dh]``.  The cache holds ``nkv`` heads
    (default ``nh``); with fewer, query head ``h`` reads head ``h // (nh // nkv)``.  ``splits`` cuts every context
    into that many pieces handled by separate CTAs and merged afterwards; ``0`` picks the count
    that gives about four CTAs per SM (bounded so that a piece keeps at least 256 tokens of the
    longest context the page table allows)."""
    B = q.shape[0]
    if splits <= 0:
        ctas = max(1, B * nh)
        splits = max(1, min(16, (4 * 148 + ctas - 1) // ctas,
                            (page_table.shape[1] * PAGE) // 256 or 1))
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    nkv = nkv or nh
    if not q.is_cuda:
        out = torch.zeros((B, nh * dh), dtype=q.dtype)
        kc = k_cache.view(-1, PAGE, nkv, dh).float()
        vc = v_cache.view(-1, PAGE, nkv, dh).float()
        for b in range(B):
            n = int(ctx_len[b])
            pages = page_table[b, :(n + PAGE - 1) // PAGE].long()
            K = kc[pages].reshape(-1, nkv, dh)[:n].repeat_interleave(nh // nkv, 1)
            V = vc[pages].reshape(-1, nkv, dh)[:n].repeat_interleave(nh // nkv, 1)
            qq = q[b, :nh * dh].float().view(nh, dh)
            s = torch.einsum("hd,nhd->hn", qq, K) * scale
            p = torch.softmax(s, -1)
            out[b] = torch.einsum("hn,nhd->hd", p, V).reshape(-1).to(q.dtype)
        return out
    out = torch.empty((B, nh * dh), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((B, nh, splits, dh), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, splits, 2), dtype=torch.float32, device=q.device)
    rc = _lib.lib().cb_decode_attn(_lib.ptr(q), q.stride(0), _lib.ptr(k_cache), _lib.ptr(v_cache),
                                   _lib.ptr(page_table), page_table.shape[1], _lib.ptr(ctx_len),
                                   _lib.ptr(out), out.stride(0), _lib.ptr(part_o),
                                   _lib.ptr(part_ml), B, nh, nkv, dh, splits, ctypes.c_float(scale),
                                   _lib.stream_ptr())
    _lib.check_rc(rc, "cb_decode_attn", launches=2 if splits > 1 else 1)
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Arg-max over the last dimension of ``[B, V]`` logits -> int64 ``[B]`` (first index wins)."""
    if not logits.is_cuda:
        return logits.float().argmax(-1)
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    rc = _lib.lib().cb_argmax(_lib.ptr(logits), logits.stride(0), B, V, _lib.ptr(out),
                              _lib.stream_ptr())
    _lib.check_rc(rc, "cb_argmax")
    return out
