"""Next-token selection from logits: greedy (the arg-max kernel) or temperature / top-k / top-p
sampling (the fields of the reference's ``BasicGenerationConfig``, src/core/model.rs:719-753,
which the reference declares but never consumes)."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.decode import argmax_rows


def apply_repetition_penalty(logits: torch.Tensor, history: torch.Tensor, penalty: float
                             ) -> torch.Tensor:
    """Divide the positive (multiply the negative) logits of tokens that already occur in
    ``history [B, n]`` (int64, entries < 0 ignored) by ``penalty``; returns fp32 logits."""
    x = logits.float().clone()
    if penalty == 1.0 or history.numel() == 0:
        return x
    valid = history >= 0
    idx = history.clamp_min(0)
    # counts, not a boolean scatter: an ignored entry is clamped onto id 0 and must not erase it
    seen = torch.zeros_like(x, dtype=torch.int32).scatter_add_(1, idx, valid.to(torch.int32)) > 0
    pen = torch.where(x > 0, x / penalty, x * penalty)
    return torch.where(seen, pen, x)


def select(logits: torch.Tensor, temperature: float = 0.0, top_k: Optional[int] = None,
           top_p: Optional[float] = None, generator: Optional[torch.Generator] = None,
           min_p: Optional[float] = None, history: Optional[torch.Tensor] = None,
           repetition_penalty: float = 1.0) -> torch.Tensor:
    """``logits [B, V]`` -> token ids ``[B]`` (int64).  ``temperature <= 0`` means greedy.
    ``min_p`` drops tokens whose probability is below ``min_p`` times the most likely one's;
    ``history`` + ``repetition_penalty`` discourage tokens that were already produced."""
    if history is not None and repetition_penalty != 1.0:
        logits = apply_repetition_penalty(logits, history, repetition_penalty)
        if temperature is None or temperature <= 0.0:
            return logits.argmax(-1)
    if temperature is None or temperature <= 0.0:
        return argmax_rows(logits)
    x = logits.float() / temperature
    if min_p is not None and 0.0 < min_p < 1.0:
        probs = torch.softmax(x, -1)
        x = x.masked_fill(probs < min_p * probs.amax(-1, keepdim=True), float("-inf"))
    if top_k is not None and 0 < top_k < x.shape[-1]:
        kth = torch.topk(x, top_k, dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        sorted_x, idx = torch.sort(x, dim=-1, descending=True)
        probs = torch.softmax(sorted_x, -1)
        cum = probs.cumsum(-1)
        drop = cum - probs > top_p
        sorted_x = sorted_x.masked_fill(drop, float("-inf"))
        x = torch.full_like(x, float("-inf")).scatter(-1, idx, sorted_x)
    probs = torch.softmax(x, -1)
    return torch.multinomial(probs, 1, generator=generator)[:, 0]
