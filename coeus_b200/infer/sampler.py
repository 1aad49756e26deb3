"""Next-token selection from logits: greedy (the arg-max kernel) or temperature / top-k / top-p
sampling (the fields of the reference's ``BasicGenerationConfig``, src/core/model.rs:719-753,
which the reference declares but never consumes)."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.decode import argmax_rows


def select(logits: torch.Tensor, temperature: float = 0.0, top_k: Optional[int] = None,
           top_p: Optional[float] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``logits [B, V]`` -> token ids ``[B]`` (int64).  ``temperature <= 0`` means greedy."""
    if temperature is None or temperature <= 0.0:
        return argmax_rows(logits)
    x = logits.float() / temperature
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
