"""Ulysses sequence parallelism: activations are sharded along the sequence everywhere except
inside attention, where an all-to-all re-shards them along the heads (every rank then sees whole
sequences for ``nh / sp`` heads), the ordinary flash-attention kernel runs, and a second
all-to-all restores the sequence sharding.  Rank ``r`` owns tokens ``[r * S/sp, (r+1) * S/sp)`` of
every sequence.  Same calling surface as :class:`coeus_b200.parallel.cp.ContextParallel`, so the
decoder takes either.  The reference has no sequence parallelism (its attention is one S x S
matrix per head on one device, plugins/model-transformer/src/lib.rs:237-277).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..foundation.error import ProcessingError
from ..ops import attention as A
from .a2a import AllToAll


class UlyssesParallel:
    n_chunks = 1

    def __init__(self, group, device, backend: Optional[str] = None,
                 wait_limit_ms: float = 5000.0) -> None:
        self.a2a = AllToAll(group, device, backend, wait_limit_ms)
        self.rank, self.cp = self.a2a.rank, self.a2a.world
        self.backend = self.a2a.backend

    def shard(self, x: torch.Tensor) -> torch.Tensor:
        """``[B, S, ...] -> [1, B, S/sp, ...]``."""
        S = x.shape[1]
        if S % self.cp:
            raise ProcessingError.invalid_input(f"sequence length {S} not divisible by {self.cp}")
        Sl = S // self.cp
        return x[:, self.rank * Sl:(self.rank + 1) * Sl].contiguous()[None]

    def position_offsets(self, Sl: int) -> Tuple[int]:
        return (self.rank * Sl,)

    # [B*Sl, W*H] (all heads, my tokens) -> [B*S, W*Hl] (my heads, all tokens)
    def _seq_to_heads(self, t: torch.Tensor, B: int, Sl: int, W: int, Hl: int) -> torch.Tensor:
        sp = self.cp
        send = t.reshape(B, Sl, W, sp, Hl).permute(3, 0, 1, 2, 4).contiguous()
        recv = self.a2a.exchange(send)                       # [sp(src), B, Sl, W, Hl]
        return recv.permute(1, 0, 2, 3, 4).reshape(B * sp * Sl, W * Hl)

    def _heads_to_seq(self, t: torch.Tensor, B: int, Sl: int, W: int, Hl: int) -> torch.Tensor:
        sp = self.cp
        send = t.reshape(B, sp, Sl, W, Hl).permute(1, 0, 2, 3, 4).contiguous()
        recv = self.a2a.exchange(send)                       # [sp(head group), B, Sl, W, Hl]
        return recv.permute(1, 2, 3, 0, 4).reshape(B * Sl, W * sp * Hl)

    def attention_fwd(self, qkv: torch.Tensor, B: int, Sl: int, nh: int, dh: int):
        if nh % self.cp:
            raise ProcessingError.invalid_input(
                f"{nh} heads cannot be split over {self.cp} ranks")
        nhl = nh // self.cp
        Hl, S = nhl * dh, Sl * self.cp
        full = self._seq_to_heads(qkv, B, Sl, 3, Hl)         # [B*S, 3*Hl]
        q, k, v = full[:, :Hl], full[:, Hl:2 * Hl], full[:, 2 * Hl:]
        o, lse = A.attention_fwd(q, k, v, B, S, nhl, dh, causal=True)
        return self._heads_to_seq(o, B, Sl, 1, Hl), (full, o, lse)

    def attention_bwd(self, do: torch.Tensor, qkv: torch.Tensor, o_local: torch.Tensor, ctx,
                      B: int, Sl: int, nh: int, dh: int,
                      dqkv: Optional[torch.Tensor] = None) -> torch.Tensor:
        full, o, lse = ctx
        nhl = nh // self.cp
        Hl, S = nhl * dh, Sl * self.cp
        do_full = self._seq_to_heads(do, B, Sl, 1, Hl)
        q, k, v = full[:, :Hl], full[:, Hl:2 * Hl], full[:, 2 * Hl:]
        fused = torch.empty((B * S, 3 * Hl), dtype=full.dtype, device=full.device)
        A.attention_bwd(do_full, q, k, v, o, lse, B, S, nhl, dh, causal=True, dqkv=fused)
        out = self._heads_to_seq(fused, B, Sl, 3, Hl)
        if dqkv is not None:
            dqkv.copy_(out)
            return dqkv
        return out
