"""Paged KV cache: fixed-size pages of 64 tokens handed out from a free list, one page table row
per sequence, so the context is bounded by device memory and not by a dense ``[B, S_max]``
allocation.  One pair of ``[num_pages, 64, heads, dh]`` bf16 tensors per layer."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..foundation.error import ResourceError
from ..ops.decode import PAGE


class PagedKVCache:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, num_pages: int,
                 max_seqs: int, max_pages_per_seq: int, device, dtype=torch.bfloat16) -> None:
        self.num_layers, self.nh, self.dh = num_layers, num_heads, head_dim
        self.num_pages = num_pages
        self.device = torch.device(device)
        shape = (num_pages, PAGE, num_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        self.page_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32,
                                      device=self.device)
        self.free: List[int] = list(range(num_pages - 1, -1, -1))
        self.owned: Dict[int, List[int]] = {}
        # pages can be shared (a cached prompt prefix used by several sequences): a page returns
        # to the free list when its last holder lets go
        self.refs: List[int] = [0] * num_pages
        self.lengths = torch.zeros(max_seqs, dtype=torch.int32, device=self.device)
        self._host_len = [0] * max_seqs

    @classmethod
    def for_model(cls, cfg, batch: int, max_len: int, device, heads: int = None) -> "PagedKVCache":
        pages_per_seq = (max_len + PAGE - 1) // PAGE
        # the cache holds the key/value heads (fewer than query heads under grouped-query
        # attention; ``heads`` overrides with a tensor-parallel rank's share)
        return cls(cfg.num_layers, heads or cfg.kv_heads, cfg.head_dim, batch * pages_per_seq,
                   batch, pages_per_seq, device)

    def reserve(self, seq: int, total_len: int) -> None:
        """Make sure sequence ``seq`` owns enough pages for ``total_len`` tokens."""
        need = (total_len + PAGE - 1) // PAGE
        have = self.owned.setdefault(seq, [])
        if need > self.page_table.shape[1]:
            raise ResourceError.exhausted("KV pages per sequence", self.page_table.shape[1], need)
        new = []
        while len(have) + len(new) < need:
            if not self.free:
                self.free.extend(reversed(new))       # nothing is taken when not all can be
                raise ResourceError.exhausted("KV cache pages", len(new), need - len(have))
            new.append(self.free.pop())
        for p in new:
            self.refs[p] = 1
        if new:
            idx = torch.tensor(new, dtype=torch.int32, device=self.device)
            self.page_table[seq, len(have):len(have) + len(new)] = idx
            have.extend(new)

    def release(self, seq: int) -> None:
        for p in reversed(self.owned.pop(seq, [])):
            self.drop(p)
        self._host_len[seq] = 0
        self.lengths[seq] = 0

    def retain(self, page: int) -> None:
        """One more holder of ``page`` (e.g. a prefix cache entry)."""
        self.refs[page] += 1

    def drop(self, page: int) -> None:
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    def adopt(self, seq: int, pages: List[int]) -> None:
        """Start sequence ``seq`` (which owns nothing yet) on existing, already filled pages."""
        if self.owned.get(seq):
            raise ResourceError.exhausted("KV slot", 0, 1)
        for p in pages:
            self.refs[p] += 1
        self.owned[seq] = list(pages)
        if pages:
            idx = torch.tensor(pages, dtype=torch.int32, device=self.device)
            self.page_table[seq, :len(pages)] = idx

    def set_length(self, seq: int, n: int) -> None:
        self._host_len[seq] = n

    def length(self, seq: int) -> int:
        return self._host_len[seq]

    def pages_in_use(self) -> int:
        return self.num_pages - len(self.free)
