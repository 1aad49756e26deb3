"""Sharding plans as pure functions (no communication): which rank owns which range of the flat
parameter buffer, and which bucket becomes ready at which point of the backward pass.  Kept free
of device code so the plans can be checked over any number of simulated ranks on a CPU."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple


@dataclass
class Bucket:
    index: int
    start: int          # first global element (multiple of 8)
    end: int            # one past the last global element
    trigger: int        # backward event that completes it: -1 head, l >= 0 layer l, -2 end
    name: str

    def shard(self, rank: int, world: int) -> Tuple[int, int]:
        """Range of this bucket owned by ``rank``: equal pieces rounded up to 8 elements, the
        last ranks may get a shorter (or empty) piece."""
        n = self.end - self.start
        per = (n + world - 1) // world
        per = (per + 7) // 8 * 8
        s = min(self.end, self.start + rank * per)
        e = min(self.end, s + per)
        return s, e


def build_buckets(layout, n_flat: int) -> List[Bucket]:
    """One bucket per transformer layer (its matrices are contiguous in the flat buffer), one for
    the output projection, one for the token embedding and one for the vector tail (norm scales,
    biases, padding), in the order in which the backward pass completes them."""
    cfg = layout.cfg
    L = cfg.num_layers
    by = layout.by_name

    def layer_start(l: int) -> int:
        return by[f"layers.{l}.attn.qkv_weights"].offset

    buckets: List[Bucket] = []
    if not cfg.tie_embeddings:
        head_start = by["output_proj"].offset
        buckets.append(Bucket(0, head_start, layout.decay_end, -1, "output_proj"))
        layers_end = head_start
    else:
        layers_end = layout.decay_end
    for l in reversed(range(L)):
        s = layer_start(l)
        e = layer_start(l + 1) if l + 1 < L else layers_end
        buckets.append(Bucket(len(buckets), s, e, l, f"layer{l}"))
    buckets.append(Bucket(len(buckets), 0, layer_start(0), -2, "token_embed"))
    buckets.append(Bucket(len(buckets), layout.decay_end, n_flat, -2, "vectors"))
    return buckets


def shard_table(buckets: List[Bucket], world: int) -> Dict[int, List[Tuple[int, int, int]]]:
    """``rank -> [(bucket, start, end)]``; together the shards tile ``[0, n_flat)`` exactly."""
    return {r: [(b.index, *b.shard(r, world)) for b in buckets] for r in range(world)}


def moment_offsets(buckets: List[Bucket], rank: int, world: int) -> Tuple[List[int], int]:
    """Offsets of each bucket's shard inside this rank's flat moment arrays, and their length."""
    offs, total = [], 0
    for b in buckets:
        s, e = b.shard(rank, world)
        offs.append(total)
        total += (e - s + 63) // 64 * 64
    return offs, total
