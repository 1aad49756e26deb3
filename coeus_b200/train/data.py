"""Token-stream data loading: fixed-length windows over one long token array (the reference's
``windows`` / ``chunks`` / ``batch`` / ``prefetch`` iterator adapters, src/foundation/iterator.rs,
as a training input pipeline).  The windows are cut, shuffled and batched by the native
``TokenBatchLoader`` (its own prefetch thread, GIL released) straight into pinned host buffers;
the host-to-device copies of batch ``i + 1`` run on a side stream while batch ``i`` trains."""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import numpy as np
import torch

from ..utils import native


class TokenDataset:
    """``tokens``: 1-D integer array.  Yields ``(ids [B, S], targets [B, S])`` where the targets
    are the ids shifted by one; windows advance by ``stride`` (default ``S``)."""

    def __init__(self, tokens, seq_len: int, batch: int, stride: Optional[int] = None,
                 shuffle: bool = False, seed: int = 0, drop_last: bool = True,
                 rank: int = 0, world: int = 1, prefetch: int = 2) -> None:
        tokens = np.ascontiguousarray(np.asarray(tokens).astype(np.int32))
        self.seq_len, self.batch, self.rank, self.world = seq_len, batch, rank, world
        # every rank walks the same shuffled window order and keeps every world-th batch
        self._loader = native.module().TokenBatchLoader(tokens, seq_len + 1, stride or seq_len,
                                                        batch, prefetch, shuffle, seed, drop_last)
        self._buf = np.empty((batch, seq_len + 1), dtype=np.int64)

    # ---- sources
    @classmethod
    def from_binary(cls, path: str, seq_len: int, batch: int, dtype=np.uint16, **kw
                    ) -> "TokenDataset":
        """A flat file of token ids (``uint16`` / ``uint32`` / ``int32``), memory-mapped while it
        is converted; the usual layout of pre-tokenised corpora."""
        return cls(np.memmap(path, dtype=dtype, mode="r"), seq_len, batch, **kw)

    @classmethod
    def from_text_files(cls, paths, tokenizer, seq_len: int, batch: int,
                        eos_id: Optional[int] = None, **kw) -> "TokenDataset":
        """Tokenise text files line by line (``tokenizer.encode_batch`` when the tokenizer has
        it -- the native tokenizers encode a batch of lines on a thread pool -- else
        ``encode``) into one stream, ``eos_id`` after every line when given."""
        return cls(tokenize_files(paths, tokenizer, eos_id), seq_len, batch, **kw)

    def num_windows(self) -> int:
        return self._loader.num_windows()

    def cursor(self) -> int:
        """Batches handed out so far in this epoch (stored in checkpoints as the data cursor)."""
        return self._loader.cursor()

    def seek(self, batches_done: int) -> None:
        """Continue the current epoch after ``batches_done`` batches (resume)."""
        self._loader.seek(batches_done)

    def reset(self, epoch: int = 0) -> None:
        """Start epoch ``epoch`` (a shuffling loader draws a new order per epoch)."""
        self._loader.reset(epoch)

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        i = 0
        while True:
            n = self._loader.next_into(self._buf)
            if n == 0:
                return
            mine = i % self.world == self.rank
            i += 1
            if not mine:
                continue
            t = torch.from_numpy(self._buf[:n].copy())
            yield t[:, :-1].contiguous(), t[:, 1:].contiguous()


def tokenize_files(paths, tokenizer, eos_id: Optional[int] = None, lines_per_call: int = 4096
                   ) -> np.ndarray:
    """All lines of ``paths`` as one ``int32`` token stream."""
    if isinstance(paths, (str, bytes)):
        paths = [paths]
    chunks = []

    def flush(lines):
        if not lines:
            return
        if hasattr(tokenizer, "encode_batch"):
            rows = tokenizer.encode_batch(lines)
        else:
            rows = [tokenizer.encode(t) for t in lines]
        for r in rows:
            chunks.append(np.asarray(r, dtype=np.int32).reshape(-1))
            if eos_id is not None:
                chunks.append(np.array([eos_id], dtype=np.int32))

    for path in paths:
        pending = []
        with open(path, "r", encoding="utf-8", errors="replace") as f:
            for line in f:
                line = line.rstrip("\n")
                if not line:
                    continue
                pending.append(line)
                if len(pending) >= lines_per_call:
                    flush(pending)
                    pending = []
        flush(pending)
    return np.concatenate(chunks) if chunks else np.zeros(0, dtype=np.int32)


def save_tokens(path: str, tokens, dtype=np.uint16) -> None:
    """Write a token stream as the flat binary file :meth:`TokenDataset.from_binary` reads."""
    arr = np.asarray(tokens)
    if arr.size and int(arr.max()) > np.iinfo(dtype).max:
        raise ValueError(f"token id {int(arr.max())} does not fit {np.dtype(dtype).name}")
    arr.astype(dtype).tofile(path)


class DevicePrefetcher:
    """Wraps an iterable of host ``(ids, targets)`` pairs: copies each into pinned memory and
    on to the device on a side stream one batch ahead of the consumer."""

    def __init__(self, it, device) -> None:
        self.it, self.device = it, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.h2d_bytes = 0

    def _stage(self, pair):
        if pair is None:
            return None
        if not self.cuda:
            return pair
        with torch.cuda.stream(self.stream):
            out = []
            for t in pair:
                p = t.pin_memory()
                self.h2d_bytes += p.numel() * p.element_size()
                out.append(p.to(self.device, non_blocking=True))
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return (*out, ev)

    def __iter__(self):
        src = iter(self.it)
        nxt = self._stage(next(src, None))
        while nxt is not None:
            cur = nxt
            nxt = self._stage(next(src, None))
            if self.cuda:
                x, y, ev = cur
                torch.cuda.current_stream(self.device).wait_event(ev)
                x.record_stream(torch.cuda.current_stream(self.device))
                y.record_stream(torch.cuda.current_stream(self.device))
                yield x, y
            else:
                yield cur
