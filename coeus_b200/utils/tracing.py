"""Tracing and timing: NVTX ranges around phases (visible in any CUDA timeline tool) and CUDA
event timers whose per-phase totals are reduced with the maximum over ranks, which is how every
multi-GPU number of this framework is reported.  The reference times with ``Instant::now()`` in
its examples (examples/transformer_250m.rs:43-48) and reports progress through
``FnMut(done, total)`` callbacks on checkpoint IO (src/core/serialization.rs:118-127), which the
IO layer here keeps."""
from __future__ import annotations

import contextlib
import time
from typing import Dict, List, Tuple

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX push/pop on CUDA builds, nothing otherwise."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """``with timer.phase("fwd"): ...`` records a CUDA event pair on the current stream (or wall
    clock on CPU); ``summary()`` synchronises once and returns milliseconds per phase."""

    def __init__(self, device=None, enabled: bool = True) -> None:
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.enabled = enabled
        self._pairs: List[Tuple[str, object, object]] = []
        self._wall: Dict[str, float] = {}
        self._count: Dict[str, int] = {}

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        with nvtx_range(name):
            if self.cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                try:
                    yield
                finally:
                    b.record()
                    self._pairs.append((name, a, b))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._wall[name] = self._wall.get(name, 0.0) + (time.perf_counter() - t0) * 1e3
            self._count[name] = self._count.get(name, 0) + 1

    def summary(self, group=None, reset: bool = True) -> Dict[str, float]:
        """Total milliseconds per phase; with ``group`` the maximum over its ranks."""
        out = dict(self._wall)
        if self.cuda and self._pairs:
            torch.cuda.synchronize(self.device)
            for name, a, b in self._pairs:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        if group is not None and out:
            import torch.distributed as dist
            names = sorted(out)
            t = torch.tensor([out[n] for n in names], dtype=torch.float64,
                             device=self.device if self.cuda else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = dict(zip(names, t.tolist()))
        if reset:
            self._pairs.clear()
            self._wall.clear()
        return out

    def counts(self) -> Dict[str, int]:
        return dict(self._count)
