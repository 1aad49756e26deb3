"""Failure detection, host-side fault injection and elastic regrouping.

* :class:`Heartbeat` -- every rank bumps a counter in a key-value store from a background thread;
  ``dead_peers()`` names the ranks whose counter has not moved for ``timeout_s``.  Checked on the
  host between steps, before the next launch, so no kernel ever waits for a rank that is gone
  (device-side waits are bounded as well and come back with ``CommError.timeout``).
* :class:`StepWatchdog` -- flags steps that take much longer than the running median.
* :class:`FaultInjector` -- raises :class:`InjectedFault` at named points of the host code
  (``COEUS_FAULT="after_bucket:3"``: the third time ``after_bucket`` is reached); nothing is ever
  injected on the device.
* :func:`regroup` -- survivors agree on the new membership through the store and build a new
  process group of the smaller world; training continues from the last sharded checkpoint, which
  does not depend on the world size (``Trainer.load_checkpoint``).

The reference's nearest pieces are the plugin ``Error -> Registered`` recovery transition and the
unimplemented ``HealthCheck`` trait (src/core/plugin.rs:160-161,195-197; src/core/traits.rs:197-208).
"""
from __future__ import annotations

import os
import statistics
import threading
import time
from datetime import timedelta
from typing import Dict, List, Optional, Sequence

import torch.distributed as dist

from ..foundation.error import CommError, Error


class InjectedFault(Error):
    """Raised by :class:`FaultInjector`; carries the point that fired."""

    def __init__(self, point: str, count: int) -> None:
        super().__init__("Injected", f"injected fault at '{point}' (occurrence {count})",
                         point=point, count=count)


class FaultInjector:
    """``spec``: comma-separated ``point:n`` items (default: the ``COEUS_FAULT`` variable)."""

    def __init__(self, spec: Optional[str] = None) -> None:
        spec = os.environ.get("COEUS_FAULT", "") if spec is None else spec
        self.plan: Dict[str, int] = {}
        for item in filter(None, (s.strip() for s in spec.split(","))):
            point, _, n = item.partition(":")
            self.plan[point] = int(n) if n else 1
        self.seen: Dict[str, int] = {}

    def reach(self, point: str) -> None:
        n = self.seen.get(point, 0) + 1
        self.seen[point] = n
        if self.plan.get(point) == n:
            raise InjectedFault(point, n)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2,
                 timeout_s: float = 2.0, prefix: str = "hb") -> None:
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._last: Dict[int, tuple] = {}
        self._count = 0
        self._thread = threading.Thread(target=self._run, name=f"heartbeat-{rank}", daemon=True)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def start(self) -> "Heartbeat":
        self.store.set(self._key(self.rank), "0")
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            self._count += 1
            try:
                self.store.set(self._key(self.rank), str(self._count))
            except Exception:        # the store is gone: nothing left to report to
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    def dead_peers(self, ranks: Optional[Sequence[int]] = None) -> List[int]:
        """Ranks whose counter has not advanced for ``timeout_s`` (never started counts too)."""
        now = time.monotonic()
        dead = []
        for r in (ranks if ranks is not None else range(self.world)):
            if r == self.rank:
                continue
            try:
                value = self.store.get(self._key(r)).decode() if self.store.check([self._key(r)]) \
                    else None
            except Exception:
                value = None
            prev = self._last.get(r)
            if prev is None or prev[0] != value:
                self._last[r] = (value, now)
                continue
            if now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def require_alive(self, ranks: Optional[Sequence[int]] = None) -> None:
        dead = self.dead_peers(ranks)
        if dead:
            raise CommError.peer_lost(dead[0], f"no heartbeat for {self.timeout_s:.1f} s "
                                               f"(all silent ranks: {dead})")


class StepWatchdog:
    """``observe(seconds)`` returns True when the step is an outlier (> ``factor`` x median of the
    last ``window`` steps, after ``warmup`` steps)."""

    def __init__(self, factor: float = 3.0, window: int = 50, warmup: int = 5) -> None:
        self.factor, self.window, self.warmup = factor, window, warmup
        self.history: List[float] = []
        self.outliers = 0

    def observe(self, seconds: float) -> bool:
        slow = False
        if len(self.history) >= self.warmup:
            slow = seconds > self.factor * statistics.median(self.history[-self.window:])
        self.history.append(seconds)
        self.outliers += int(slow)
        return slow


def regroup(store, old_rank: int, alive: Sequence[int], generation: int, backend: str = "gloo",
            timeout_s: float = 30.0):
    """Build the process group of the survivors.  ``alive`` (old ranks, the same list on every
    survivor) defines the new ranks by position.  The old default group must have been destroyed
    by the caller (between steps, nothing in flight).  Returns ``(new_rank, new_world)``."""
    alive = sorted(alive)
    if old_rank not in alive:
        raise CommError.mismatch(f"rank {old_rank} is not among the survivors {alive}")
    new_rank, new_world = alive.index(old_rank), len(alive)
    sub = dist.PrefixStore(f"gen{generation}", store)
    dist.init_process_group(backend, store=sub, rank=new_rank, world_size=new_world,
                            timeout=timedelta(seconds=timeout_s))
    return new_rank, new_world


def agree_on_survivors(store, rank: int, world: int, dead: Sequence[int], generation: int,
                       wait_s: float = 10.0) -> List[int]:
    """Every survivor publishes the ranks it saw die; the union (read after all survivors of the
    union have reported) is the agreed set, so that ranks with different views converge."""
    key = f"dead/gen{generation}/{rank}"
    store.set(key, ",".join(str(d) for d in sorted(dead)))
    known = set(dead)
    deadline = time.monotonic() + wait_s
    while True:
        pending = [r for r in range(world) if r not in known and r != rank]
        missing = []
        for r in pending:
            k = f"dead/gen{generation}/{r}"
            if store.check([k]):
                v = store.get(k).decode()
                known.update(int(x) for x in v.split(",") if x)
            else:
                missing.append(r)
        missing = [r for r in missing if r not in known]
        if not missing:
            break
        if time.monotonic() > deadline:
            known.update(missing)      # a rank that never reported is treated as gone
            break
        time.sleep(0.05)
    return [r for r in range(world) if r not in known]
