"""Metrics, health and events.  Implements for the trainer and the inference engine what the
reference only declares: the ``Metrics`` and ``HealthCheck`` traits (src/core/traits.rs:197-221)
and the domain event enums that are never emitted (``TrainingEvent::{Started, EpochCompleted}``,
``PersistenceEvent``, ``InferenceEvent``; src/domain/*/mod.rs).  Events go to any number of sinks
(JSON lines on rank 0, stdout, user callbacks)."""
from __future__ import annotations

import json
import math
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

from ..core.traits import HealthCheck, Metrics
from ..foundation.memory import MemoryStats


@dataclass
class Metric:
    name: str
    value: float
    unit: str = ""


@dataclass
class Health:
    healthy: bool
    details: Dict[str, Any] = field(default_factory=dict)


class EventBus:
    """``emit(kind, **fields)`` fans out to the subscribed sinks (thread-safe)."""

    def __init__(self) -> None:
        self._sinks: List[Callable[[dict], None]] = []
        self._lock = threading.Lock()

    def subscribe(self, sink: Callable[[dict], None]) -> None:
        with self._lock:
            self._sinks.append(sink)

    def emit(self, kind: str, **fields: Any) -> dict:
        ev = {"event": kind, "time": time.time(), **fields}
        with self._lock:
            sinks = list(self._sinks)
        for s in sinks:
            s(ev)
        return ev


class JsonlSink:
    def __init__(self, path: str) -> None:
        self._f = open(path, "a", buffering=1)

    def __call__(self, ev: dict) -> None:
        self._f.write(json.dumps(ev, default=str) + "\n")

    def close(self) -> None:
        self._f.close()


def stdout_sink(ev: dict) -> None:
    print(json.dumps(ev, default=str), file=sys.stdout, flush=True)


def model_flops_per_token(cfg, seq_len: int, training: bool = True) -> float:
    """Matrix-multiply FLOPs per token of the decoder: ``2 * (matrix parameters touched) +
    attention`` forward, times three with the backward pass (causal attention counted as half)."""
    H, I, L, V = cfg.hidden_dim, cfg.intermediate_dim, cfg.num_layers, cfg.vocab_size
    ff = (3 if cfg.activation == "swiglu" else 2) * H * I
    if cfg.num_experts:
        ff = ff * cfg.top_k + H * cfg.num_experts
    per_layer = H * getattr(cfg, "qkv_dim", 3 * H) + H * H + ff    # fused QKV (narrower with GQA) + O
    attn = 2 * seq_len * H          # QK^T and PV, causal half of 2 * 2 * S * H
    fwd = 2.0 * (L * per_layer + H * V) + 2.0 * L * attn
    return fwd * (3.0 if training else 1.0)


def device_memory_stats(device) -> MemoryStats:
    """The allocator's counters in the reference's ``MemoryStats`` shape (memory.rs:834-887)."""
    st = MemoryStats()
    device = torch.device(device)
    if device.type == "cuda":
        s = torch.cuda.memory_stats(device)
        st.allocated_bytes = int(s.get("allocated_bytes.all.allocated", 0))
        st.deallocated_bytes = int(s.get("allocated_bytes.all.freed", 0))
        st.used_bytes = int(s.get("allocated_bytes.all.current", 0))
        st.peak_bytes = int(s.get("allocated_bytes.all.peak", 0))
        st.allocation_count = int(s.get("allocation.all.allocated", 0))
        st.deallocation_count = int(s.get("allocation.all.freed", 0))
    return st


class TrainerMonitor(Metrics, HealthCheck):
    """Wraps a trainer: counts tokens, times steps on the device, derives tokens/s and model FLOP
    utilisation, checks the kernels' status word, the loss and (optionally) peer heartbeats."""

    def __init__(self, trainer, seq_len: int, peak_tflops: Optional[float] = None,
                 bus: Optional[EventBus] = None, heartbeat=None, watchdog=None) -> None:
        self.trainer, self.seq_len = trainer, seq_len
        self.peak_tflops = peak_tflops
        self.bus = bus or EventBus()
        self.heartbeat, self.watchdog = heartbeat, watchdog
        self.device = trainer.model.device
        self._flops_tok = model_flops_per_token(trainer.model.cfg, seq_len, True)
        self.reset_metrics()

    def id(self) -> str:
        return "trainer-monitor"

    def reset_metrics(self) -> None:
        self.tokens = 0
        self.steps = 0
        self.ms = 0.0
        self.last_loss = float("nan")
        self.slow_steps = 0

    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One monitored training step (synchronises to read the time and the loss)."""
        cuda = self.device.type == "cuda"
        if self.heartbeat is not None:
            self.heartbeat.require_alive()
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        t0 = time.perf_counter()
        loss = self.trainer.train_step(ids, targets)
        if cuda:
            b.record()
            b.synchronize()
            ms = a.elapsed_time(b)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        self.ms += ms
        self.steps += 1
        self.tokens += ids.numel()
        self.last_loss = float(loss)
        if self.watchdog is not None and self.watchdog.observe(ms / 1e3):
            self.slow_steps += 1
            self.bus.emit("TrainingEvent::SlowStep", step=self.trainer.step_index, ms=ms)
        return loss

    def metrics(self) -> List[Metric]:
        tps = self.tokens / (self.ms / 1e3) if self.ms > 0 else 0.0
        out = [Metric("steps", self.steps), Metric("tokens", self.tokens),
               Metric("tokens_per_s", tps, "tok/s"),
               Metric("ms_per_step", self.ms / max(1, self.steps), "ms"),
               Metric("loss", self.last_loss), Metric("slow_steps", self.slow_steps)]
        if self.peak_tflops:
            out.append(Metric("mfu", tps * self._flops_tok / (self.peak_tflops * 1e12)))
        mem = device_memory_stats(self.device)
        out.append(Metric("memory_peak_bytes", mem.peak_bytes, "B"))
        out.append(Metric("memory_used_bytes", mem.used_bytes, "B"))
        return out

    def health(self) -> Health:
        details: Dict[str, Any] = {"loss_finite": math.isfinite(self.last_loss) or self.steps == 0}
        if self.device.type == "cuda":
            from ..ops import _lib
            try:
                _lib.check_status(self.device)
                details["device_status"] = "ok"
            except Exception as e:      # a kernel reported a bounded-wait timeout or a bad index
                details["device_status"] = repr(e)
        if self.heartbeat is not None:
            details["silent_peers"] = self.heartbeat.dead_peers()
        ok = details["loss_finite"] and details.get("device_status", "ok") == "ok" \
            and not details.get("silent_peers")
        return Health(bool(ok), details)

    def fit(self, batches, epochs: int = 1) -> None:
        """``batches``: a callable returning an iterable of ``(ids, targets)`` per epoch.  Emits
        ``TrainingEvent::Started`` and ``TrainingEvent::EpochCompleted`` like the reference's
        example loop (examples/training_example.rs:257-276)."""
        self.bus.emit("TrainingEvent::Started", epochs=epochs)
        for epoch in range(epochs):
            tot, n = 0.0, 0
            for ids, targets in batches():
                tot += float(self.step(ids, targets))
                n += 1
            self.bus.emit("TrainingEvent::EpochCompleted", epoch=epoch, mean_loss=tot / max(1, n),
                          **{m.name: m.value for m in self.metrics()})
