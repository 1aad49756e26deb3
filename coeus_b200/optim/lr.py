"""Learning-rate schedules.  The reference has a fixed ``learning_rate`` field only
(src/domain/training/mod.rs:14-20, ``OptimizerState::set_learning_rate`` in
src/core/model.rs:652-667); these drive that setter once per step."""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class WarmupCosine:
    """Linear warm-up from 0 to ``peak`` over ``warmup`` steps, then cosine decay to ``floor`` at
    ``total`` steps (constant afterwards)."""

    peak: float
    warmup: int
    total: int
    floor: float = 0.0

    def at(self, step: int) -> float:
        if self.warmup > 0 and step < self.warmup:
            return self.peak * (step + 1) / self.warmup
        if step >= self.total:
            return self.floor
        t = (step - self.warmup) / max(1, self.total - self.warmup)
        return self.floor + 0.5 * (self.peak - self.floor) * (1.0 + math.cos(math.pi * t))


@dataclass
class WarmupLinear:
    peak: float
    warmup: int
    total: int
    floor: float = 0.0

    def at(self, step: int) -> float:
        if self.warmup > 0 and step < self.warmup:
            return self.peak * (step + 1) / self.warmup
        t = min(1.0, (step - self.warmup) / max(1, self.total - self.warmup))
        return self.peak + (self.floor - self.peak) * t


@dataclass
class Constant:
    peak: float

    def at(self, step: int) -> float:
        return self.peak
