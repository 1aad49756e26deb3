"""Training context (src/domain/training/mod.rs:6-34): ``TrainingConfig{learning_rate,
batch_size, epochs}``, the ``Optimizer`` choice, sessions and the ``Started`` / ``EpochCompleted``
events, which :class:`TrainingService` really emits while driving a trainer over a data source."""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Callable, Iterable, List


@dataclass
class TrainingConfig:
    learning_rate: float = 3e-4
    batch_size: int = 8
    epochs: int = 1


@dataclass(frozen=True)
class Optimizer:
    kind: str                      # SGD | Adam
    momentum: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.999

    @classmethod
    def SGD(cls, momentum: float = 0.0) -> "Optimizer":
        return cls("SGD", momentum=momentum)

    @classmethod
    def Adam(cls, beta1: float = 0.9, beta2: float = 0.999) -> "Optimizer":
        return cls("Adam", beta1=beta1, beta2=beta2)


@dataclass
class TrainingSession:
    id: str
    model_id: str


@dataclass(frozen=True)
class TrainingEvent:
    kind: str                      # Started | EpochCompleted
    session_id: str
    epoch: int = 0
    loss: float = 0.0


class TrainingService:
    _ids = itertools.count()

    def __init__(self, trainer, model_id: str = "model") -> None:
        self.trainer, self.model_id = trainer, model_id
        self.listeners: List[Callable[[TrainingEvent], None]] = []

    def subscribe(self, f: Callable[[TrainingEvent], None]) -> None:
        self.listeners.append(f)

    def _emit(self, e: TrainingEvent) -> None:
        for f in self.listeners:
            f(e)

    def fit(self, epochs: int, batches: Callable[[int], Iterable]) -> List[float]:
        """``batches(epoch)`` yields ``(ids, targets)``; returns the mean loss per epoch."""
        session = TrainingSession(f"train-{next(self._ids)}", self.model_id)
        self._emit(TrainingEvent("Started", session.id))
        history = []
        for epoch in range(epochs):
            total, n = 0.0, 0
            for ids, targets in batches(epoch):
                total += float(self.trainer.train_step(ids, targets))
                n += 1
            mean = total / max(1, n)
            history.append(mean)
            self._emit(TrainingEvent("EpochCompleted", session.id, epoch, mean))
        return history
