"""Modeling context (src/domain/modeling/mod.rs:10-43)."""
from __future__ import annotations

import abc
from dataclasses import dataclass
from typing import List, Optional


@dataclass(frozen=True)
class Architecture:
    kind: str                     # Transformer | RNN | CNN
    layers: int = 0
    heads: int = 0

    @classmethod
    def Transformer(cls, layers: int, heads: int) -> "Architecture":
        return cls("Transformer", layers, heads)

    @classmethod
    def RNN(cls, layers: int = 0) -> "Architecture":
        return cls("RNN", layers)

    @classmethod
    def CNN(cls, layers: int = 0) -> "Architecture":
        return cls("CNN", layers)


@dataclass
class ModelAggregate:
    id: str
    architecture: Architecture
    num_parameters: int = 0


class ModelingService:
    @staticmethod
    def describe(cfg) -> Architecture:
        return Architecture.Transformer(cfg.num_layers, cfg.num_heads)


@dataclass(frozen=True)
class ModelingEvent:
    kind: str                     # Created | Built
    model_id: str


class ModelRepository(abc.ABC):
    @abc.abstractmethod
    def save(self, model: ModelAggregate) -> None: ...

    @abc.abstractmethod
    def load(self, id: str) -> Optional[ModelAggregate]: ...

    @abc.abstractmethod
    def list(self) -> List[str]: ...
