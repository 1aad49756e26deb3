"""Inference context (src/domain/inference/mod.rs:6-32): the request / result types the
generation engine consumes and produces, sessions and events."""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Callable, List, Optional


@dataclass
class InferenceRequest:
    tokens: List[int]
    max_length: int
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None


@dataclass
class InferenceResult:
    predictions: List[int]


@dataclass
class InferenceSession:
    id: str
    model_id: str


@dataclass(frozen=True)
class InferenceEvent:
    kind: str          # Started | Completed
    session_id: str


class InferenceService:
    """Runs requests on a model that offers ``generate(ids, BasicGenerationConfig)`` and emits
    ``Started`` / ``Completed`` events to its listeners."""

    _ids = itertools.count()

    def __init__(self, model, model_id: str = "model") -> None:
        self.model, self.model_id = model, model_id
        self.listeners: List[Callable[[InferenceEvent], None]] = []

    def subscribe(self, f: Callable[[InferenceEvent], None]) -> None:
        self.listeners.append(f)

    def run(self, request: InferenceRequest) -> InferenceResult:
        from ..core.model import BasicGenerationConfig
        session = InferenceSession(f"session-{next(self._ids)}", self.model_id)
        for f in self.listeners:
            f(InferenceEvent("Started", session.id))
        cfg = BasicGenerationConfig(request.max_length, request.temperature, request.top_k,
                                    request.top_p)
        out = self.model.generate(request.tokens, cfg)
        for f in self.listeners:
            f(InferenceEvent("Completed", session.id))
        return InferenceResult(list(out))
