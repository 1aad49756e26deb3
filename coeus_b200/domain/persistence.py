"""Persistence context (src/domain/persistence/mod.rs:6-36): storage backends, serialization
formats, checkpoint records and events; :class:`PersistenceService` is the facade over
:mod:`coeus_b200.checkpoint` that emits ``Saved`` / ``Loaded``."""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass
from typing import Callable, Dict, List


@dataclass(frozen=True)
class StorageBackend:
    kind: str                       # FileSystem | Memory
    path: str = ""

    @classmethod
    def FileSystem(cls, path: str) -> "StorageBackend":
        return cls("FileSystem", path)

    @classmethod
    def Memory(cls) -> "StorageBackend":
        return cls("Memory")


class SerializationFormat(enum.Enum):
    GGUF = "gguf"
    SafeTensors = "safetensors"
    Custom = "rustllm"


@dataclass
class Checkpoint:
    id: str
    model_id: str
    epoch: int


@dataclass(frozen=True)
class PersistenceEvent:
    kind: str                       # Saved | Loaded
    checkpoint_id: str


class PersistenceService:
    def __init__(self, backend: StorageBackend) -> None:
        self.backend = backend
        self.listeners: List[Callable[[PersistenceEvent], None]] = []
        self._memory: Dict[str, bytes] = {}

    def subscribe(self, f: Callable[[PersistenceEvent], None]) -> None:
        self.listeners.append(f)

    def _path(self, ckpt: Checkpoint, fmt: SerializationFormat) -> str:
        return os.path.join(self.backend.path, f"{ckpt.id}.{fmt.value}")

    def save(self, model, ckpt: Checkpoint,
             fmt: SerializationFormat = SerializationFormat.SafeTensors) -> str:
        """``model`` is a ``TransformerModel``; returns where it was stored."""
        if self.backend.kind == "Memory":
            import io
            buf = io.BytesIO()
            model.write_to(buf)
            self._memory[ckpt.id] = buf.getvalue()
            where = f"memory:{ckpt.id}"
        else:
            os.makedirs(self.backend.path, exist_ok=True)
            where = self._path(ckpt, fmt)
            model.save(where, fmt.value)
        for f in self.listeners:
            f(PersistenceEvent("Saved", ckpt.id))
        return where

    def load(self, ckpt: Checkpoint, fmt: SerializationFormat = SerializationFormat.SafeTensors,
             device: str = "auto"):
        from ..plugins.builtin.model_transformer import TransformerModel
        if self.backend.kind == "Memory":
            import io
            model = TransformerModel.read_from(io.BytesIO(self._memory[ckpt.id]), device=device)
        else:
            model = TransformerModel.load(self._path(ckpt, fmt), device=device)
        for f in self.listeners:
            f(PersistenceEvent("Loaded", ckpt.id))
        return model
