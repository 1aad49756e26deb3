"""The trait set of the reference (src/core/traits.rs) as abstract base classes with the same
names and default methods: ``Identity``, ``Versioned``, ``Metadata``, ``Lifecycle``,
``AsyncLifecycle``, ``Process`` (+ ``StreamProcess``, ``BatchProcess``, ``Pipeline.pipe`` ->
``Piped``), ``Serialize``, ``Checkpoint``, ``HealthCheck``, ``Metrics``, ``Component`` +
``ComponentInfo``, ``Factory``, ``Builder``, ``Adapter``, ``Strategy``, ``Validate``,
``Constraint``.  ``Checkpoint``, ``HealthCheck`` and ``Metrics`` are implemented by the trainer,
the inference engine and the communication layer; the reference declares them without
implementors."""
from __future__ import annotations

import abc
from dataclasses import dataclass
from typing import Any, Generic, Iterable, Iterator, List, Sequence, TypeVar

from ..foundation.types import Version

I = TypeVar("I")
O = TypeVar("O")
T = TypeVar("T")


class Identity(abc.ABC):
    @abc.abstractmethod
    def id(self) -> str: ...

    def type_name(self) -> str:
        cls = type(self)
        return f"{cls.__module__}.{cls.__qualname__}"


class Versioned(abc.ABC):
    @abc.abstractmethod
    def version(self) -> Version: ...

    def is_compatible_with(self, required: Version) -> bool:
        return self.version().is_compatible_with(required)


class Metadata(abc.ABC):
    def description(self) -> str:
        return ""

    def author(self) -> str:
        return ""

    def license(self) -> str:
        return ""

    def tags(self) -> List[str]:
        return []


class Lifecycle(abc.ABC):
    @abc.abstractmethod
    def state(self) -> Any: ...

    @abc.abstractmethod
    def initialize(self) -> None: ...

    @abc.abstractmethod
    def shutdown(self) -> None: ...

    def validate(self) -> None:
        return None


class AsyncLifecycle(Lifecycle):
    async def initialize_async(self) -> None:
        self.initialize()

    async def shutdown_async(self) -> None:
        self.shutdown()


class Process(Identity, Generic[I, O]):
    @abc.abstractmethod
    def process(self, input: I) -> O: ...

    # Pipeline (blanket impl in the reference)
    def pipe(self, nxt: "Process[O, Any]") -> "Piped":
        return Piped(self, nxt)


class StreamProcess(Process[I, O]):
    def process_stream(self, inputs: Iterable[I]) -> Iterator[O]:
        return (self.process(x) for x in inputs)


class BatchProcess(Process[I, O]):
    def process_batch(self, inputs: Sequence[I]) -> List[O]:
        return [self.process(x) for x in inputs]


Pipeline = Process


class Piped(Process[Any, Any]):
    """``first.pipe(second)``: id is the first stage's id (traits.rs:282-318)."""

    def __init__(self, first: Process, second: Process) -> None:
        self.first, self.second = first, second

    new = classmethod(lambda cls, first, second: cls(first, second))

    def id(self) -> str:
        return self.first.id()

    def process(self, input: Any) -> Any:
        return self.second.process(self.first.process(input))


class Serialize(Identity):
    @abc.abstractmethod
    def serialize(self) -> bytes: ...

    @classmethod
    @abc.abstractmethod
    def deserialize(cls, data: bytes) -> "Serialize": ...


class Checkpoint(Serialize):
    def checkpoint(self) -> bytes:
        return self.serialize()

    @abc.abstractmethod
    def restore(self, checkpoint: bytes) -> None: ...


class HealthCheck(Identity):
    @abc.abstractmethod
    def health(self) -> Any: ...

    def check_health(self) -> Any:
        return self.health()


class Metrics(Identity):
    @abc.abstractmethod
    def metrics(self) -> List[Any]: ...

    @abc.abstractmethod
    def reset_metrics(self) -> None: ...


@dataclass
class ComponentInfo:
    id: str
    type_name: str
    version: Version
    description: str
    state: str
    health: str


class Component(HealthCheck, Versioned, Metadata, Lifecycle):
    def info(self) -> ComponentInfo:
        return ComponentInfo(self.id(), self.type_name(), self.version(), self.description(),
                             repr(self.state()), repr(self.health()))


class Factory(Identity, Generic[T]):
    @abc.abstractmethod
    def create(self, config: Any) -> T: ...


class Builder(Identity, Generic[T]):
    @abc.abstractmethod
    def build(self) -> T: ...


class Adapter(Identity, Generic[T]):
    @classmethod
    @abc.abstractmethod
    def adapt_from(cls, source: T) -> "Adapter[T]": ...

    @abc.abstractmethod
    def adapt_to(self) -> T: ...


class Strategy(Identity):
    @abc.abstractmethod
    def execute(self, context: Any) -> Any: ...


class IntoIterator(Identity):
    @abc.abstractmethod
    def into_iter(self) -> Iterator[Any]: ...


class FromIterator(Identity):
    @classmethod
    @abc.abstractmethod
    def from_iter(cls, it: Iterable[Any]) -> "FromIterator": ...


class Validate(abc.ABC):
    @abc.abstractmethod
    def validate(self) -> None:
        """Raise on an invalid value."""

    def is_valid(self) -> bool:
        try:
            self.validate()
            return True
        except Exception:
            return False


class Constraint(abc.ABC, Generic[T]):
    @abc.abstractmethod
    def check(self, value: T) -> bool: ...

    @abc.abstractmethod
    def description(self) -> str: ...


class IntoIterator(Identity):
    """A component that produces an iterator (traits.rs:386-395)."""

    @abc.abstractmethod
    def into_iter(self) -> Iterator[Any]: ...

    def __iter__(self) -> Iterator[Any]:
        return self.into_iter()


class FromIterator(Identity):
    """A component that can be built from an iterator (traits.rs:399-402)."""

    @classmethod
    @abc.abstractmethod
    def from_iter(cls, iter: Iterable[Any]) -> "FromIterator": ...
