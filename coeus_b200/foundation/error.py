"""Error model.

Mirrors the reference's ``enum Error {Plugin, Processing, Io, Config, Resource, Composite}``
(src/foundation/error.rs:25-44) as an exception hierarchy: one class per category, one
``kind`` per variant, fields as attributes, and ``str(err)`` equal to the reference's ``Display``
text (error.rs:386-588), which the reference's tests match by substring.  Two categories are
added for the device side: :class:`CommError` (a wait on a peer ran out of time, a peer was
lost, ranks disagree) and :class:`DeviceError` (a kernel launch failed or a kernel's index check
tripped and recorded a status word).
"""
from __future__ import annotations

import inspect
import time
from dataclasses import dataclass, field
from typing import Any, Generic, List, Optional, Sequence, TypeVar

T = TypeVar("T")


class Error(Exception):
    """Base of all framework errors.  ``category`` is the reference's enum variant name."""

    category = "Error"
    prefix = "Error"

    def __init__(self, kind: str, message: str, **fields: Any) -> None:
        super().__init__(message)
        self.kind = kind
        self.message = message
        self.fields = fields
        for k, v in fields.items():
            setattr(self, k, v)

    def __str__(self) -> str:
        return f"{self.prefix}: {self.message}"

    def __repr__(self) -> str:
        args = ", ".join(f"{k}={v!r}" for k, v in self.fields.items())
        return f"{self.category}({self.kind}{{{args}}})"

    # ErrorExt::context / with_context (error.rs:352-380)
    def context(self, ctx: "ErrorContext") -> "ContextualError":
        return ContextualError(self, ctx)

    def with_context(self, f) -> "ContextualError":
        """``f`` is an operation name, an ``ErrorContext`` or a callable returning one."""
        if isinstance(f, str):      # error.rs:368-370: operation "operation", the text as details
            return ContextualError(self, ErrorContext("operation").with_details(f))
        if isinstance(f, ErrorContext):
            return ContextualError(self, f)
        return ContextualError(self, f())


class PluginError(Error):
    category = "Plugin"
    prefix = "Plugin error"

    @classmethod
    def not_found(cls, name: str, available: Sequence[str] = ()) -> "PluginError":
        msg = f"Plugin '{name}' not found"
        if available:
            msg += ". Available: " + ", ".join(available)
        return cls("NotFound", msg, name=name, available=list(available))

    @classmethod
    def lifecycle(cls, name: str, current_state: str, operation: str) -> "PluginError":
        return cls("Lifecycle", f"Plugin '{name}' cannot {operation} in state \"{current_state}\"",
                   name=name, current_state=current_state, operation=operation)

    @classmethod
    def dependency(cls, plugin: str, dependency: str,
                   version_constraint: Optional[str] = None) -> "PluginError":
        msg = f"Plugin '{plugin}' missing dependency '{dependency}'"
        if version_constraint is not None:
            msg += f" (version {version_constraint})"
        return cls("Dependency", msg, plugin=plugin, dependency=dependency,
                   version_constraint=version_constraint)


class ProcessingError(Error):
    category = "Processing"
    prefix = "Processing error"

    @classmethod
    def not_initialized(cls, component: str) -> "ProcessingError":
        return cls("NotInitialized", f"{component} not initialized", component=component)

    @classmethod
    def invalid_input(cls, description: str, position: Optional[int] = None) -> "ProcessingError":
        msg = f"Invalid input: {description}"
        if position is not None:
            msg += f" at position {position}"
        return cls("InvalidInput", msg, description=description, position=position)

    @classmethod
    def limit_exceeded(cls, limit_type: str, limit: int, actual: int) -> "ProcessingError":
        return cls("LimitExceeded", f"{limit_type} limit exceeded: {actual} > {limit}",
                   limit_type=limit_type, limit=limit, actual=actual)

    @classmethod
    def shape_mismatch(cls, expected: str, actual: str) -> "ProcessingError":
        return cls("ShapeMismatch", f"Shape mismatch: expected {expected}, got {actual}",
                   expected=expected, actual=actual)

    @classmethod
    def unsupported(cls, operation: str, reason: Optional[str] = None) -> "ProcessingError":
        msg = f"Unsupported operation: {operation}"
        if reason is not None:
            msg += f" ({reason})"
        return cls("Unsupported", msg, operation=operation, reason=reason)

    @classmethod
    def failed(cls, component: str, reason: str) -> "ProcessingError":
        return cls("Failed", f"{component} failed: {reason}", component=component, reason=reason)


class IoOperation:
    Read, Write, Create, Delete, Open, Close = "Read", "Write", "Create", "Delete", "Open", "Close"


class IoError(Error):
    category = "Io"
    prefix = "I/O error"

    @classmethod
    def file_system(cls, path: str, operation: str, source: Optional[str] = None) -> "IoError":
        msg = f"File system error on '{path}' during {operation}"
        if source is not None:
            msg += f": {source}"
        return cls("FileSystem", msg, path=path, operation=operation, source=source)

    @classmethod
    def network(cls, description: str, endpoint: Optional[str] = None) -> "IoError":
        msg = "Network error"
        if endpoint is not None:
            msg += f" on '{endpoint}'"
        msg += f": {description}"
        return cls("Network", msg, endpoint=endpoint, description=description)


class ConfigError(Error):
    category = "Config"
    prefix = "Configuration error"

    @classmethod
    def missing(cls, key: str, expected: str) -> "ConfigError":
        return cls("Missing", f"Missing configuration '{key}' (expected {expected})", key=key,
                   expected=expected)

    @classmethod
    def invalid(cls, key: str, value: Any, error: str) -> "ConfigError":
        return cls("Invalid", f"Invalid configuration '{key}' = '{value}': {error}", key=key,
                   value=str(value), error=error)

    @classmethod
    def conflict(cls, key1: str, key2: str, description: str) -> "ConfigError":
        return cls("Conflict",
                   f"Configuration conflict between '{key1}' and '{key2}': {description}",
                   key1=key1, key2=key2, description=description)


class ResourceError(Error):
    category = "Resource"
    prefix = "Resource error"

    @classmethod
    def not_available(cls, resource_type: str, identifier: str) -> "ResourceError":
        return cls("NotAvailable", f"{resource_type} '{identifier}' not available",
                   resource_type=resource_type, identifier=identifier)

    @classmethod
    def exhausted(cls, resource_type: str, available: int, required: int) -> "ResourceError":
        return cls("Exhausted",
                   f"{resource_type} exhausted: {available} available, {required} required",
                   resource_type=resource_type, available=available, required=required)

    @classmethod
    def busy(cls, resource_type: str, identifier: str,
             holder: Optional[str] = None) -> "ResourceError":
        msg = f"{resource_type} '{identifier}' is busy"
        if holder is not None:
            msg += f" (held by {holder})"
        return cls("Busy", msg, resource_type=resource_type, identifier=identifier, holder=holder)


class CompositeError(Error):
    """Several failures of one logical operation (error.rs:319-349)."""

    category = "Composite"
    prefix = "Composite error"

    def __init__(self, primary: Error) -> None:
        super().__init__("Composite", str(primary))
        self.primary = primary
        self.related: List[Error] = []
        self.transaction_id: Optional[str] = None

    def with_related(self, err: Error) -> "CompositeError":
        self.related.append(err)
        return self

    def with_transaction_id(self, tx: str) -> "CompositeError":
        self.transaction_id = tx
        return self

    def __str__(self) -> str:
        s = f"Composite error: {self.primary}"
        if self.related:
            s += f" ({len(self.related)} related errors)"
        return s


class CommError(Error):
    """Communication failures between ranks (no counterpart in the reference, which is a
    single process)."""

    category = "Comm"
    prefix = "Communication error"

    @classmethod
    def timeout(cls, peer: int, what: str = "signal wait") -> "CommError":
        return cls("Timeout", f"{what} on peer {peer} ran out of time", peer=peer, what=what)

    @classmethod
    def peer_lost(cls, peer: int, reason: str = "missed heartbeats") -> "CommError":
        return cls("PeerLost", f"peer {peer} lost: {reason}", peer=peer, reason=reason)

    @classmethod
    def mismatch(cls, description: str) -> "CommError":
        return cls("Mismatch", f"ranks disagree: {description}", description=description)


class DeviceError(Error):
    """A kernel reported a problem through its status word, or a launch failed."""

    category = "Device"
    prefix = "Device error"
    _names = {1: "WaitTimeout", 2: "BoundsCheck", 3: "BadArgument", 4: "CommTimeout"}

    @classmethod
    def from_status(cls, code: int, where: int) -> "DeviceError":
        kind = cls._names.get(code, "Unknown")
        return cls(kind, f"kernel status {kind} (code {code}) at {where}", code=code, where=where)

    @classmethod
    def launch_failed(cls, name: str, rc: int) -> "DeviceError":
        return cls("LaunchFailed", f"launch of {name} failed with code {rc}", name=name, rc=rc)


# -------------------------------------------------------------------------------- context
@dataclass
class Location:
    file: str
    line: int
    column: int = 0


@dataclass
class ErrorContext:
    """What was being done when an error occurred (error.rs:49-109)."""

    operation: str
    location: Optional[Location] = None
    details: Optional[str] = None
    timestamp: Optional[float] = None

    def at(self, file: str, line: int, column: int = 0) -> "ErrorContext":
        self.location = Location(file, line, column)
        return self

    def with_details(self, details: str) -> "ErrorContext":
        self.details = str(details)
        return self

    def with_timestamp(self) -> "ErrorContext":
        self.timestamp = time.time()
        return self


def error_context(operation: str, details: Optional[str] = None) -> ErrorContext:
    """Counterpart of the ``error_context!`` macro: records the caller's file and line."""
    fr = inspect.stack()[1]
    ctx = ErrorContext(operation).at(fr.filename, fr.lineno, 0)
    if details is not None:
        ctx.with_details(details)
    return ctx


class ContextualError(Error, Generic[T]):
    category = "Contextual"

    def __init__(self, error: Any, context: ErrorContext) -> None:
        Exception.__init__(self, str(error))
        self.error = error
        self.ctx = context
        self.kind = getattr(error, "kind", "Contextual")
        self.message = str(error)
        self.fields = {}

    def __str__(self) -> str:
        s = f"[{self.ctx.operation}] {self.error}"
        if self.ctx.details is not None:
            s += f": {self.ctx.details}"
        if self.ctx.location is not None:
            loc = self.ctx.location
            s += f" at {loc.file}:{loc.line}:{loc.column}"
        if self.ctx.timestamp is not None:
            s += f" ({int(self.ctx.timestamp)})"
        return s


def with_context(value: Any, ctx: ErrorContext) -> ContextualError:
    """``ErrorExt::context`` for arbitrary values."""
    return ContextualError(value, ctx)


class ErrorExt:
    """``ErrorExt`` (error.rs:352-371), which the reference implements for every type: wrap any
    value with a context.  :class:`Error` carries the same two methods itself."""

    @staticmethod
    def context(value: Any, ctx: ErrorContext) -> ContextualError:
        return ContextualError(value, ctx)

    @staticmethod
    def with_context(value: Any, context: str) -> ContextualError:
        return ContextualError(value, ErrorContext("operation").with_details(context))


# -------------------------------------------------------------------------------- helpers
def not_initialized(component: str) -> Error:
    return ProcessingError.not_initialized(component)


def invalid_input(description: str) -> Error:
    return ProcessingError.invalid_input(description)


def limit_exceeded(limit_type: str, limit: int, actual: int) -> Error:
    return ProcessingError.limit_exceeded(limit_type, limit, actual)


def internal_error(reason: str) -> Error:
    return ProcessingError.failed("internal", reason)


Result = Any  # Python raises instead of returning Result<T>
