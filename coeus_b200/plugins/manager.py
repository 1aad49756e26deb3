"""Plugin manager (counterpart of src/plugins/manager.rs): ``register`` / ``load`` /
``load_with_deps`` / ``start`` / ``stop`` / ``unload`` / ``with_plugin`` / ``info`` /
``list_registered`` / ``list_loaded`` / ``clear`` / ``subscribe`` with the five ``PluginEvent``
kinds.  ``load`` checks and inserts under ONE lock: the reference takes the lock twice
(manager.rs:97-132), which lets two racing loaders both succeed."""
from __future__ import annotations

import sys
import threading
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Sequence, Type

from ..core.plugin import Plugin, PluginCapabilities, PluginEntry, PluginState
from ..foundation.error import PluginError
from ..foundation.types import PluginName, Version
from .registry import PluginRegistry


@dataclass(frozen=True)
class PluginEvent:
    kind: str   # Registered | Loaded | Started | Stopped | Unloaded
    name: PluginName

    @classmethod
    def Registered(cls, name: str) -> "PluginEvent":
        return cls("Registered", PluginName(name))

    @classmethod
    def Loaded(cls, name: str) -> "PluginEvent":
        return cls("Loaded", PluginName(name))

    @classmethod
    def Started(cls, name: str) -> "PluginEvent":
        return cls("Started", PluginName(name))

    @classmethod
    def Stopped(cls, name: str) -> "PluginEvent":
        return cls("Stopped", PluginName(name))

    @classmethod
    def Unloaded(cls, name: str) -> "PluginEvent":
        return cls("Unloaded", PluginName(name))


@dataclass
class PluginInfo:
    name: str
    version: Version
    state: PluginState
    capabilities: PluginCapabilities
    dependencies: List[PluginName]


class PluginManager:
    def __init__(self) -> None:
        self._registry = PluginRegistry()
        self._plugins: Dict[str, PluginEntry] = {}
        self._subscribers: List[Callable[[PluginEvent], None]] = []
        self._lock = threading.RLock()

    new = classmethod(lambda cls: cls())

    def _emit(self, event: PluginEvent) -> None:
        with self._lock:
            subs = list(self._subscribers)
        for h in subs:
            h(event)

    def subscribe(self, handler: Callable[[PluginEvent], None]) -> None:
        with self._lock:
            self._subscribers.append(handler)

    def register(self, plugin_type: Type[Plugin], deps: Sequence[str] = ()) -> None:
        with self._lock:
            if deps:
                self._registry.register_with_deps(plugin_type, deps)
            else:
                self._registry.register(plugin_type)
            name = self._registry.name_for_type(plugin_type)
        self._emit(PluginEvent.Registered(name))

    def register_factory(self, name: str, factory: Callable[[], Plugin],
                         deps: Sequence[str] = ()) -> None:
        with self._lock:
            self._registry.register_factory_with_deps(name, factory, deps)
        self._emit(PluginEvent.Registered(name))

    def load(self, name: str) -> None:
        with self._lock:
            if name in self._plugins:
                raise PluginError.lifecycle(name, "loaded", "load")
            plugin = self._registry.create(name)
            entry = PluginEntry(plugin)
            for d in self._registry.dependencies(name):
                entry.add_dependency(d)
            entry.transition_to(PluginState.Ready)
            self._plugins[name] = entry
        self._emit(PluginEvent.Loaded(name))

    def load_with_deps(self, name: str) -> None:
        for d in self._registry.dependencies(name):
            try:
                self.load_with_deps(str(d))
            except PluginError as err:
                if err.kind == "Lifecycle" and getattr(err, "current_state", "") == "loaded":
                    continue
                print(f"Failed to load dependency '{d}': {err!r}", file=sys.stderr)
        self.load(name)

    def _entry(self, name: str) -> PluginEntry:
        entry = self._plugins.get(name)
        if entry is None:
            raise PluginError.not_found(name, self.list_loaded())
        return entry

    def unload(self, name: str) -> None:
        events = []
        with self._lock:
            entry = self._plugins.pop(name, None)
            if entry is None:
                raise PluginError.not_found(name, self.list_loaded())
            if entry.state() is PluginState.Running:
                entry.transition_to(PluginState.Stopped)
                events.append(PluginEvent.Stopped(name))
            entry.plugin().on_unload()
            events.append(PluginEvent.Unloaded(name))
        for e in events:
            self._emit(e)

    def start(self, name: str) -> None:
        with self._lock:
            entry = self._entry(name)
            if not entry.state().can_start():
                raise PluginError.lifecycle(name, entry.state().value, "start")
            entry.transition_to(PluginState.Running)
        self._emit(PluginEvent.Started(name))

    def stop(self, name: str) -> None:
        with self._lock:
            entry = self._entry(name)
            if not entry.state().can_stop():
                raise PluginError.lifecycle(name, entry.state().value, "stop")
            entry.transition_to(PluginState.Stopped)
        self._emit(PluginEvent.Stopped(name))

    def with_plugin(self, name: str, f: Callable[[Plugin], Any]) -> Any:
        with self._lock:
            entry = self._entry(name)
            return f(entry.plugin())

    def list_registered(self) -> List[str]:
        with self._lock:
            return self._registry.list()

    def list_loaded(self) -> List[str]:
        with self._lock:
            return list(self._plugins.keys())

    def info(self, name: str) -> PluginInfo:
        with self._lock:
            e = self._entry(name)
            return PluginInfo(e.name(), e.version(), e.state(), e.plugin().capabilities(),
                              e.dependencies())

    def mark_error(self, name: str) -> None:
        """Move a plugin to ``Error`` (always allowed); ``recover`` brings it back to
        ``Registered`` -> ``Ready`` (the reference's recovery transition, plugin.rs:195-197)."""
        with self._lock:
            self._entry(name).transition_to(PluginState.Error)

    def recover(self, name: str) -> None:
        with self._lock:
            e = self._entry(name)
            e.transition_to(PluginState.Registered)
            e.transition_to(PluginState.Ready)

    def discover(self) -> List[str]:
        with self._lock:
            return self._registry.discover_entry_points()

    def clear(self) -> None:
        with self._lock:
            self._plugins.clear()
            self._registry.clear()
