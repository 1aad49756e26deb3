"""Plugin contracts (counterpart of src/core/plugin.rs): ``Plugin`` with capabilities and
``on_unload``, the ``PluginState`` machine with the reference's transition table
(plugin.rs:181-205), ``PluginEntry`` / ``PluginBuilder``, and the three specialised plugin kinds
``TokenizerPlugin.create_tokenizer``, ``ModelBuilderPlugin.create_builder`` and
``ModelLoaderPlugin.{supported_formats, load_model}`` (plugin.rs:334-361)."""
from __future__ import annotations

import abc
import enum
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence

from ..foundation.error import PluginError
from ..foundation.types import PluginName, Version
from .traits import HealthCheck, Identity, Lifecycle, Metrics, Versioned


@dataclass
class PluginCapabilities:
    """plugin.rs:55-100."""

    lifecycle: bool = False
    health: bool = False
    metrics: bool = False
    configurable: bool = False
    features: List[str] = field(default_factory=list)

    @classmethod
    def none(cls) -> "PluginCapabilities":
        return cls()

    @classmethod
    def standard(cls) -> "PluginCapabilities":
        return cls(lifecycle=True, health=True, metrics=False, configurable=True)

    def with_feature(self, feature: str) -> "PluginCapabilities":
        self.features.append(feature)
        return self

    def has_feature(self, feature: str) -> bool:
        return feature in self.features


class Plugin(Identity, Versioned):
    """Base of all plugins.  Subclasses define ``id()`` and ``version()``."""

    def capabilities(self) -> PluginCapabilities:
        return PluginCapabilities.none()

    def on_unload(self) -> None:
        return None

    def __repr__(self) -> str:
        return f"{type(self).__name__}(id={self.id()!r}, version={self.version()})"


class PluginLifecycle(Plugin, Lifecycle):
    pass


class PluginHealth(Plugin, HealthCheck):
    pass


class PluginMetrics(Plugin, Metrics):
    pass


class PluginConfig(abc.ABC):
    @abc.abstractmethod
    def get(self, key: str) -> Optional[Any]: ...

    def clone_box(self) -> "PluginConfig":
        import copy
        return copy.deepcopy(self)

    def validate(self) -> None:
        return None


class PluginFactory(abc.ABC):
    @abc.abstractmethod
    def create(self, config: Optional[PluginConfig] = None) -> Plugin: ...

    @abc.abstractmethod
    def plugin_type(self) -> str: ...


class PluginState(enum.Enum):
    Registered = "Registered"
    Ready = "Ready"
    Running = "Running"
    Stopped = "Stopped"
    Error = "Error"

    def is_usable(self) -> bool:
        return self in (PluginState.Ready, PluginState.Running)

    def can_start(self) -> bool:
        return self in (PluginState.Ready, PluginState.Stopped)

    def can_stop(self) -> bool:
        return self is PluginState.Running

    def can_transition_to(self, nxt: "PluginState") -> bool:
        S = PluginState
        if (self, nxt) in ((S.Registered, S.Ready), (S.Ready, S.Running), (S.Stopped, S.Running),
                           (S.Running, S.Stopped), (S.Error, S.Registered)):
            return True
        if nxt is S.Error:
            return True
        return self is nxt

    def __repr__(self) -> str:
        return self.value


class PluginEntry:
    """A loaded plugin with its state and dependencies (plugin.rs:217-289)."""

    def __init__(self, plugin: Plugin) -> None:
        self._plugin = plugin
        self._state = PluginState.Registered
        self._deps: List[PluginName] = []

    new = classmethod(lambda cls, plugin: cls(plugin))

    def name(self) -> str:
        return self._plugin.id()

    def version(self) -> Version:
        return self._plugin.version()

    def state(self) -> PluginState:
        return self._state

    def transition_to(self, new_state: PluginState) -> None:
        if not self._state.can_transition_to(new_state):
            raise PluginError.lifecycle(self.name(), self._state.value, "transition")
        self._state = new_state

    def plugin(self) -> Plugin:
        return self._plugin

    plugin_mut = plugin

    def add_dependency(self, dep: str) -> None:
        if dep not in self._deps:
            self._deps.append(PluginName(dep))

    def dependencies(self) -> List[PluginName]:
        return list(self._deps)


class PluginBuilder:
    def __init__(self, plugin: Plugin) -> None:
        self.plugin = plugin
        self.deps: List[PluginName] = []

    new = classmethod(lambda cls, plugin: cls(plugin))

    def depends_on(self, name: str) -> "PluginBuilder":
        self.deps.append(PluginName(name))
        return self

    def build(self) -> PluginEntry:
        entry = PluginEntry(self.plugin)
        for d in self.deps:
            entry.add_dependency(d)
        return entry


class TokenizerPlugin(Plugin):
    @abc.abstractmethod
    def create_tokenizer(self) -> Any: ...


class ModelBuilderPlugin(Plugin):
    @abc.abstractmethod
    def create_builder(self) -> Any: ...


class ModelLoaderPlugin(Plugin):
    @abc.abstractmethod
    def supported_formats(self) -> Sequence[str]: ...

    @abc.abstractmethod
    def load_model(self, path: str) -> Any: ...


def impl_plugin(name: str, version: Version, features: Sequence[str] = ()):
    """Class decorator standing for the ``impl_plugin!`` macro (plugin.rs:371-412): supplies
    ``id``, ``version`` and ``capabilities`` from constants."""

    def deco(cls):
        cls.id = lambda self: name
        cls.version = lambda self: version
        caps = list(features)

        def capabilities(self) -> PluginCapabilities:
            c = PluginCapabilities.standard()
            for f in caps:
                c.with_feature(f)
            return c
        cls.capabilities = capabilities
        cls.__abstractmethods__ = frozenset(
            m for m in getattr(cls, "__abstractmethods__", ()) if m not in ("id", "version"))
        return cls
    return deco
