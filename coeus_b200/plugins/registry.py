"""Plugin registry (counterpart of src/plugins/registry.rs): ``name -> factory``, ``type ->
name`` and ``name -> dependencies`` maps with ``register`` (the plugin's default-constructed
``id()`` is its name), ``register_with_deps``, ``register_with_factory``,
``register_factory_with_deps``, ``create``, ``list``, ``contains``, ``name_for_type``,
``dependencies``, ``unregister``, ``clear`` and a builder.  A duplicate registration raises
``PluginError::Lifecycle{current_state: "Ready", operation: "register"}`` (registry.rs:50-56).
On top of the reference: ``discover_entry_points`` registers plugins that installed packages
advertise under the ``coeus_b200.plugins`` entry-point group."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Type

from ..core.plugin import Plugin
from ..foundation.error import PluginError
from ..foundation.types import PluginName

Factory = Callable[[], Plugin]


class PluginRegistry:
    def __init__(self) -> None:
        self._factories: Dict[str, Factory] = {}
        self._types: Dict[type, str] = {}
        self._deps: Dict[str, List[PluginName]] = {}

    new = classmethod(lambda cls: cls())

    def _check_new(self, name: str) -> None:
        if name in self._factories:
            raise PluginError.lifecycle(name, "Ready", "register")

    def register(self, plugin_type: Type[Plugin]) -> None:
        name = plugin_type().id()
        self._check_new(name)
        self._factories[name] = plugin_type
        self._types[plugin_type] = name

    def register_with_deps(self, plugin_type: Type[Plugin], deps: Sequence[str]) -> None:
        self.register(plugin_type)
        self._deps[plugin_type().id()] = [PluginName(d) for d in deps]

    def register_with_factory(self, name: str, factory: Factory) -> None:
        self._check_new(name)
        self._factories[name] = factory

    def register_factory_with_deps(self, name: str, factory: Factory, deps: Sequence[str]) -> None:
        self.register_with_factory(name, factory)
        self._deps[name] = [PluginName(d) for d in deps]

    def create(self, name: str) -> Plugin:
        f = self._factories.get(name)
        if f is None:
            raise PluginError.not_found(name, self.list())
        return f()

    def list(self) -> List[str]:
        return list(self._factories.keys())

    def contains(self, name: str) -> bool:
        return name in self._factories

    def name_for_type(self, plugin_type: type) -> Optional[str]:
        return self._types.get(plugin_type)

    def dependencies(self, name: str) -> List[PluginName]:
        return list(self._deps.get(name, []))

    def unregister(self, name: str) -> None:
        if name not in self._factories:
            raise PluginError.not_found(name, self.list())
        del self._factories[name]
        self._deps.pop(name, None)
        for t, n in list(self._types.items()):
            if n == name:
                del self._types[t]

    def clear(self) -> None:
        self._factories.clear()
        self._types.clear()
        self._deps.clear()

    def discover_entry_points(self, group: str = "coeus_b200.plugins") -> List[str]:
        from importlib import metadata
        found = []
        try:
            eps = metadata.entry_points(group=group)
        except TypeError:  # pragma: no cover - very old importlib
            eps = metadata.entry_points().get(group, [])
        for ep in eps:
            cls = ep.load()
            if not self.contains(cls().id()):
                self.register(cls)
                found.append(cls().id())
        return found


class PluginRegistryBuilder:
    def __init__(self) -> None:
        self._registry = PluginRegistry()

    new = classmethod(lambda cls: cls())

    def with_plugin(self, plugin_type: Type[Plugin]) -> "PluginRegistryBuilder":
        self._registry.register(plugin_type)
        return self

    def with_factory(self, name: str, factory: Factory) -> "PluginRegistryBuilder":
        self._registry.register_with_factory(name, factory)
        return self

    def build(self) -> PluginRegistry:
        return self._registry
