"""Plugin system: registry (name -> factory) and manager (lifecycle, events)."""
from .manager import PluginEvent, PluginInfo, PluginManager  # noqa: F401
from .registry import PluginRegistry, PluginRegistryBuilder  # noqa: F401
