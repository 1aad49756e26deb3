"""Configuration system (counterpart of src/core/config.rs): the ``ConfigValue`` tagged union with
its ``as_*`` accessors (an integer reads as a float too, config.rs:45-51), ``ConfigBuilder``,
the thread-safe ``ConfigStore`` (``merge``: the other store's values win), ``Configurable`` and
``PluginConfigManager`` (keys ``plugin.<name>`` and ``plugin.<name>.<key>``).  On top of the
reference: loaders that layer JSON / YAML files, ``COEUS_*`` environment variables and
``--key=value`` command-line flags into a store, and the typed ``ParallelConfig``."""
from __future__ import annotations

import abc
import json
import os
import threading
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

from ..foundation.error import ConfigError


class ConfigValue:
    """``Bool | Integer | Float | String | List | Map``."""

    BOOL, INTEGER, FLOAT, STRING, LIST, MAP = "Bool", "Integer", "Float", "String", "List", "Map"

    __slots__ = ("kind", "value")

    def __init__(self, kind: str, value: Any) -> None:
        self.kind, self.value = kind, value

    # constructors (the reference's From impls)
    @classmethod
    def of(cls, v: Any) -> "ConfigValue":
        if isinstance(v, ConfigValue):
            return v
        if isinstance(v, bool):
            return cls(cls.BOOL, v)
        if isinstance(v, int):
            return cls(cls.INTEGER, int(v))
        if isinstance(v, float):
            return cls(cls.FLOAT, float(v))
        if isinstance(v, str):
            return cls(cls.STRING, v)
        if isinstance(v, (list, tuple)):
            return cls(cls.LIST, [cls.of(x) for x in v])
        if isinstance(v, dict):
            return cls(cls.MAP, {str(k): cls.of(x) for k, x in v.items()})
        raise ConfigError.invalid("value", v, "Unsupported configuration value type")

    Bool = classmethod(lambda cls, v: cls(cls.BOOL, bool(v)))
    Integer = classmethod(lambda cls, v: cls(cls.INTEGER, int(v)))
    Float = classmethod(lambda cls, v: cls(cls.FLOAT, float(v)))
    String = classmethod(lambda cls, v: cls(cls.STRING, str(v)))
    List = classmethod(lambda cls, v: cls(cls.LIST, [cls.of(x) for x in v]))
    Map = classmethod(lambda cls, v: cls(cls.MAP, {k: cls.of(x) for k, x in v.items()}))

    def as_bool(self) -> Optional[bool]:
        return self.value if self.kind == self.BOOL else None

    def as_integer(self) -> Optional[int]:
        return self.value if self.kind == self.INTEGER else None

    def as_float(self) -> Optional[float]:
        if self.kind == self.FLOAT:
            return self.value
        if self.kind == self.INTEGER:
            return float(self.value)
        return None

    def as_string(self) -> Optional[str]:
        return self.value if self.kind == self.STRING else None

    def as_list(self) -> Optional[List["ConfigValue"]]:
        return self.value if self.kind == self.LIST else None

    def as_map(self) -> Optional[Dict[str, "ConfigValue"]]:
        return self.value if self.kind == self.MAP else None

    def to_python(self) -> Any:
        if self.kind == self.LIST:
            return [v.to_python() for v in self.value]
        if self.kind == self.MAP:
            return {k: v.to_python() for k, v in self.value.items()}
        return self.value

    def clone(self) -> "ConfigValue":
        return ConfigValue.of(self.to_python())

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ConfigValue) and self.kind == other.kind \
            and self.to_python() == other.to_python()

    def __repr__(self) -> str:
        return f"{self.kind}({self.to_python()!r})"


class ConfigBuilder:
    def __init__(self) -> None:
        self._value = ConfigValue(ConfigValue.MAP, {})

    @classmethod
    def map(cls) -> "ConfigBuilder":
        return cls()

    def with_(self, key: str, value: Any) -> "ConfigBuilder":
        self._value.value[str(key)] = ConfigValue.of(value)
        return self

    def build(self) -> ConfigValue:
        return self._value


class ConfigStore:
    """Thread-safe ``key -> ConfigValue`` map; ``clone()`` shares the underlying storage like
    the reference's ``Arc`` (config.rs:156-246)."""

    def __init__(self, _shared: Optional[tuple] = None) -> None:
        if _shared is None:
            self._configs: Dict[str, ConfigValue] = {}
            self._lock = threading.RLock()
        else:
            self._configs, self._lock = _shared

    new = classmethod(lambda cls: cls())

    def clone(self) -> "ConfigStore":
        return ConfigStore((self._configs, self._lock))

    def set(self, key: str, value: Any) -> None:
        with self._lock:
            self._configs[str(key)] = ConfigValue.of(value)

    def get(self, key: str) -> Optional[ConfigValue]:
        with self._lock:
            v = self._configs.get(key)
            return None if v is None else v.clone()

    def get_or_default(self, key: str, default: Any) -> ConfigValue:
        v = self.get(key)
        return ConfigValue.of(default) if v is None else v

    def remove(self, key: str) -> Optional[ConfigValue]:
        with self._lock:
            return self._configs.pop(key, None)

    def clear(self) -> None:
        with self._lock:
            self._configs.clear()

    def keys(self) -> List[str]:
        with self._lock:
            return list(self._configs.keys())

    def merge(self, other: "ConfigStore") -> None:
        with other._lock:
            items = list(other._configs.items())
        with self._lock:
            for k, v in items:
                self._configs[k] = v.clone()

    # ---- layered loading (not in the reference)
    def load_mapping(self, mapping: Dict[str, Any], prefix: str = "") -> None:
        """Flatten nested dicts into dotted keys."""
        for k, v in mapping.items():
            key = f"{prefix}{k}"
            if isinstance(v, dict):
                self.load_mapping(v, key + ".")
            else:
                self.set(key, v)

    def load_file(self, path: str) -> None:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
        if path.endswith((".yaml", ".yml")):
            import yaml
            data = yaml.safe_load(text) or {}
        else:
            data = json.loads(text)
        if not isinstance(data, dict):
            raise ConfigError.invalid(path, type(data).__name__, "Top level must be a mapping")
        self.load_mapping(data)

    def load_env(self, prefix: str = "COEUS_", environ: Optional[Dict[str, str]] = None) -> None:
        """``COEUS_TRAIN__LR=3e-4`` sets ``train.lr`` (double underscore = dot)."""
        env = os.environ if environ is None else environ
        for k, v in env.items():
            if k.startswith(prefix):
                self.set(k[len(prefix):].lower().replace("__", "."), _parse_scalar(v))

    def load_args(self, argv: Sequence[str]) -> List[str]:
        """Consume ``--key=value`` / ``--flag`` items; returns the arguments left over."""
        rest = []
        for a in argv:
            if a.startswith("--") and "=" in a:
                k, v = a[2:].split("=", 1)
                self.set(k.replace("-", "_"), _parse_scalar(v))
            elif a.startswith("--"):
                self.set(a[2:].replace("-", "_"), True)
            else:
                rest.append(a)
        return rest


def _parse_scalar(s: str) -> Any:
    low = s.lower()
    if low in ("true", "false"):
        return low == "true"
    for conv in (int, float):
        try:
            return conv(s)
        except ValueError:
            pass
    return s


class Configurable(abc.ABC):
    @abc.abstractmethod
    def configure(self, config: ConfigValue) -> None: ...

    @abc.abstractmethod
    def get_config(self) -> ConfigValue: ...


class PluginConfigManager:
    def __init__(self) -> None:
        self.store = ConfigStore()

    new = classmethod(lambda cls: cls())

    def set_plugin_config(self, plugin: str, config: Any) -> None:
        self.store.set(f"plugin.{plugin}", config)

    def get_plugin_config(self, plugin: str) -> Optional[ConfigValue]:
        return self.store.get(f"plugin.{plugin}")

    def set_plugin_key(self, plugin: str, key: str, value: Any) -> None:
        self.store.set(f"plugin.{plugin}.{key}", value)

    def get_plugin_key(self, plugin: str, key: str) -> Optional[ConfigValue]:
        return self.store.get(f"plugin.{plugin}.{key}")


@dataclass
class ParallelConfig:
    """Degrees of each parallelism strategy; their product is the world size."""

    dp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    cp: int = 1
    pp_chunks: int = 1         # > 1: interleaved 1F1B with this many model chunks per rank
    pp_transport: str = "auto"  # "nccl" (point-to-point) | "peer" (pushes into NVLink peer memory,
                               # GPUs only) | "auto": nccl for 1F1B, peer for interleaved on GPUs
    sp: bool = True            # sequence-parallel activations inside a tensor-parallel group
    ulysses: bool = False      # context parallelism by head all-to-all instead of a K/V ring
    zero_stage: int = 2        # 0: replicated optimizer state (all-reduce comparator);
                               # 1 / 2: optimizer state sharded, gradients reduce-scattered
    dp_backend: str = "p2p"    # "p2p" (fused kernel over NVLink peer memory) | "collective"

    def world_size(self) -> int:
        return self.dp * self.tp * self.pp * self.cp

    def validate(self, world: Optional[int] = None) -> None:
        if self.zero_stage not in (0, 1, 2):
            raise ConfigError.invalid("zero_stage", self.zero_stage,
                                      "Stages 0 (replicated) and 1/2 (sharded state) are built; "
                                      "parameter sharding (3) is not")
        if self.tp > 1 and not self.sp:
            raise ConfigError.invalid("sp", self.sp, "Tensor parallelism here always keeps the "
                                      "activations between blocks sequence-sharded")
        if self.pp_chunks < 1:
            raise ConfigError.invalid("pp_chunks", self.pp_chunks, "Must be >= 1")
        if self.pp_transport not in ("auto", "nccl", "peer"):
            raise ConfigError.invalid("pp_transport", self.pp_transport,
                                      "Must be one of auto, nccl, peer")
        for k in ("dp", "tp", "pp", "ep", "cp"):
            if getattr(self, k) < 1:
                raise ConfigError.invalid(k, getattr(self, k), "Parallel degree must be >= 1")
        if self.dp % self.ep != 0 and self.ep % self.dp != 0:
            raise ConfigError.conflict("dp", "ep", "expert parallelism must divide or be divided "
                                       "by the data-parallel degree")
        if world is not None and self.world_size() != world:
            raise ConfigError.conflict("world_size", "dp*tp*pp*cp",
                                       f"{world} ranks but the degrees multiply to "
                                       f"{self.world_size()}")
