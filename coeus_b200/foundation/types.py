"""Core types (counterpart of src/foundation/types.rs): ``Version`` with its compatibility rule,
``Shape``, the ``PluginName`` / ``ConfigKey`` newtypes, scalar aliases and the dtype enum (the
reference is fp32 only; bf16 and fp8 are added for the device paths)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from functools import total_ordering
from typing import Iterable, Sequence, Tuple

from .error import invalid_input

TokenId = int          # u32 in the reference
VocabSize = int
SequenceLength = int
BatchSize = int
ModelDim = int
HeadCount = int
LayerCount = int
ModelFloat = float     # f32
ModelDouble = float    # f64


class DType(enum.Enum):
    F32 = "f32"
    F64 = "f64"
    BF16 = "bf16"
    F16 = "f16"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"
    I32 = "i32"
    I64 = "i64"
    U8 = "u8"

    def to_torch(self):
        import torch
        return {"f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16,
                "f16": torch.float16, "fp8_e4m3": torch.float8_e4m3fn,
                "fp8_e5m2": torch.float8_e5m2, "i32": torch.int32, "i64": torch.int64,
                "u8": torch.uint8}[self.value]

    @property
    def itemsize(self) -> int:
        return {"f32": 4, "f64": 8, "bf16": 2, "f16": 2, "fp8_e4m3": 1, "fp8_e5m2": 1, "i32": 4,
                "i64": 8, "u8": 1}[self.value]


@total_ordering
@dataclass(frozen=True)
class Version:
    """``major.minor.patch`` (u16 each).  ``a.is_compatible_with(b)`` holds when the majors are
    equal and ``a.minor >= b.minor`` (types.rs:30-33)."""

    major: int
    minor: int
    patch: int

    def __post_init__(self) -> None:
        for v in (self.major, self.minor, self.patch):
            if not (0 <= v <= 0xFFFF):
                raise invalid_input("Version component out of u16 range")

    @classmethod
    def new(cls, major: int, minor: int, patch: int) -> "Version":
        return cls(major, minor, patch)

    def is_compatible_with(self, other: "Version") -> bool:
        return self.major == other.major and self.minor >= other.minor

    @classmethod
    def parse(cls, s: str) -> "Version":
        parts = s.split(".")
        if len(parts) != 3:
            raise invalid_input("Invalid version format")
        try:
            nums = [int(p) for p in parts]
        except ValueError:
            raise invalid_input("Invalid version number") from None
        for p, n in zip(parts, nums):
            if n < 0 or not p.isdigit():
                raise invalid_input("Invalid version number")
        return cls(*nums)

    from_str = parse

    def __str__(self) -> str:
        return f"{self.major}.{self.minor}.{self.patch}"

    def _key(self) -> Tuple[int, int, int]:
        return (self.major, self.minor, self.patch)

    def __lt__(self, other: "Version") -> bool:
        return self._key() < other._key()


class PluginName(str):
    """Newtype over the plugin's name (types.rs:116-147)."""

    def as_str(self) -> str:
        return str(self)


class ConfigKey(str):
    def as_str(self) -> str:
        return str(self)


@dataclass(frozen=True)
class Shape:
    """Tensor shape.  ``is_compatible_with``: same rank and every dimension equal or one of the
    two is 1 (types.rs:205-214); printed as ``[a, b]``."""

    dims_: Tuple[int, ...]

    def __init__(self, dims: Iterable[int]) -> None:
        object.__setattr__(self, "dims_", tuple(int(d) for d in dims))

    @classmethod
    def new(cls, dims: Sequence[int]) -> "Shape":
        return cls(dims)

    def ndim(self) -> int:
        return len(self.dims_)

    def dims(self) -> Tuple[int, ...]:
        return self.dims_

    def numel(self) -> int:
        n = 1
        for d in self.dims_:
            n *= d
        return n

    def is_compatible_with(self, other: "Shape") -> bool:
        if len(self.dims_) != len(other.dims_):
            return False
        return all(a == b or a == 1 or b == 1 for a, b in zip(self.dims_, other.dims_))

    def __str__(self) -> str:
        return "[" + ", ".join(str(d) for d in self.dims_) + "]"


class markers:
    """Phantom marker types of the reference (types.rs:226-244), kept as tags."""

    class Initialized:
        pass

    class Uninitialized:
        pass

    class Trained:
        pass

    class Untrained:
        pass


# ``dyn core::error::Error + Send + Sync`` (src/foundation/types.rs:112): any exception object.
DynError = Exception
