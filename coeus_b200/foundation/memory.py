"""Memory utilities (counterpart of src/foundation/memory.rs).

The host-side pieces keep the reference's names and observable behaviour: ``Arena`` (chunked bump
allocation with ``reset``), ``TrackingArena`` + ``MemoryStats``, ``BumpAllocator`` (fixed buffer,
``None`` when full), ``Pool`` / ``TokenBufferPool``, ``CowStr``, ``ZeroCopyStringBuilder``,
``Rope``, ``StringInterner``, ``SliceView``, ``MappedBuffer`` (a real ``mmap`` here; the reference
only wraps a pointer), ``LazyAlloc`` and the allocation benchmark structs.  The device-side
counterparts are ``DeviceArena`` (a bump allocator over one big CUDA buffer that is reset every
step, so steady-state steps never call the allocator) and ``PinnedPool`` (page-locked staging
buffers for host-to-device copies).
"""
from __future__ import annotations

import mmap
import os
import threading
import time
from dataclasses import dataclass
from typing import Any, Callable, Generic, List, Optional, Sequence, TypeVar

T = TypeVar("T")


# ------------------------------------------------------------------------------ statistics
@dataclass
class MemoryStats:
    """memory.rs:834-887."""

    allocated_bytes: int = 0
    deallocated_bytes: int = 0
    used_bytes: int = 0
    peak_bytes: int = 0
    allocation_count: int = 0
    deallocation_count: int = 0

    def record_allocation(self, nbytes: int) -> None:
        self.allocated_bytes += nbytes
        self.used_bytes += nbytes
        self.allocation_count += 1
        self.peak_bytes = max(self.peak_bytes, self.used_bytes)

    def record_deallocation(self, nbytes: int) -> None:
        self.deallocated_bytes += nbytes
        self.used_bytes = max(0, self.used_bytes - nbytes)
        self.deallocation_count += 1

    def fragmentation_ratio(self) -> float:
        if self.allocated_bytes == 0:
            return 0.0
        return 1.0 - self.used_bytes / self.allocated_bytes


# ------------------------------------------------------------------------------ arenas
class _Chunk:
    __slots__ = ("data", "used")

    def __init__(self, size: int) -> None:
        self.data = bytearray(size)
        self.used = 0


class Arena:
    """Chunked bump allocator (memory.rs:48-228).  ``alloc`` keeps Python objects alive for the
    arena's lifetime; ``alloc_bytes`` / ``alloc_slice`` hand out aligned ``memoryview`` slices of
    the chunks.  A request that does not fit opens a new chunk of
    ``max(chunk_size, size + alignment)`` bytes.  Single owner: not shared between threads."""

    def __init__(self, chunk_size: int, alignment: int = 8) -> None:
        if alignment <= 0 or alignment & (alignment - 1):
            raise ValueError("Alignment must be a power of two")
        self.chunk_size = chunk_size
        self.alignment = alignment
        self.chunks: List[_Chunk] = []
        self.current = 0
        self.objects: List[Any] = []

    @classmethod
    def new(cls, chunk_size: int) -> "Arena":
        return cls(chunk_size)

    @classmethod
    def with_alignment(cls, chunk_size: int, alignment: int) -> "Arena":
        return cls(chunk_size, alignment)

    def alloc(self, value: T) -> T:
        self.objects.append(value)
        self.alloc_bytes(max(1, _sizeof(value)))
        return value

    def alloc_bytes(self, size: int, align: Optional[int] = None) -> memoryview:
        align = align or self.alignment
        while True:
            if self.current < len(self.chunks):
                ch = self.chunks[self.current]
                start = (ch.used + align - 1) // align * align
                if start + size <= len(ch.data):
                    ch.used = start + size
                    return memoryview(ch.data)[start:start + size]
                self.current += 1
                continue
            self.chunks.append(_Chunk(max(self.chunk_size, size + align)))
            self.current = len(self.chunks) - 1

    def alloc_slice(self, data: Sequence[int]) -> memoryview:
        b = bytes(data)
        mv = self.alloc_bytes(len(b))
        mv[:] = b
        return mv

    def alloc_uninit_slice(self, length: int, itemsize: int = 1) -> memoryview:
        return self.alloc_bytes(length * itemsize)

    def reset(self) -> None:
        for ch in self.chunks:
            ch.used = 0
        self.current = 0
        self.objects.clear()

    def capacity(self) -> int:
        return sum(len(c.data) for c in self.chunks)

    def used(self) -> int:
        return sum(c.used for c in self.chunks)


def _sizeof(value: Any) -> int:
    try:
        return len(value)
    except TypeError:
        return 8


class TrackingArena:
    """Arena that records ``MemoryStats`` (memory.rs:891-943)."""

    def __init__(self, chunk_size: int, alignment: int = 8) -> None:
        self.arena = Arena(chunk_size, alignment)
        self._stats = MemoryStats()

    new = classmethod(lambda cls, chunk_size: cls(chunk_size))
    with_alignment = classmethod(lambda cls, chunk_size, alignment: cls(chunk_size, alignment))

    def alloc(self, value: T) -> T:
        self._stats.record_allocation(max(1, _sizeof(value)))
        return self.arena.alloc(value)

    def alloc_slice(self, data: Sequence[int]) -> memoryview:
        self._stats.record_allocation(len(data))
        return self.arena.alloc_slice(data)

    def reset(self) -> None:
        self._stats.record_deallocation(self._stats.used_bytes)
        self.arena.reset()

    def stats(self) -> MemoryStats:
        return MemoryStats(**self._stats.__dict__)


class BumpAllocator:
    """One fixed buffer; allocation returns ``None`` when it does not fit (memory.rs:1259-1333)."""

    def __init__(self, capacity: int) -> None:
        self.buf = bytearray(capacity)
        self._used = 0
        self._lock = threading.Lock()
        self.objects: List[Any] = []

    new = classmethod(lambda cls, capacity: cls(capacity))

    def alloc_bytes(self, size: int, align: int = 8) -> Optional[memoryview]:
        with self._lock:
            start = (self._used + align - 1) // align * align
            if start + size > len(self.buf):
                return None
            self._used = start + size
            return memoryview(self.buf)[start:start + size]

    def alloc(self, value: T) -> Optional[T]:
        if self.alloc_bytes(max(1, _sizeof(value))) is None:
            return None
        self.objects.append(value)
        return value

    def alloc_slice(self, data: Sequence[int]) -> Optional[memoryview]:
        b = bytes(data)
        mv = self.alloc_bytes(len(b), 1)
        if mv is not None:
            mv[:] = b
        return mv

    def reset(self) -> None:
        with self._lock:
            self._used = 0
            self.objects.clear()

    def used(self) -> int:
        return self._used

    def capacity(self) -> int:
        return len(self.buf)

    def remaining(self) -> int:
        return len(self.buf) - self._used


# ------------------------------------------------------------------------------ pools
class Pool(Generic[T]):
    """Capacity-bounded object pool (memory.rs:235-312)."""

    def __init__(self, capacity: int, init: Optional[Callable[[], T]] = None) -> None:
        self.capacity = capacity
        self.init = init
        self.items: List[T] = []
        self._lock = threading.Lock()

    new = classmethod(lambda cls, capacity: cls(capacity))
    with_initializer = classmethod(lambda cls, capacity, init: cls(capacity, init))

    def take(self, default: Optional[Callable[[], T]] = None) -> T:
        with self._lock:
            if self.items:
                return self.items.pop()
        factory = default or self.init
        if factory is None:
            raise LookupError("Pool is empty and has no initializer")
        return factory()

    def take_or_init(self) -> T:
        return self.take()

    def put(self, item: T) -> None:
        with self._lock:
            if len(self.items) < self.capacity:
                self.items.append(item)

    def put_and_reset(self, item: T) -> None:
        reset = getattr(item, "reset", None) or getattr(item, "clear", None)
        if reset is not None:
            reset()
        self.put(item)

    def len(self) -> int:
        return len(self.items)

    __len__ = len

    def is_empty(self) -> bool:
        return not self.items


class PoolReset:
    """Trait of poolable objects (memory.rs:309-312)."""

    def reset(self) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class TokenBufferPool:
    """Pool of byte buffers (memory.rs:576-609): ``acquire`` returns an empty buffer with
    ``buffer_size`` capacity, ``release`` clears it and keeps at most ``max_buffers``."""

    def __init__(self, buffer_size: int, max_buffers: int) -> None:
        self.buffer_size, self.max_buffers = buffer_size, max_buffers
        self.buffers: List[bytearray] = []
        self._lock = threading.Lock()

    new = classmethod(lambda cls, buffer_size, max_buffers: cls(buffer_size, max_buffers))

    def acquire(self) -> bytearray:
        with self._lock:
            if self.buffers:
                return self.buffers.pop()
        return bytearray()

    def release(self, buffer: bytearray) -> None:
        buffer.clear()
        with self._lock:
            if len(self.buffers) < self.max_buffers:
                self.buffers.append(buffer)


class PinnedPool:
    """Page-locked host staging buffers for asynchronous host-to-device copies (the device-side
    use of the reference's ``Pool``): fixed size, reused, never freed while training runs."""

    def __init__(self, shape, dtype, count: int = 2) -> None:
        import torch
        pin = torch.cuda.is_available()
        self.buffers = [torch.empty(shape, dtype=dtype, pin_memory=pin) for _ in range(count)]
        self.next = 0

    def acquire(self):
        b = self.buffers[self.next]
        self.next = (self.next + 1) % len(self.buffers)
        return b


class DeviceArena:
    """Bump allocator over one CUDA buffer for per-step activations and workspaces: ``alloc``
    returns 256-byte-aligned tensor views, ``reset`` rewinds at the end of the step.  Keeps the
    six ``MemoryStats`` counters; 256 bytes of canary pattern can be placed after every
    allocation and verified (``check_canaries``) in debug runs."""

    ALIGN = 256

    def __init__(self, nbytes: int, device="cuda", canaries: bool = False) -> None:
        import torch
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.offset = 0
        self.canaries = canaries
        self._marks: List[int] = []
        self.stats = MemoryStats()

    def alloc(self, shape, dtype):
        import torch
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.offset + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        end = start + nbytes
        pad = self.ALIGN if self.canaries else 0
        if end + pad > self.buf.numel():
            from .error import ResourceError
            raise ResourceError.exhausted("device arena", self.buf.numel() - self.offset, nbytes)
        if self.canaries:
            self.buf[end:end + pad].fill_(0xA5)
            self._marks.append(end)
        self.offset = end + pad
        self.stats.record_allocation(nbytes)
        return self.buf[start:end].view(dtype).view(shape)

    def check_canaries(self) -> bool:
        return all(bool((self.buf[m:m + self.ALIGN] == 0xA5).all()) for m in self._marks)

    def reset(self) -> None:
        self.stats.record_deallocation(self.stats.used_bytes)
        self.offset = 0
        self._marks.clear()

    def used(self) -> int:
        return self.offset

    def capacity(self) -> int:
        return self.buf.numel()


# ------------------------------------------------------------------------------ strings
class CowStr:
    """Borrowed / owned / shared string (memory.rs:320-423)."""

    BORROWED, OWNED, SHARED = "Borrowed", "Owned", "Shared"

    def __init__(self, s: str, kind: str = "Borrowed") -> None:
        self._s, self.kind = s, kind

    @classmethod
    def borrowed(cls, s: str) -> "CowStr":
        return cls(s, cls.BORROWED)

    @classmethod
    def owned(cls, s: str) -> "CowStr":
        return cls(s, cls.OWNED)

    @classmethod
    def shared(cls, s: str) -> "CowStr":
        return cls(s, cls.SHARED)

    def as_str(self) -> str:
        return self._s

    def into_owned(self) -> str:
        return self._s

    def to_mut(self) -> List[str]:
        """Converts to the owned variant and returns a one-element list standing for ``&mut
        String``; use ``push_str`` for in-place edits."""
        self.kind = self.OWNED
        return [self._s]

    def push_str(self, more: str) -> None:
        self.kind = self.OWNED
        self._s += more

    def is_borrowed(self) -> bool:
        return self.kind == self.BORROWED

    def len(self) -> int:
        return len(self._s.encode())

    __len__ = len

    def is_empty(self) -> bool:
        return not self._s

    def __str__(self) -> str:
        return self._s

    def __eq__(self, other: object) -> bool:
        return str(self) == str(other)

    def __hash__(self) -> int:
        return hash(self._s)


class ZeroCopyStringBuilder:
    """Collects segments and joins them once (memory.rs:434-569)."""

    def __init__(self, capacity: int = 0) -> None:
        self.segments: List[str] = []
        self.total_len = 0

    new = classmethod(lambda cls: cls())
    with_capacity = classmethod(lambda cls, capacity: cls(capacity))

    def _push(self, s: str) -> "ZeroCopyStringBuilder":
        if s:
            self.segments.append(s)
            self.total_len += len(s.encode())
        return self

    append_borrowed = _push
    append_owned = _push
    append_shared = _push

    def append_char(self, ch: str) -> "ZeroCopyStringBuilder":
        return self._push(ch)

    def write_str(self, s: str) -> None:
        self._push(s)

    def len(self) -> int:
        return self.total_len

    __len__ = len

    def is_empty(self) -> bool:
        return self.total_len == 0

    def build(self) -> str:
        return "".join(self.segments)


class Rope:
    """Concatenation tree of string pieces (memory.rs:949-1046)."""

    def __init__(self, left: Optional["Rope"] = None, right: Optional["Rope"] = None,
                 leaf: Optional[str] = None) -> None:
        self.left, self.right, self.leaf = left, right, leaf
        if leaf is not None:
            self._len = len(leaf.encode())
        else:
            self._len = (left._len if left else 0) + (right._len if right else 0)

    new = classmethod(lambda cls: cls(leaf=""))

    @classmethod
    def from_str(cls, s: str) -> "Rope":
        return cls(leaf=s)

    def len(self) -> int:
        return self._len

    __len__ = len

    def is_empty(self) -> bool:
        return self._len == 0

    def concat(self, other: "Rope") -> "Rope":
        if self.is_empty():
            return other
        if other.is_empty():
            return self
        return Rope(self, other)

    def leaves(self):
        stack = [self]
        while stack:
            n = stack.pop()
            if n.leaf is not None:
                yield n.leaf
            else:
                if n.right is not None:
                    stack.append(n.right)
                if n.left is not None:
                    stack.append(n.left)

    def to_string(self) -> str:
        return "".join(self.leaves())

    __str__ = to_string


@dataclass
class InternerStats:
    total_requests: int = 0
    cache_hits: int = 0
    unique_strings: int = 0
    memory_saved: int = 0


class StringInterner:
    """Thread-safe string deduplication with hit statistics (memory.rs:1135-1252)."""

    def __init__(self) -> None:
        self._strings = {}
        self._stats = InternerStats()
        self._lock = threading.RLock()

    new = classmethod(lambda cls: cls())

    def intern(self, s: str) -> str:
        with self._lock:
            self._stats.total_requests += 1
            got = self._strings.get(s)
            if got is not None:
                self._stats.cache_hits += 1
                self._stats.memory_saved += len(s.encode())
                return got
            self._strings[s] = s
            self._stats.unique_strings += 1
            return s

    def stats(self) -> InternerStats:
        with self._lock:
            return InternerStats(**self._stats.__dict__)

    def clear(self) -> None:
        with self._lock:
            self._strings.clear()
            self._stats = InternerStats()

    def len(self) -> int:
        return len(self._strings)

    __len__ = len

    def is_empty(self) -> bool:
        return not self._strings


# ------------------------------------------------------------------------------ views
class SliceView(Generic[T]):
    """Lazy chain of ``map`` functions over a sequence (memory.rs:621-688)."""

    def __init__(self, data: Sequence[T]) -> None:
        self.data = data
        self.fns: List[Callable[[Any], Any]] = []

    new = classmethod(lambda cls, data: cls(data))

    def map(self, f: Callable[[Any], Any]) -> "SliceView":
        self.fns.append(f)
        return self

    def get(self, index: int) -> Optional[Any]:
        if index < 0 or index >= len(self.data):
            return None
        v = self.data[index]
        for f in self.fns:
            v = f(v)
        return v

    def len(self) -> int:
        return len(self.data)

    __len__ = len

    def is_empty(self) -> bool:
        return len(self.data) == 0

    def to_vec(self) -> List[Any]:
        return [self.get(i) for i in range(len(self.data))]


class MappedBuffer:
    """Read-only memory-mapped file (the reference's type of this name only wraps a raw pointer,
    memory.rs:699-745; checkpoint loaders here use it to read tensors without copying)."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self._size = size

    def as_slice(self) -> memoryview:
        return memoryview(self._mm) if self._mm is not None else memoryview(b"")

    def len(self) -> int:
        return self._size

    __len__ = len

    def is_empty(self) -> bool:
        return self._size == 0

    def slice(self, start: int, end: int) -> Optional[memoryview]:
        if start <= end <= self._size:
            return self.as_slice()[start:end]
        return None

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


class LazyAlloc(Generic[T]):
    """Initialise on first use, once (memory.rs:756-826)."""

    def __init__(self, init: Callable[[], T]) -> None:
        self._init = init
        self._value: Optional[T] = None
        self._done = False
        self._lock = threading.Lock()

    new = classmethod(lambda cls, init: cls(init))

    def get_or_init(self) -> T:
        if not self._done:
            with self._lock:
                if not self._done:
                    self._value = self._init()
                    self._done = True
        return self._value  # type: ignore[return-value]

    def is_initialized(self) -> bool:
        return self._done


# ------------------------------------------------------------------------------ benchmarks
@dataclass
class AllocationBenchmark:
    """memory.rs:1054-1093."""

    allocations: int = 0
    bytes_allocated: int = 0
    peak_usage: int = 0

    def record_allocation(self, nbytes: int) -> None:
        self.allocations += 1
        self.bytes_allocated += nbytes
        self.peak_usage = max(self.peak_usage, self.bytes_allocated)

    def record_deallocation(self, nbytes: int) -> None:
        self.bytes_allocated = max(0, self.bytes_allocated - nbytes)

    def reset(self) -> None:
        self.allocations = self.bytes_allocated = self.peak_usage = 0


@dataclass
class BenchmarkResult:
    """memory.rs:1096-1127; ``elapsed`` in seconds."""

    allocations: int = 0
    bytes_allocated: int = 0
    peak_usage: int = 0
    elapsed: float = 0.0

    def allocations_per_second(self) -> float:
        return self.allocations / self.elapsed if self.elapsed > 0 else 0.0

    def mb_per_second(self) -> float:
        return (self.bytes_allocated / 1_048_576.0) / self.elapsed if self.elapsed > 0 else 0.0
