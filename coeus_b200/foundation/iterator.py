"""Iterator adapters (counterpart of src/foundation/iterator.rs).

``Iter`` wraps any iterable and offers the reference's ``IteratorExt`` methods (``windows``,
``windows_step``, ``chunks``, ``stride``, ``batch``, ``scan_with``, ``prefetch``,
``stream_fusion``, ``cache_oblivious``, ``into_zipper``) with the same observable results:
``windows`` yields ``len - N + 1`` windows and stops when the source runs dry in the middle of a
step (iterator.rs:160-182), ``chunks`` yields a short last chunk (:500-504), ``stride`` takes one
and skips ``S - 1`` (:539-547).  One deliberate difference: ``batch(...).with_memory_limit``
carries the item that overflowed the limit into the next batch, where the reference drops it
(iterator.rs:617-624).  The "literature" iterators (rope, B-tree, suffix array, wavelet-tree
placeholder, trie, Bloom-filter bits) follow.  The token-stream versions that feed training
(windows / chunks / batch over int32 arrays with a pinned double-buffer prefetch) are native, in
``csrc/host/pipeline.cpp``, and are reached through :mod:`coeus_b200.train.data`.
"""
from __future__ import annotations

import math
import sys
import threading
from collections import deque
from typing import Any, Callable, Generic, Iterable, Iterator, List, Optional, Sequence, Tuple, TypeVar

T = TypeVar("T")
U = TypeVar("U")


# ------------------------------------------------------------------------------ adapters
class Windows(Generic[T]):
    def __init__(self, it: Iterable[T], size: int, step: int = 1) -> None:
        assert size > 0, "Window size must be greater than 0"
        assert step > 0, "Step size must be greater than 0"
        self.it = iter(it)
        self.size, self.step = size, step
        self.buf: List[T] = []
        self.exhausted = False

    def window_size(self) -> int:
        return self.size

    def step_size(self) -> int:
        return self.step

    def __iter__(self) -> "Windows[T]":
        return self

    def __next__(self) -> Tuple[T, ...]:
        if self.exhausted:
            raise StopIteration
        while len(self.buf) < self.size:
            try:
                self.buf.append(next(self.it))
            except StopIteration:
                self.exhausted = True
                raise
        out = tuple(self.buf)
        for _ in range(self.step):
            self.buf.pop(0)
            try:
                self.buf.append(next(self.it))
            except StopIteration:
                self.exhausted = True
                break
        return out


class SliceWindows(Generic[T]):
    """Views of a sequence without copying the source (iterator.rs:226-270)."""

    def __init__(self, data: Sequence[T], size: int, step: int = 1) -> None:
        assert size > 0 and step > 0
        self.data, self.size, self.step = data, size, step
        self.pos = 0

    def __len__(self) -> int:
        n = len(self.data) - self.pos
        return 0 if n < self.size else (n - self.size) // self.step + 1

    len = __len__

    def size_hint(self) -> Tuple[int, Optional[int]]:
        return (len(self), len(self))

    def __iter__(self) -> "SliceWindows[T]":
        return self

    def __next__(self) -> Sequence[T]:
        if self.pos + self.size > len(self.data):
            raise StopIteration
        w = self.data[self.pos:self.pos + self.size]
        self.pos += self.step
        return w


def slice_windows(data: Sequence[T], size: int) -> SliceWindows[T]:
    return SliceWindows(data, size, 1)


def slice_windows_step(data: Sequence[T], size: int, step: int) -> SliceWindows[T]:
    return SliceWindows(data, size, step)


class StreamFusion(Generic[T, U]):
    """filter + map in one pass: ``f`` returns ``None`` to drop (iterator.rs:279-324)."""

    def __init__(self, it: Iterable[T], f: Callable[[T], Optional[U]]) -> None:
        self.it, self.f = iter(it), f

    def __iter__(self):
        for x in self.it:
            y = self.f(x)
            if y is not None:
                yield y


class CacheOblivious(Generic[T]):
    """Block-buffered pass-through (iterator.rs:333-379)."""

    def __init__(self, it: Iterable[T], block_size: int) -> None:
        self.it, self.block_size = iter(it), block_size

    def __iter__(self):
        while True:
            block = []
            for _ in range(self.block_size):
                try:
                    block.append(next(self.it))
                except StopIteration:
                    break
            if not block:
                return
            yield from block


class Zipper(Generic[T]):
    """Huet zipper.  As in the reference the initial focus is the LAST element and
    ``into_vec`` after moves returns the rotated order its test asserts (``[5,1,2,3,4]``,
    iterator.rs:398-452, :1588-1613)."""

    def __init__(self, items: Sequence[T]) -> None:
        items = list(items)
        self.focus: Optional[T] = items.pop() if items else None
        items.reverse()
        self.left: List[T] = []
        self.right: List[T] = items

    new = classmethod(lambda cls, items: cls(items))

    def move_right(self) -> bool:
        if self.right:
            item = self.right.pop()
            if self.focus is not None:
                self.left.append(self.focus)
            self.focus = item
            return True
        return False

    def move_left(self) -> bool:
        if self.left:
            item = self.left.pop()
            if self.focus is not None:
                self.right.append(self.focus)
            self.focus = item
            return True
        return False

    def current(self) -> Optional[T]:
        return self.focus

    def set_current(self, value: T) -> None:
        self.focus = value

    def into_vec(self) -> List[T]:
        right = list(reversed(self.right))
        out = list(self.left)
        if self.focus is not None:
            out.append(self.focus)
        out.extend(right)
        return out


class Chunks(Generic[T]):
    def __init__(self, it: Iterable[T], size: int) -> None:
        assert size > 0, "Chunk size must be greater than 0"
        self.it, self.size = iter(it), size

    def __iter__(self):
        while True:
            chunk = []
            for _ in range(self.size):
                try:
                    chunk.append(next(self.it))
                except StopIteration:
                    break
            if not chunk:
                return
            yield chunk


class Stride(Generic[T]):
    def __init__(self, it: Iterable[T], stride: int) -> None:
        assert stride > 0, "Stride must be greater than 0"
        self.it, self.stride = iter(it), stride

    def __iter__(self):
        while True:
            try:
                item = next(self.it)
            except StopIteration:
                return
            yield item
            for _ in range(self.stride - 1):
                try:
                    next(self.it)
                except StopIteration:
                    return


class BatchIterator(Generic[T]):
    """Batches of ``min_size..max_size`` items, optionally bounded by an estimated memory size
    (iterator.rs:562-640).  The item that would overflow the memory limit starts the next batch
    (the reference loses it)."""

    def __init__(self, it: Iterable[T], min_size: int, max_size: int) -> None:
        assert min_size > 0, "Min batch size must be greater than 0"
        assert max_size >= min_size, "Max batch size must be >= min batch size"
        self.it = iter(it)
        self.min_size, self.max_size = min_size, max_size
        self.max_memory: Optional[int] = None
        self._carry: List[T] = []

    def with_memory_limit(self, nbytes: int) -> "BatchIterator[T]":
        self.max_memory = nbytes
        return self

    @staticmethod
    def estimate_size(item: Any) -> int:
        return 4 if isinstance(item, int) else sys.getsizeof(item)

    def __iter__(self):
        while True:
            batch: List[T] = []
            mem = 0
            while len(batch) < self.max_size:
                if self._carry:
                    item = self._carry.pop()
                else:
                    try:
                        item = next(self.it)
                    except StopIteration:
                        break
                size = self.estimate_size(item)
                if (self.max_memory is not None and mem + size > self.max_memory
                        and len(batch) >= self.min_size):
                    self._carry.append(item)
                    break
                mem += size
                batch.append(item)
            if not batch:
                return
            yield batch


class Scan(Generic[T, U]):
    """Stateful map: ``f(state, item) -> (state, output or None)``; ``None`` ends the scan
    (iterator.rs:697-735)."""

    def __init__(self, it: Iterable[T], state: Any, f: Callable[[Any, T], Tuple[Any, Optional[U]]]) -> None:
        self.it, self.state, self.f = iter(it), state, f

    def __iter__(self):
        for x in self.it:
            self.state, out = self.f(self.state, x)
            if out is None:
                return
            yield out


class Prefetch(Generic[T]):
    """Keeps up to ``n`` items fetched ahead of the consumer (iterator.rs:740-801).  With
    ``threaded=True`` a background thread fills the buffer, which is what hides data-loading
    latency behind a training step."""

    def __init__(self, it: Iterable[T], n: int, threaded: bool = False) -> None:
        assert n > 0
        self.it, self.n, self.threaded = iter(it), n, threaded

    def __iter__(self):
        if not self.threaded:
            buf: deque = deque()
            done = False
            while True:
                while not done and len(buf) < self.n:
                    try:
                        buf.append(next(self.it))
                    except StopIteration:
                        done = True
                if not buf:
                    return
                yield buf.popleft()
        else:
            import queue
            q: "queue.Queue" = queue.Queue(maxsize=self.n)
            end = object()

            def fill():
                try:
                    for x in self.it:
                        q.put(x)
                finally:
                    q.put(end)

            t = threading.Thread(target=fill, daemon=True)
            t.start()
            while True:
                x = q.get()
                if x is end:
                    return
                yield x


class ZeroCopyTokenizer:
    """Splits on a one-byte delimiter, yielding slices; a trailing empty piece is dropped and
    the delimiter is treated as a single byte (iterator.rs:644-692)."""

    def __init__(self, text: str, delimiter: str) -> None:
        self.text, self.delim = text, delimiter

    def __iter__(self):
        text, pos, n = self.text, 0, len(self.text)
        while pos < n:
            start = pos
            idx = text.find(self.delim, pos)
            pos = n if idx < 0 else idx
            token = text[start:pos]
            if pos < n:
                pos += 1
            if token == "" and pos >= n:
                return
            yield token


class ZeroCopySplit:
    """``str::split`` without allocation of the pieces (iterator.rs:1455-1498): keeps empty
    pieces, including a trailing one."""

    def __init__(self, text: str, delimiter: str) -> None:
        self.text, self.delim = text, delimiter

    def __iter__(self):
        if self.text == "":
            return
        yield from self.text.split(self.delim)


class Iter(Generic[T]):
    """``IteratorExt`` as a wrapper: ``Iter(xs).windows(3)`` ... every method returns an
    ``Iter`` so adapters chain like in the reference (iterator.rs:1362-1431)."""

    def __init__(self, it: Iterable[T]) -> None:
        self._it = it

    def __iter__(self) -> Iterator[T]:
        return iter(self._it)

    def windows(self, n: int) -> "Iter[Tuple[T, ...]]":
        return Iter(Windows(self._it, n, 1))

    def windows_step(self, n: int, step: int) -> "Iter[Tuple[T, ...]]":
        return Iter(Windows(self._it, n, step))

    def stream_fusion(self, f: Callable[[T], Optional[U]]) -> "Iter[U]":
        return Iter(StreamFusion(self._it, f))

    def cache_oblivious(self, block_size: int) -> "Iter[T]":
        return Iter(CacheOblivious(self._it, block_size))

    def into_zipper(self) -> Zipper[T]:
        return Zipper(list(self._it))

    def chunks(self, n: int) -> "Iter[List[T]]":
        return Iter(Chunks(self._it, n))

    def stride(self, s: int) -> "Iter[T]":
        return Iter(Stride(self._it, s))

    def batch(self, min_size: int, max_size: int) -> BatchIterator[T]:
        return BatchIterator(self._it, min_size, max_size)

    def scan_with(self, state: Any, f) -> "Iter[Any]":
        return Iter(Scan(self._it, state, f))

    def prefetch(self, n: int, threaded: bool = False) -> "Iter[T]":
        return Iter(Prefetch(self._it, n, threaded))

    def map(self, f: Callable[[T], U]) -> "Iter[U]":
        return Iter(map(f, self._it))

    def filter(self, f: Callable[[T], bool]) -> "Iter[T]":
        return Iter(filter(f, self._it))

    def collect(self) -> List[T]:
        return list(self._it)

    # AdvancedIteratorExt (iterator.rs:1257-1285)
    def into_rope_owned(self) -> "OwnedRopeIterator":
        return OwnedRopeIterator(list(self._it))

    def into_suffix_array(self) -> "SuffixArrayIterator":
        return SuffixArrayIterator("".join(self._it))


IteratorExt = Iter
AdvancedIteratorExt = Iter


class IteratorAdapter:
    """An iterator that wraps a source iterator (iterator.rs:37-46)."""

    def source(self):
        return self._it

    def source_mut(self):
        return self._it


class StatefulIterator:
    """An iterator with an inspectable, resettable state (iterator.rs:49-58)."""

    def state(self):
        raise NotImplementedError

    def reset_state(self) -> None:
        raise NotImplementedError


class PreciseSizeHint:
    """``exact_size`` / ``is_empty`` on top of a size hint (iterator.rs:63-79; the reference
    implements it for every iterator).  ``size_hint`` returns ``(lower, upper or None)``."""

    def __init__(self, it: Iterable) -> None:
        self._it = it

    def __iter__(self):
        return iter(self._it)

    def size_hint(self) -> Tuple[int, Optional[int]]:
        try:
            n = len(self._it)              # type: ignore[arg-type]
            return n, n
        except TypeError:
            import operator
            return operator.length_hint(self._it, 0), None

    def exact_size(self) -> Optional[int]:
        lo, hi = self.size_hint()
        return lo if hi == lo else None

    def is_empty(self) -> bool:
        return self.size_hint()[1] == 0


# ------------------------------------------------------------------------------ literature
class RopeNode:
    """``Leaf(str)`` or ``Branch{left,right}`` (public constructors, unlike the reference's
    private node type, iterator.rs:812-829)."""

    def __init__(self, leaf: Optional[str] = None, left: Optional["RopeNode"] = None,
                 right: Optional["RopeNode"] = None) -> None:
        self.leaf, self.left, self.right = leaf, left, right

    @classmethod
    def Leaf(cls, s: str) -> "RopeNode":
        return cls(leaf=s)

    @classmethod
    def Branch(cls, left: "RopeNode", right: "RopeNode") -> "RopeNode":
        return cls(left=left, right=right)


class RopeIterator:
    """Characters of a rope in order."""

    def __init__(self, root: RopeNode) -> None:
        self.root = root

    new = classmethod(lambda cls, root: cls(root))

    def __iter__(self):
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n.leaf is not None:
                yield from n.leaf
            else:
                if n.right is not None:
                    stack.append(n.right)
                if n.left is not None:
                    stack.append(n.left)


class OwnedRopeIterator:
    def __init__(self, pieces: Sequence[str]) -> None:
        self.pieces = list(pieces)

    def __iter__(self):
        for p in self.pieces:
            yield from p


class BTreeNode(Generic[T]):
    def __init__(self, keys: Sequence[T], children: Optional[Sequence[int]] = None) -> None:
        self.keys = list(keys)
        self.children = list(children) if children is not None else None
        self.is_leaf = children is None

    @property
    def len(self) -> int:
        return len(self.keys)


class BTreeIterator(Generic[T]):
    """In-order traversal of index-linked B-tree nodes; the root is the LAST node of the list
    (iterator.rs:882-988; its test builds leaves first, root last)."""

    def __init__(self, nodes: Sequence[BTreeNode[T]]) -> None:
        self.nodes = list(nodes)

    new = classmethod(lambda cls, nodes: cls(nodes))

    def __iter__(self):
        if not self.nodes:
            return
        yield from self._walk(len(self.nodes) - 1)

    def _walk(self, idx: int):
        node = self.nodes[idx]
        if node.is_leaf:
            yield from node.keys
            return
        for i, key in enumerate(node.keys):
            if i < len(node.children):
                yield from self._walk(node.children[i])
            yield key
        if len(node.children) > len(node.keys):
            yield from self._walk(node.children[len(node.keys)])


def suffix_array(text: str) -> List[int]:
    """Prefix doubling, O(n log^2 n) -- which is what the reference implements under a "DC3"
    comment (iterator.rs:1019-1058).  The native version is ``textalgo.suffix_array``."""
    n = len(text)
    if n == 0:
        return []
    sa = list(range(n))
    rank = [ord(c) for c in text]
    k = 1
    while True:
        key = lambda i: (rank[i], rank[i + k] if i + k < n else -1)  # noqa: E731
        sa.sort(key=key)
        tmp = [0] * n
        for j in range(1, n):
            tmp[sa[j]] = tmp[sa[j - 1]] + (1 if key(sa[j]) != key(sa[j - 1]) else 0)
        rank = tmp
        if rank[sa[-1]] == n - 1:
            break
        k <<= 1
    return sa


class SuffixArrayIterator:
    """Yields the suffixes of a text in sorted order."""

    def __init__(self, text: str) -> None:
        self.text = text
        try:
            from ..utils import native
            self.sa = native.suffix_array(text) if native.available() and text.isascii() \
                else suffix_array(text)
        except Exception:
            self.sa = suffix_array(text)

    new = classmethod(lambda cls, text: cls(text))

    def __iter__(self):
        for i in self.sa:
            yield self.text[i:]


class WaveletTreeIterator(Generic[T]):
    """Placeholder kept from the reference: sorts and iterates (iterator.rs:1084-1125)."""

    def __init__(self, data: Sequence[T]) -> None:
        self.data = sorted(data)

    new = classmethod(lambda cls, data: cls(data))

    def __iter__(self):
        return iter(self.data)


class TrieNode:
    __slots__ = ("children", "is_end")

    def __init__(self) -> None:
        self.children: List[Optional["TrieNode"]] = [None] * 26
        self.is_end = False


class TrieIterator:
    """26-ary trie over lowercase ASCII words; depth-first iteration yields the stored words in
    lexicographic order (iterator.rs:1132-1171)."""

    def __init__(self, words: Iterable[str] = ()) -> None:
        self.root = TrieNode()
        for w in words:
            self.insert(w)

    new = classmethod(lambda cls, words=(): cls(words))

    def insert(self, word: str) -> None:
        node = self.root
        for ch in word:
            i = ord(ch) - 97
            if not 0 <= i < 26:
                return
            if node.children[i] is None:
                node.children[i] = TrieNode()
            node = node.children[i]
        node.is_end = True

    def __iter__(self):
        stack: List[Tuple[TrieNode, str]] = [(self.root, "")]
        while stack:
            node, prefix = stack.pop()
            if node.is_end:
                yield prefix
            for i in range(25, -1, -1):
                c = node.children[i]
                if c is not None:
                    stack.append((c, prefix + chr(97 + i)))


class BloomFilterBitIterator:
    """Bit vector of a Bloom filter with the reference's sizing formula and multiplicative hash
    (iterator.rs:1181-1254).  Iterating yields the BITS, not members."""

    MASK = (1 << 64) - 1

    def __init__(self, expected_items: int, false_positive_rate: float) -> None:
        bits_per_item = -(math.log(false_positive_rate) / (math.log(2.0) ** 2))
        total = int(math.ceil(expected_items * bits_per_item))
        self.hash_count = int(math.ceil(bits_per_item * math.log(2.0)))
        self.bits = [False] * total

    new = classmethod(lambda cls, n, p: cls(n, p))

    def set_bit(self, index: int) -> None:
        if 0 <= index < len(self.bits):
            self.bits[index] = True

    def get_bit(self, index: int) -> bool:
        return self.bits[index] if 0 <= index < len(self.bits) else False

    def bit_count(self) -> int:
        return len(self.bits)

    def popcount(self) -> int:
        return sum(self.bits)

    def _murmur(self, data: bytes, seed: int) -> int:
        h = seed
        for b in data:
            h ^= b
            h = (h * 0x5BD1E995) & self.MASK
            h ^= h >> 15
        return h

    def hash(self, item: bytes, k: int) -> int:
        h1 = self._murmur(item, 0)
        h2 = self._murmur(item, h1)
        return ((h1 + k * h2) & self.MASK) % len(self.bits)

    def insert(self, item: bytes) -> None:
        for k in range(self.hash_count):
            self.set_bit(self.hash(item, k))

    def contains(self, item: bytes) -> bool:
        return all(self.get_bit(self.hash(item, k)) for k in range(self.hash_count))

    def __iter__(self):
        return iter(self.bits)
