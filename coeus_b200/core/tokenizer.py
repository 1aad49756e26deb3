"""Tokenizer contracts (counterpart of src/core/tokenizer.rs): ``Token`` / ``StringToken`` /
``PositionedToken``, the ``Tokenizer`` interface (``tokenize``, ``tokenize_str``, ``decode``,
``vocab_size``, ``name``) and its extensions, and ``TokenizerConfig`` with the padding and
truncation strategies.  Added for the device path: ``encode`` / ``encode_batch`` that return token
ids directly (lists or an int32 tensor) without materialising token objects."""
from __future__ import annotations

import abc
import enum
from dataclasses import dataclass
from typing import Iterable, Iterator, List, Optional, Sequence


# ``Box<dyn Iterator<Item = T>>`` (src/core/tokenizer.rs:14): any iterator of tokens.
TokenIterator = Iterator

class Token(abc.ABC):
    @abc.abstractmethod
    def id(self) -> int: ...

    @abc.abstractmethod
    def as_str(self) -> Optional[str]: ...

    def as_bytes(self) -> Optional[bytes]:
        s = self.as_str()
        return None if s is None else s.encode("utf-8")


class StringToken(Token):
    """A token backed by its string; ``id()`` is 0 when no id was given (tokenizer.rs:61-63)."""

    __slots__ = ("value", "_id")

    def __init__(self, value: str, id: Optional[int] = None) -> None:
        self.value, self._id = value, id

    @classmethod
    def new(cls, value: str) -> "StringToken":
        return cls(value)

    @classmethod
    def with_id(cls, value: str, id: int) -> "StringToken":
        return cls(value, id)

    def id(self) -> int:
        return 0 if self._id is None else self._id

    def as_str(self) -> Optional[str]:
        return self.value

    def len(self) -> int:
        return len(self.value.encode("utf-8"))

    __len__ = len

    def is_empty(self) -> bool:
        return self.value == ""

    def __eq__(self, other: object) -> bool:
        return isinstance(other, StringToken) and (self.value, self._id) == (other.value, other._id)

    def __hash__(self) -> int:
        return hash((self.value, self._id))

    def __repr__(self) -> str:
        return f"StringToken({self.value!r}, id={self._id})"


class PositionedToken(Token):
    def __init__(self, token: Token, start: int, end: int) -> None:
        self._token, self._start, self._end = token, start, end

    new = classmethod(lambda cls, token, start, end: cls(token, start, end))

    def token(self) -> Token:
        return self._token

    def start(self) -> int:
        return self._start

    def end(self) -> int:
        return self._end

    def id(self) -> int:
        return self._token.id()

    def as_str(self) -> Optional[str]:
        return self._token.as_str()


class Tokenizer(abc.ABC):
    @abc.abstractmethod
    def tokenize(self, input: str) -> Iterator[Token]: ...

    def tokenize_str(self, input: str) -> Iterator[Token]:
        return self.tokenize(input)

    @abc.abstractmethod
    def decode(self, tokens: Iterable[Token]) -> str: ...

    @abc.abstractmethod
    def vocab_size(self) -> int: ...

    @abc.abstractmethod
    def name(self) -> str: ...

    # ---- id-level fast path (no counterpart in the reference)
    def encode(self, text: str) -> List[int]:
        return [t.id() for t in self.tokenize(text)]

    def encode_batch(self, texts: Sequence[str], as_tensor: bool = False):
        rows = [self.encode(t) for t in texts]
        if not as_tensor:
            return rows
        import torch
        n = max((len(r) for r in rows), default=0)
        out = torch.zeros((len(rows), n), dtype=torch.int32)
        for i, r in enumerate(rows):
            out[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        return out


class VocabularyTokenizer(Tokenizer):
    @abc.abstractmethod
    def add_token(self, token: str) -> int: ...

    @abc.abstractmethod
    def remove_token(self, token: str) -> None: ...

    @abc.abstractmethod
    def contains_token(self, token: str) -> bool: ...

    @abc.abstractmethod
    def token_from_id(self, id: int) -> Optional[str]: ...

    @abc.abstractmethod
    def id_from_token(self, token: str) -> Optional[int]: ...


class SpecialTokenizer(Tokenizer):
    def pad_token(self) -> Optional[Token]:
        return None

    def unk_token(self) -> Optional[Token]:
        return None

    def bos_token(self) -> Optional[Token]:
        return None

    def eos_token(self) -> Optional[Token]:
        return None

    def mask_token(self) -> Optional[Token]:
        return None


class NormalizingTokenizer(Tokenizer):
    @abc.abstractmethod
    def normalize(self, text: str) -> str: ...

    def tokenize_normalized(self, input: str) -> Iterator[Token]:
        return self.tokenize(self.normalize(input))


class PreTokenizer(abc.ABC):
    @abc.abstractmethod
    def pre_tokenize(self, input: str) -> Iterator[str]: ...


class PostProcessor(abc.ABC):
    @abc.abstractmethod
    def post_process(self, tokens: List[Token]) -> List[Token]: ...


class PaddingStrategy(enum.Enum):
    None_ = "None"
    MaxLength = "MaxLength"
    Longest = "Longest"


class TruncationStrategy(enum.Enum):
    None_ = "None"
    MaxLength = "MaxLength"
    LongestFirst = "LongestFirst"
    OnlySecond = "OnlySecond"


@dataclass
class TokenizerConfig:
    """tokenizer.rs:214-246."""

    max_length: Optional[int] = None
    add_special_tokens: bool = True
    lowercase: bool = False
    strip_accents: bool = False
    padding: PaddingStrategy = PaddingStrategy.None_
    truncation: TruncationStrategy = TruncationStrategy.None_

    def apply(self, ids: List[int], pad_id: int = 0) -> List[int]:
        """Truncate / pad one id sequence according to this configuration."""
        if self.max_length is not None and self.truncation is not TruncationStrategy.None_:
            ids = ids[: self.max_length]
        if self.max_length is not None and self.padding is PaddingStrategy.MaxLength:
            ids = ids + [pad_id] * max(0, self.max_length - len(ids))
        return ids
