"""Tokenization context (src/domain/tokenization/mod.rs): ``Token{id,text,score}``,
``Vocabulary``, the ``TokenizerConfig`` entity (constructible here; the reference's has private
fields and no constructor), ``TokenizerAggregate.tokenize`` (whitespace split, optional lowercase,
out-of-vocabulary words are dropped, mod.rs:150-163), ``TokenizationService``, events, repository
interface and application service."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..foundation.error import ConfigError, PluginError


@dataclass(frozen=True)
class Token:
    id: int
    text: str
    score: Optional[float] = None

    @classmethod
    def new(cls, id: int, text: str) -> "Token":
        return cls(id, text)

    def with_score(self, score: float) -> "Token":
        return Token(self.id, self.text, score)


class Vocabulary:
    def __init__(self, tokens: Sequence[str]) -> None:
        self.tokens: List[str] = list(tokens)
        self._index: Dict[str, int] = {t: i for i, t in enumerate(self.tokens)}

    new = classmethod(lambda cls, tokens: cls(tokens))

    def token_to_id(self, token: str) -> Optional[int]:
        return self._index.get(token)

    def id_to_token(self, id: int) -> Optional[str]:
        return self.tokens[id] if 0 <= id < len(self.tokens) else None

    def size(self) -> int:
        return len(self.tokens)

    __len__ = size


@dataclass
class TokenizerConfig:
    id_: str
    name: str
    vocab_size: int
    special_tokens: List[str] = field(default_factory=list)
    lowercase: bool = False
    strip_accents: bool = False

    def id(self) -> str:
        return self.id_


class TokenizerAggregate:
    def __init__(self, config: TokenizerConfig, vocabulary: Vocabulary) -> None:
        self.config, self.vocabulary = config, vocabulary
        self._state = "Initialized"

    new = classmethod(lambda cls, config, vocabulary: cls(config, vocabulary))

    def tokenize(self, text: str) -> List[Token]:
        self._state = "Processing"
        out = []
        for word in text.split():
            w = word.lower() if self.config.lowercase else word
            i = self.vocabulary.token_to_id(w)
            if i is not None:
                out.append(Token.new(i, w))
        self._state = "Ready"
        return out

    def state(self) -> str:
        return self._state


class TokenizationService:
    @staticmethod
    def merge_vocabularies(vocabs: Sequence[Vocabulary]) -> Vocabulary:
        seen, merged = set(), []
        for v in vocabs:
            for t in v.tokens:
                if t not in seen:
                    seen.add(t)
                    merged.append(t)
        return Vocabulary(merged)

    @staticmethod
    def validate_config(config: TokenizerConfig) -> None:
        if config.vocab_size == 0:
            raise ConfigError.invalid("vocab_size", config.vocab_size,
                                      "Vocabulary size must be greater than 0")


@dataclass(frozen=True)
class TokenizationEvent:
    kind: str          # Started | Completed | Failed | VocabularyUpdated
    tokenizer_id: str
    text_length: int = 0
    token_count: int = 0
    error: str = ""
    new_size: int = 0


class TokenizerRepository(abc.ABC):
    @abc.abstractmethod
    def save(self, config: TokenizerConfig) -> None: ...

    @abc.abstractmethod
    def load(self, id: str) -> TokenizerConfig: ...

    @abc.abstractmethod
    def list(self) -> List[str]: ...

    @abc.abstractmethod
    def delete(self, id: str) -> None: ...


class InMemoryTokenizerRepository(TokenizerRepository):
    def __init__(self) -> None:
        self._items: Dict[str, TokenizerConfig] = {}

    def save(self, config: TokenizerConfig) -> None:
        self._items[config.id()] = config

    def load(self, id: str) -> TokenizerConfig:
        if id not in self._items:
            raise PluginError.not_found(id, list(self._items))
        return self._items[id]

    def list(self) -> List[str]:
        return list(self._items)

    def delete(self, id: str) -> None:
        self._items.pop(id, None)


class TokenizationApplicationService:
    def __init__(self, repository: TokenizerRepository) -> None:
        self.repository = repository
        self.domain_service = TokenizationService()
        self.events: List[TokenizationEvent] = []

    new = classmethod(lambda cls, repository: cls(repository))

    def create_tokenizer(self, config: TokenizerConfig, vocabulary: Vocabulary) -> TokenizerAggregate:
        TokenizationService.validate_config(config)
        self.repository.save(config)
        self.events.append(TokenizationEvent("VocabularyUpdated", config.id(),
                                             new_size=vocabulary.size()))
        return TokenizerAggregate(config, vocabulary)

    def load_tokenizer(self, id: str, vocabulary: Vocabulary) -> TokenizerAggregate:
        return TokenizerAggregate(self.repository.load(id), vocabulary)
