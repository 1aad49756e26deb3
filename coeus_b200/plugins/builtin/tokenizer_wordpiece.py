"""WordPiece tokenizer (plugins/tokenizer-wordpiece/src/lib.rs) over the native trie in
``csrc/host/tokenizers.cpp``: vocabulary ``[UNK]=0 [CLS]=1 [SEP]=2 [PAD]=3 [MASK]=4``, ``a..z`` =
100..125, ``A..Z`` = 126..151, thirteen ``##`` suffixes = 152..164; NFD normalisation, word
segmentation, greedy longest match with ``##`` continuation (a miss emits ``[UNK]`` and abandons
the word), output wrapped in ``[CLS] ... [SEP]``; ``decode`` skips bracketed tokens, glues ``##``
pieces and joins words with one space."""
from __future__ import annotations

from typing import Iterable, Iterator, List, Optional

from ...core.plugin import PluginCapabilities, TokenizerPlugin
from ...core.tokenizer import (NormalizingTokenizer, SpecialTokenizer, StringToken, Token,
                               TokenizerConfig)
from ...foundation.types import Version
from ...utils import native


class WordPieceTokenizer(NormalizingTokenizer, SpecialTokenizer):
    def __init__(self, config: Optional[TokenizerConfig] = None) -> None:
        self._config = config or TokenizerConfig()
        self._t = native.module().WordPieceTokenizer()

    new = classmethod(lambda cls, config=None: cls(config))

    def name(self) -> str:
        return "wordpiece"

    def normalize(self, text: str) -> str:
        return native.module().nfd(text)

    def encode(self, text: str) -> List[int]:
        return list(self._t.encode(text))

    def tokenize(self, input: str) -> Iterator[Token]:
        return iter([StringToken.with_id(self._t.id_to_token(i), int(i)) for i in self._t.encode(input)])

    def decode(self, tokens: Iterable[Token]) -> str:
        return self._t.decode_strings([t.as_str() or "" for t in tokens])

    def vocab_size(self) -> int:
        return self._t.vocab_size()

    def token_to_id(self, token: str) -> Optional[int]:
        return self._t.token_to_id(token)

    def id_to_token(self, id: int) -> Optional[str]:
        return self._t.id_to_token(int(id))

    def add_token(self, token: str, id: int) -> None:
        self._t.add_token(token, int(id))

    # ---- persistence
    def vocabulary(self, max_id: int = 1 << 22) -> List[tuple]:
        """``(token, id)`` for every entry, by id."""
        out, want = [], self._t.vocab_size()
        i = 0
        while len(out) < want and i < max_id:
            t = self._t.id_to_token(i)
            if t is not None:
                out.append((t, i))
            i += 1
        return out

    def save(self, path: str) -> None:
        import json
        with open(path, "w", encoding="utf-8") as f:
            json.dump({"type": "wordpiece_tokenizer", "version": 1,
                       "vocab": self.vocabulary()}, f, ensure_ascii=False)

    @classmethod
    def load(cls, path: str, config: Optional[TokenizerConfig] = None) -> "WordPieceTokenizer":
        import json
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
        if d.get("type") != "wordpiece_tokenizer":
            raise ValueError(f"{path} is not a saved WordPiece tokenizer")
        t = cls(config)
        have = dict(t.vocabulary())
        for tok, i in d["vocab"]:
            if have.get(tok) != i:
                t.add_token(tok, int(i))
        return t

    def longest_match(self, text: str):
        return self._t.longest_match(text)

    def config(self) -> TokenizerConfig:
        return self._config

    def unk_token(self) -> Token:
        return StringToken.with_id("[UNK]", 0)

    def pad_token(self) -> Token:
        return StringToken.with_id("[PAD]", 3)

    def bos_token(self) -> Token:
        return StringToken.with_id("[CLS]", 1)

    def eos_token(self) -> Token:
        return StringToken.with_id("[SEP]", 2)

    def mask_token(self) -> Token:
        return StringToken.with_id("[MASK]", 4)


class WordPieceTokenizerPlugin(TokenizerPlugin):
    def id(self) -> str:
        return "wordpiece_tokenizer"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        c = PluginCapabilities.standard()
        for f in ("tokenization", "wordpiece", "unicode", "subword"):
            c.with_feature(f)
        return c

    def create_tokenizer(self) -> WordPieceTokenizer:
        return WordPieceTokenizer(TokenizerConfig())
