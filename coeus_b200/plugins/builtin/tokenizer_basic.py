"""Whitespace tokenizer (plugins/tokenizer-basic/src/lib.rs): ``tokenize`` splits on Unicode
whitespace into id-less ``StringToken``s, ``decode`` joins with one space, ``vocab_size`` is 0."""
from __future__ import annotations

from typing import Iterable, Iterator

from ...core.plugin import PluginCapabilities, TokenizerPlugin
from ...core.tokenizer import StringToken, Token, Tokenizer
from ...foundation.types import Version
from ...utils import native


class BasicTokenizer(Tokenizer):
    def tokenize(self, input: str) -> Iterator[Token]:
        return iter([StringToken.new(w) for w in native.module().split_whitespace(input)])

    def decode(self, tokens: Iterable[Token]) -> str:
        return " ".join(t.as_str() or "" for t in tokens)

    def vocab_size(self) -> int:
        return 0

    def name(self) -> str:
        return "basic"


class BasicTokenizerPlugin(TokenizerPlugin):
    def id(self) -> str:
        return "basic_tokenizer"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        return PluginCapabilities.standard().with_feature("tokenization").with_feature("whitespace")

    def create_tokenizer(self) -> BasicTokenizer:
        return BasicTokenizer()
