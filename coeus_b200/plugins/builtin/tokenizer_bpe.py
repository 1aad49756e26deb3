"""Byte-level BPE tokenizer (plugins/tokenizer-bpe/src/lib.rs) over the native implementation in
``csrc/host/tokenizers.cpp``.

Observable behaviour of the reference is kept: 256 byte tokens (bytes >= 0x80 spelled
``<0xNN>``) with ``<PAD> <UNK> <BOS> <EOS>`` overlaid on ids 0..3 (``vocab_size() == 260`` before
training), whitespace runs collapsed to one space token (id 32), merges applied in learned
order, unknown strings mapped to id 1, and ``decode`` turning every byte >= 0x80 into U+FFFD.
Differences: ties between equally frequent pairs during training are broken deterministically
(smallest pair of token strings) where the reference depends on hash-map iteration order, and
``encode`` / ``encode_batch`` / ``decode_ids`` work on ids without building token objects."""
from __future__ import annotations

from typing import Iterable, Iterator, List, Optional, Sequence

import numpy as np

from ...core.plugin import PluginCapabilities, TokenizerPlugin
from ...core.tokenizer import SpecialTokenizer, StringToken, Token, VocabularyTokenizer
from ...foundation.error import ProcessingError
from ...foundation.types import Version
from ...utils import native


class BpeTokenizer(VocabularyTokenizer, SpecialTokenizer):
    def __init__(self) -> None:
        self._t = native.module().BpeTokenizer()

    new = classmethod(lambda cls: cls())

    def train(self, corpus: Sequence[str], num_merges: int) -> None:
        self._t.train(list(corpus), int(num_merges))

    def tokenize(self, input: str) -> Iterator[Token]:
        ids, strs = self._t.encode_with_strings(input)
        return iter([StringToken.with_id(s, int(i)) for s, i in zip(strs, ids)])

    def decode(self, tokens: Iterable[Token]) -> str:
        return self._t.decode_strings([t.as_str() or "" for t in tokens])

    def vocab_size(self) -> int:
        return self._t.vocab_size()

    def name(self) -> str:
        return "bpe_tokenizer"

    # ---- id-level fast path
    def encode(self, text: str) -> np.ndarray:
        return self._t.encode(text)

    def encode_batch(self, texts: Sequence[str], as_tensor: bool = False):
        rows = self._t.encode_batch(list(texts))
        if not as_tensor:
            return rows
        import torch
        n = max((len(r) for r in rows), default=0)
        out = torch.zeros((len(rows), n), dtype=torch.int32)
        for i, r in enumerate(rows):
            out[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        return out

    def decode_ids(self, ids, ref_compat: bool = True) -> str:
        """``ref_compat=True`` is the reference's decoding: a byte token above 0x7F becomes
        U+FFFD on its own (``String::from_utf8_lossy`` of one byte,
        plugins/tokenizer-bpe/src/lib.rs:319-342), so characters whose bytes were never merged
        do not survive, and ids 0..3 print as ``<PAD>`` .. ``<EOS>``.  ``ref_compat=False`` joins
        the bytes first (ids 0..3 as the control bytes they also are) and decodes once: any text
        round-trips."""
        ids = [int(i) for i in ids]
        if ref_compat:
            return self._t.decode_ids(ids)
        return self._t.decode_ids_bytes(ids).decode("utf-8", errors="replace")

    # ---- VocabularyTokenizer
    def add_token(self, token: str) -> int:
        return self._t.add_token(token)

    def remove_token(self, token: str) -> None:
        if not self._t.remove_token(token):
            raise ProcessingError.invalid_input(f"Token not found: {token}")

    def contains_token(self, token: str) -> bool:
        return self._t.contains_token(token)

    def token_from_id(self, id: int) -> Optional[str]:
        return self._t.token_from_id(int(id))

    def id_from_token(self, token: str) -> Optional[int]:
        return self._t.id_from_token(token)

    def merges(self) -> List[tuple]:
        return [self._t.merge_at(i) for i in range(self._t.num_merges())]

    # ---- persistence (the reference's tokenizer lives and dies with its process)
    def save(self, path: str) -> None:
        """The learned merges, in order, as JSON (token bytes in hex): enough to rebuild the
        tokenizer with the same ids."""
        import json
        pairs = [self._t.merge_at_bytes(i) for i in range(self._t.num_merges())]
        with open(path, "w", encoding="utf-8") as f:
            json.dump({"type": "bpe_tokenizer", "version": 1,
                       "merges": [[a.hex(), b.hex()] for a, b in pairs]}, f)

    @classmethod
    def load(cls, path: str) -> "BpeTokenizer":
        import json
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
        if d.get("type") != "bpe_tokenizer":
            raise ProcessingError.invalid_input(f"{path} is not a saved BPE tokenizer")
        t = cls()
        t._t.load_merges([(bytes.fromhex(a), bytes.fromhex(b)) for a, b in d["merges"]])
        return t

    # ---- SpecialTokenizer
    def pad_token(self) -> Token:
        return StringToken.with_id("<PAD>", 0)

    def unk_token(self) -> Token:
        return StringToken.with_id("<UNK>", 1)

    def bos_token(self) -> Token:
        return StringToken.with_id("<BOS>", 2)

    def eos_token(self) -> Token:
        return StringToken.with_id("<EOS>", 3)


class BpeTokenizerPlugin(TokenizerPlugin):
    def id(self) -> str:
        return "bpe_tokenizer"

    def version(self) -> Version:
        return Version(0, 1, 0)

    def capabilities(self) -> PluginCapabilities:
        return PluginCapabilities.standard().with_feature("tokenization").with_feature("bpe")

    def create_tokenizer(self) -> BpeTokenizer:
        return BpeTokenizer()
