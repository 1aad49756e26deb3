#!/usr/bin/env python
"""Tokenizer micro-benchmarks with the workloads of the reference's criterion harnesses
(benches/tokenizer_bench.rs: basic/BPE tokenize of four short texts and a 445-byte Lorem ipsum,
decode, BPE training with 10/50/100 merges on six sentences, vocabulary operations;
plugins/tokenizer-wordpiece/benches/wordpiece_bench.rs: encode/decode of short, medium and long
texts plus vocabulary lookups).  Prints one JSON object of nanoseconds per operation."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import (BasicTokenizerPlugin, BpeTokenizerPlugin,
                                WordPieceTokenizerPlugin)

TEXTS = ["Hello, world!", "The quick brown fox jumps over the lazy dog.",
         "Rust is a systems programming language.", "Tokenization is the first step in NLP."]
LOREM = ("Lorem ipsum dolor sit amet, consectetur adipiscing elit, sed do eiusmod tempor incididunt "
         "ut labore et dolore magna aliqua. Ut enim ad minim veniam, quis nostrud exercitation "
         "ullamco laboris nisi ut aliquip ex ea commodo consequat. Duis aute irure dolor in "
         "reprehenderit in voluptate velit esse cillum dolore eu fugiat nulla pariatur. Excepteur "
         "sint occaecat cupidatat non proident, sunt in culpa qui officia deserunt mollit anim id est.")
SENTENCES = ["the cat sat on the mat", "the dog sat on the log", "the cat and the dog",
             "a quick brown fox", "jumps over the lazy dog", "tokenizers split text into pieces"]


def ns_per_op(fn, min_time: float = 0.05) -> float:
    fn()
    n, t = 0, 0.0
    t0 = time.perf_counter()
    while t < min_time:
        fn()
        n += 1
        t = time.perf_counter() - t0
    return t / n * 1e9


def main() -> dict:
    out = {}
    basic = BasicTokenizerPlugin().create_tokenizer()
    bpe = BpeTokenizerPlugin().create_tokenizer()
    for name, tok in (("basic", basic), ("bpe", bpe)):
        for i, text in enumerate(TEXTS + [LOREM]):
            label = f"{name}/tokenize/{'lorem' if i == 4 else i}"
            out[label] = ns_per_op(lambda: list(tok.tokenize_str(text)))
        toks = list(tok.tokenize_str(LOREM))
        out[f"{name}/decode/lorem"] = ns_per_op(lambda: tok.decode(toks))
    for merges in (10, 50, 100):
        def train():
            t = BpeTokenizerPlugin().create_tokenizer()
            t.train(SENTENCES, merges)
        out[f"bpe/train/{merges}"] = ns_per_op(train, 0.1)
    out["bpe/vocab/contains"] = ns_per_op(lambda: bpe.contains_token("a"))
    out["bpe/vocab/id_from_token"] = ns_per_op(lambda: bpe.id_from_token("<UNK>"))
    out["bpe/vocab/token_from_id"] = ns_per_op(lambda: bpe.token_from_id(97))
    wp = WordPieceTokenizerPlugin().create_tokenizer()
    for i, piece in enumerate(("the", "quick", "brown", "fox", "jump", "##s", "over", "lazy", "dog",
                               "token", "##ization", "##ize", "##r")):
        wp.add_token(piece, wp.vocab_size() + i)
    for label, text in (("short", "the quick brown fox"), ("medium", " ".join(TEXTS)),
                        ("long", LOREM * 4)):
        out[f"wordpiece/encode/{label}"] = ns_per_op(lambda: wp.encode(text))
        toks = list(wp.tokenize_str(text))
        out[f"wordpiece/decode/{label}"] = ns_per_op(lambda: wp.decode(toks))
    out["wordpiece/vocab/token_to_id"] = ns_per_op(lambda: wp.token_to_id("fox"))
    out = {k: round(v, 1) for k, v in out.items()}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
