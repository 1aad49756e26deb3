#!/usr/bin/env python
"""WordPiece tokenization with a small vocabulary and a chars/s micro-benchmark (counterpart of
examples/wordpiece_tokenizer.rs)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import WordPieceTokenizerPlugin


def main(iterations: int = 100) -> dict:
    tok = WordPieceTokenizerPlugin().create_tokenizer()
    pieces = ("un", "##aff", "##able", "play", "##ing", "##ed", "the", "quick", "brown", "fox")
    for i, piece in enumerate(pieces):
        tok.add_token(piece, tok.vocab_size() + i)
    samples = ["unaffable", "playing played", "the quick brown fox", "xylophone"]
    shown = {s: [t.as_str() for t in tok.tokenize_str(s)] for s in samples}
    for s, pieces in shown.items():
        print(f"{s!r} -> {pieces}")
    text = " ".join(samples) * 20
    t0 = time.perf_counter()
    n = 0
    for _ in range(iterations):
        n += sum(1 for _ in tok.tokenize_str(text))
    dt = time.perf_counter() - t0
    print(f"{iterations * len(text) / dt:,.0f} chars/s")
    return {"pieces": shown, "chars_per_s": iterations * len(text) / dt, "tokens": n}


if __name__ == "__main__":
    main()
