#!/usr/bin/env python
"""Stream a text file line by line through a tokenizer with a tokens/s readout, sliding windows
over the stream, chunked BPE over many sentences and a frequency count (counterpart of
examples/streaming.rs)."""
import os
import sys
import tempfile
import time
from collections import Counter

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import BasicTokenizerPlugin, BpeTokenizerPlugin, Iter


def main(lines: int = 10_000, sentences: int = 100) -> dict:
    path = os.path.join(tempfile.mkdtemp(), "stream.txt")
    with open(path, "w") as f:
        for i in range(lines):
            f.write(f"line {i} of the streaming example with some repeated words words\n")
    tok = BasicTokenizerPlugin().create_tokenizer()
    t0 = time.perf_counter()
    total = 0
    with open(path) as f:
        for line in f:
            total += sum(1 for _ in tok.tokenize_str(line))
    dt = time.perf_counter() - t0
    print(f"{total} tokens in {dt:.3f} s = {total / dt:,.0f} tokens/s")
    words = [t.as_str() for t in tok.tokenize_str("the quick brown fox jumps over the lazy dog")]
    w3 = Iter(words).windows(3).collect()
    w5 = Iter(words).windows(5).collect()
    bpe = BpeTokenizerPlugin().create_tokenizer()
    corpus = [f"sentence number {i} talks about tokens and merges" for i in range(sentences)]
    bpe.train(corpus, 50)
    chunk_tokens = 0
    for chunk in Iter(corpus).chunks(10):
        chunk_tokens += sum(len(list(bpe.tokenize_str(s))) for s in chunk)
    freq = Counter(t.as_str() for s in corpus[:10] for t in tok.tokenize_str(s))
    return {"stream_tokens": total, "tokens_per_s": total / dt, "windows3": len(w3),
            "windows5": len(w5), "bpe_tokens": chunk_tokens, "top": freq.most_common(3)}


if __name__ == "__main__":
    print(main())
