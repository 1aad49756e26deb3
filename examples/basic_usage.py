#!/usr/bin/env python
"""Register the built-in plugins, tokenize and decode, slide windows over tokens, run the basic
model, and use the memory utilities (counterpart of the reference's examples/basic_usage.rs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import (Arena, BasicModelConfig, BasicModelPlugin, BasicTokenizerPlugin,
                                BpeTokenizerPlugin, CowStr, Iter, PluginManager,
                                ZeroCopyStringBuilder)


def main() -> dict:
    mgr = PluginManager.new()
    for plugin in (BasicTokenizerPlugin, BpeTokenizerPlugin, BasicModelPlugin):
        mgr.register(plugin)
    mgr.load("basic_tokenizer")
    tok = BasicTokenizerPlugin().create_tokenizer()
    text = "Hello, RustLLM Core! This is a simple example."
    tokens = list(tok.tokenize_str(text))
    decoded = tok.decode(tokens)
    print(f"{len(tokens)} tokens -> '{decoded}'")
    trigrams = Iter([t.as_str() for t in tokens]).windows(3).collect()
    print("first trigram:", trigrams[0])
    model = BasicModelPlugin().create_builder().build(BasicModelConfig())
    out = model.forward([1.0, 2.0, 3.0])
    print("basic model output:", out)
    arena = Arena.new(1024)
    arena.alloc(42)
    cow = CowStr.borrowed("hello")
    cow.push_str(" world")
    built = ZeroCopyStringBuilder.new().append_borrowed("zero").append_owned("-copy").build()
    return {"tokens": len(tokens), "decoded": decoded, "trigrams": len(trigrams), "out": out,
            "arena_used": arena.used(), "cow": cow.as_str(), "built": built,
            "loaded": mgr.list_loaded()}


if __name__ == "__main__":
    main()
