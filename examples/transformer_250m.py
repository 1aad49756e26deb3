#!/usr/bin/env python
"""Build the transformer from its config through the plugin API, run a forward pass, print the
top logits, save and load a ``.rustllm`` file and generate a few tokens (counterpart of
examples/transformer_250m.rs; ``--small`` shrinks the model so it finishes in seconds on a CPU)."""
import argparse
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import (BasicGenerationConfig, PluginManager, Transformer250MConfig,
                                TransformerModel, TransformerModelPlugin)


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    cfg = Transformer250MConfig()
    if a.small:
        cfg = Transformer250MConfig(hidden_dim=64, num_layers=2, num_heads=2, intermediate_dim=128,
                                    vocab_size=320, max_seq_len=32)
    print(f"hidden {cfg.hidden_dim}, layers {cfg.num_layers}, heads {cfg.num_heads}, "
          f"vocab {cfg.vocab_size}: {cfg.buffer_parameters():,} parameters")
    t0 = time.perf_counter()
    model = TransformerModelPlugin().create_builder(device=a.device).build(cfg)
    t_build = time.perf_counter() - t0
    ids = [1, 2, 3, 4, 5]
    t0 = time.perf_counter()
    logits = model.forward(ids)
    t_fwd = time.perf_counter() - t0
    top = sorted(range(len(logits)), key=lambda i: -logits[i])[:5]
    print(f"build {t_build:.2f} s, forward {t_fwd * 1e3:.1f} ms, top-5 ids {top}")
    path = os.path.join(tempfile.mkdtemp(), "model.rustllm")
    with open(path, "wb") as f:
        model.write_to(f)
    with open(path, "rb") as f:
        back = TransformerModel.read_from(f, device=a.device)
    same = max(abs(x - y) for x, y in zip(back.forward(ids), logits)) == 0.0
    gen = model.generate(ids, BasicGenerationConfig(max_length=8, temperature=0.0))
    mgr = PluginManager.new()
    mgr.register(TransformerModelPlugin)
    mgr.load("transformer_model")
    return {"params": cfg.buffer_parameters(), "logits": len(logits), "top5": top,
            "file_bytes": os.path.getsize(path), "roundtrip_identical": same,
            "generated": list(gen), "loaded": mgr.list_loaded()}


if __name__ == "__main__":
    print(main())
