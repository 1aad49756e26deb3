"""Serve completions over HTTP with continuous batching.

    python examples/serve_completions.py --port 8000
    curl -s localhost:8000/v1/completions -d '{"prompt": "the cat", "max_tokens": 8}' \
         -H 'content-type: application/json'

Uses a randomly initialised small model and a BPE tokenizer trained on a toy corpus (there are no
pretrained weights here); pass ``--weights file.safetensors`` to load a checkpoint written by
``model.save``.  The reference stops at the ``InferenceService`` data types
(src/domain/inference/mod.rs:6-32)."""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build(device: str, weights: str | None):
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.prelude import BpeTokenizerPlugin
    tok = BpeTokenizerPlugin().create_tokenizer()
    tok.train(["the cat sat on the mat", "the dog sat on the log", "a cat and a dog"], 50)
    cfg = DecoderConfig(hidden_dim=256, num_layers=4, num_heads=4, intermediate_dim=1024,
                        vocab_size=max(512, tok.vocab_size()), max_seq_len=1024, use_bias=False,
                        activation="swiglu", norm="rmsnorm", pos="rope")
    if weights:
        from coeus_b200.checkpoint.formats import load_model
        return load_model(weights, device=device)[0], tok
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    return DecoderLM(cfg, device, dtype=dtype, training=False), tok


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-seqs", type=int, default=16)
    ap.add_argument("--weights", default=None)
    ap.add_argument("--dry-run", action="store_true", help="build the app, answer one request "
                    "in-process, exit")
    a = ap.parse_args(argv)
    from coeus_b200.serve import create_app
    model, tok = build(a.device, a.weights)
    app = create_app(model, tokenizer=tok, max_seqs=a.max_seqs, max_len=model.cfg.max_seq_len)
    if a.dry_run:
        from fastapi.testclient import TestClient
        with TestClient(app) as c:
            r = c.post("/v1/completions", json={"prompt": "the cat", "max_tokens": 4})
            print(r.status_code, r.json())
        return 0 if r.status_code == 200 else 1
    import uvicorn
    uvicorn.run(app, host=a.host, port=a.port, log_level="info")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
