#!/usr/bin/env python
"""CPU baselines of the smallest configuration.

(a) Transformer-250M preset (vocab 32000, hidden 1024, 16 layers, 16 heads, FFN 4096, context 512),
    weights N(0, 0.02) seed 0, fp32, batch 4 x 512, token ids uniform in [0, vocab):
    * ``oracle``: the C++ restatement of the reference's own forward loops (64^3-blocked scalar
      matmul, S x S attention per head, one thread) -- the reference has no batching, backward or
      optimizer, so this arm is four sequential forward calls and is run on ``--oracle-seq`` tokens
      (default 64; the full 512 takes minutes) with the time scaled per token;
    * ``torch-cpu``: forward + backward + AdamW of the same model through this framework's CPU
      path (PyTorch fp32 ops, all cores).
(b) BPE tokenize + decode of 1 MB of seeded random ASCII words with the native tokenizer after
    training 200 merges on the first 64 KB.

    python benchmarks/cpu_baseline.py [--skip-oracle] [--steps 2]
"""
import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch


def bench_bpe(mb: float = 1.0):
    from coeus_b200.plugins.builtin import BpeTokenizer
    rng = random.Random(0)
    words, n = [], 0
    target = int(mb * (1 << 20))
    while n < target:
        w = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(1, 10)))
        words.append(w)
        n += len(w) + 1
    text = " ".join(words)[:target]
    tok = BpeTokenizer()
    t0 = time.perf_counter()
    tok.train([text[:65536]], 200)
    t_train = time.perf_counter() - t0
    t0 = time.perf_counter()
    ids = tok.encode(text)
    t_enc = time.perf_counter() - t0
    t0 = time.perf_counter()
    back = tok.decode_ids(ids)
    t_dec = time.perf_counter() - t0
    return {"bytes": len(text), "tokens": len(ids), "train_200_merges_s": round(t_train, 3),
            "encode_mb_per_s": round(len(text) / t_enc / 1e6, 2),
            "encode_tokens_per_s": round(len(ids) / t_enc, 0),
            "decode_mb_per_s": round(len(text) / t_dec / 1e6, 2),
            "roundtrip_exact": back == text}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--skip-oracle", action="store_true")
    ap.add_argument("--oracle-seq", type=int, default=64)
    ap.add_argument("--layers", type=int, default=16)
    a = ap.parse_args()
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = DecoderConfig.transformer_250m(max_seq_len=512)
    cfg.num_layers = a.layers
    out = {"config": {"model": "Transformer-250M preset", "layers": a.layers, "batch": [4, 512],
                      "dtype": "fp32", "threads": torch.get_num_threads()}}
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (4, 513), generator=gen)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    model = DecoderLM(cfg, "cpu", seed=0, dtype=torch.float32)
    tr = Trainer(model, TrainConfig(learning_rate=3e-4))
    tr.train_step(x, y)                                   # warm-up
    t0 = time.perf_counter()
    for _ in range(a.steps):
        loss = tr.train_step(x, y)
    dt = (time.perf_counter() - t0) / a.steps
    out["torch_cpu_train"] = {"s_per_step": round(dt, 3), "tokens_per_s": round(4 * 512 / dt, 1),
                              "loss": float(loss)}
    t0 = time.perf_counter()
    model.forward_logits(x, last_only=True)
    dt = time.perf_counter() - t0
    out["torch_cpu_forward"] = {"s": round(dt, 3), "tokens_per_s": round(4 * 512 / dt, 1)}
    if not a.skip_oracle:
        from coeus_b200.checkpoint.formats import named_from_model, to_reference_flat
        from coeus_b200.utils import native
        flat = to_reference_flat(named_from_model(model), cfg).numpy()
        S = a.oracle_seq
        t0 = time.perf_counter()
        native.module().oracle_forward(flat, cfg.hidden_dim, cfg.num_layers, cfg.num_heads,
                                       cfg.intermediate_dim, cfg.vocab_size, cfg.max_seq_len,
                                       cfg.norm_eps, cfg.use_bias, np.asarray(x[0, :S]), False, False)
        dt = time.perf_counter() - t0
        out["reference_loops_forward"] = {"seq": S, "s": round(dt, 3),
                                          "tokens_per_s": round(S / dt, 2),
                                          "note": "one sequence, one thread, forward only"}
    out["bpe_1mb"] = bench_bpe(1.0)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
