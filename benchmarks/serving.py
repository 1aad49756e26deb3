"""Serving throughput: requests with random prompt lengths and budgets through the continuous
batcher against the same requests generated one at a time.

    python benchmarks/serving.py --device cuda --requests 64 --max-seqs 16

Prints one JSON line: generated tokens/s of both modes, request latency percentiles of the batcher
(a request's latency runs from submission, all at time zero, to its last token).  Random-init
weights, uniform random prompts (synthetic).  The reference has no serving path to compare with
(src/domain/inference/mod.rs:6-32 are data types only)."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--max-seqs", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--prompt-max", type=int, default=512)
    ap.add_argument("--new-max", type=int, default=64)
    ap.add_argument("--skip-sequential", action="store_true")
    ap.add_argument("--system-prompt", type=int, default=0,
                    help="tokens of a prompt prefix shared by every request")
    ap.add_argument("--prefix-cache", action="store_true",
                    help="reuse the cache pages of the shared prefix")
    a = ap.parse_args(argv)
    from coeus_b200.infer.engine import InferenceEngine
    from coeus_b200.infer.scheduler import ContinuousBatcher
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    dev = torch.device(a.device)
    cfg = DecoderConfig(hidden_dim=a.hidden, num_layers=a.layers, num_heads=a.heads,
                        intermediate_dim=4 * a.hidden, vocab_size=32000,
                        max_seq_len=a.prompt_max + a.new_max, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = DecoderLM(cfg, dev, dtype=dtype, training=False)
    g = torch.Generator().manual_seed(0)
    reqs = []
    system = torch.randint(0, cfg.vocab_size, (a.system_prompt,), generator=g).tolist()
    for _ in range(a.requests):
        n = int(torch.randint(4, max(5, a.prompt_max - a.system_prompt) + 1, (1,), generator=g))
        k = int(torch.randint(1, a.new_max + 1, (1,), generator=g))
        reqs.append((system + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), k))
    total_new = sum(k for _, k in reqs)

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)

    cb = ContinuousBatcher(InferenceEngine(model, max_batch=a.max_seqs, use_graph=False),
                           max_seqs=a.max_seqs, max_len=cfg.max_seq_len,
                           prefix_cache=a.prefix_cache)
    # warm-up: one short request end to end
    cb.submit(reqs[0][0][:8], 2)
    cb.run()
    sync()
    t0 = time.perf_counter()
    ids = {cb.submit(p, k): None for p, k in reqs}
    lat = {}
    while cb.pending():
        for r in cb.step():
            sync()
            lat[r.id] = time.perf_counter() - t0
    sync()
    t_batch = time.perf_counter() - t0
    ls = sorted(lat[i] for i in ids)
    out = {"requests": a.requests, "max_seqs": a.max_seqs, "generated_tokens": total_new,
           "batched_tokens_per_s": total_new / t_batch,
           "latency_s": {"p50": ls[len(ls) // 2], "p90": ls[int(len(ls) * 0.9)], "max": ls[-1]},
           "decode_steps": cb.stats["steps"], "device": str(dev), "data": "synthetic",
           "prefix_cache_hits": cb.prefix.hits if cb.prefix is not None else None}
    if not a.skip_sequential:
        eng = InferenceEngine(model, max_batch=1, use_graph=False)
        eng.generate(torch.tensor(reqs[0][0][:8], device=dev)[None], 2)
        sync()
        t0 = time.perf_counter()
        for p, k in reqs:
            eng.generate(torch.tensor(p, device=dev)[None], k)
        sync()
        out["sequential_tokens_per_s"] = total_new / (time.perf_counter() - t0)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
