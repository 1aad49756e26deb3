#!/usr/bin/env python
"""Batched tensor-parallel inference of the 1.3B decoder (hidden 2048, 24 layers, 16 heads,
SwiGLU 5504, RoPE, RMSNorm, vocab 32000), bf16, TP = world size: 64 sequences, random prompt ids
of length 2048 (prefill), then 256 greedy decode steps over the paged KV cache.  The weights are
random-init, written once to a SafeTensors file in the reference's tensor naming and loaded from
it by every rank.

    python -m torch.distributed.run --nproc-per-node 8 benchmarks/infer_tp.py
    python -m torch.distributed.run --nproc-per-node 8 benchmarks/infer_tp.py --ar nccl --no-graph

Timed with CUDA events on every rank, maximum over ranks."""
import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--ar", default=None, choices=["nvls", "fused", "nccl"])
    ap.add_argument("--tp-backend", default=None, choices=["fused", "nccl"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--weights", default=None, help="SafeTensors file (written if absent)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29535")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.checkpoint.formats import load_model, save_model
    from coeus_b200.infer.tp_engine import TPInferenceEngine
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM
    cfg = DecoderConfig.decoder_1p3b(max_seq_len=a.prompt + a.new)
    cfg.num_layers = a.layers
    path = a.weights or os.path.join(tempfile.gettempdir(), f"coeus_1p3b_{a.layers}l.safetensors")
    if rank == 0 and not os.path.exists(path):
        save_model(DecoderLM(cfg, dev, seed=0, training=False), path, "safetensors")
        torch.cuda.empty_cache()
    dist.barrier()
    full, _ = load_model(path, dev)
    tp = TensorParallel(dist.group.WORLD, dev, backend=a.tp_backend if world > 1 else "nccl")
    model = TPDecoderLM(full.cfg, tp, dev, full=full)
    del full
    torch.cuda.empty_cache()
    eng = TPInferenceEngine(model, max_batch=a.batch, use_graph=not a.no_graph, ar_backend=a.ar)
    gen = torch.Generator().manual_seed(9)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=gen).to(dev)
    total = a.prompt + a.new
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    # warm-up: a prefill and a few decode steps (also captures the decode graph)
    nxt = eng._greedy_from_local(eng.prefill(ids, total))
    for _ in range(3):
        nxt = eng.decode_step(nxt)
    dist.barrier()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ev[0].record()
    nxt = eng._greedy_from_local(eng.prefill(ids, total))
    ev[1].record()
    for _ in range(a.new - 1):
        nxt = eng.decode_step(nxt)
    ev[2].record()
    dist.barrier()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device=dev,
                     dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        pf, dc = t[0].item(), t[1].item()
        print(json.dumps({"bench": "infer_tp_1p3b", "tp": world, "layers": a.layers,
                          "batch": a.batch, "prompt": a.prompt, "new_tokens": a.new,
                          "allreduce": eng.ar.backend, "graph": eng.use_graph,
                          "prefill_ms": round(pf, 2),
                          "prefill_tokens_per_s": round(a.batch * a.prompt / pf * 1e3, 1),
                          "decode_ms_per_step": round(dc / (a.new - 1), 4),
                          "decode_tokens_per_s": round(a.batch * (a.new - 1) / dc * 1e3, 1)}))
    eng.close()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
