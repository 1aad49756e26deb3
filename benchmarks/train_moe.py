#!/usr/bin/env python
"""Expert-parallel training throughput of the MoE decoder (hidden 2048, 16 layers, 16 heads,
8 experts top-2, expert SwiGLU FFN 5632, capacity factor 1.25, RoPE, RMSNorm, vocab 32000), bf16,
global batch 16 x 2048 split over the ranks, EP = world size.

    python -m torch.distributed.run --nproc-per-node 8 benchmarks/train_moe.py --backend fused
    python -m torch.distributed.run --nproc-per-node 8 benchmarks/train_moe.py --backend nccl

``fused`` exchanges the tokens inside the expert GEMMs over NVLink peer memory, ``nccl`` wraps
plain GEMMs in ``all_to_all_single`` (the baseline).  Timed with CUDA events on every rank,
maximum over ranks; synthetic token ids, random-init weights."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--batch", type=int, default=16, help="global batch (sequences)")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.ep import ExpertParallel, ExpertParallelTrainer
    cfg = DecoderConfig.moe_8x(max_seq_len=a.seq)
    cfg.num_layers = a.layers
    if a.batch % world:
        raise SystemExit("global batch must be divisible by the number of ranks")
    epx = ExpertParallel(dist.group.WORLD, dev, backend=a.backend if world > 1 else "nccl")
    model = DecoderLM(cfg, dev, epx=epx)
    trainer = ExpertParallelTrainer(model)
    gen = torch.Generator().manual_seed(5 + rank)
    b = a.batch // world
    batch = torch.randint(0, cfg.vocab_size, (b, a.seq + 1), generator=gen).to(dev)
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    for _ in range(a.warmup):
        loss = trainer.train_step(x, y)
    dist.barrier()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = trainer.train_step(x, y)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"bench": "train_moe_8x", "backend": a.backend, "ep": world,
                          "layers": a.layers, "global_batch": [a.batch, a.seq],
                          "ms_per_step": round(ms.item(), 3),
                          "tokens_per_s": round(a.batch * a.seq / ms.item() * 1e3, 1),
                          "loss": float(loss)}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
