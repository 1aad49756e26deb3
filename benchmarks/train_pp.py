#!/usr/bin/env python
"""Pipeline-parallel training throughput, PP = world size: the 1F1B schedule over NCCL
point-to-point, the same schedule over NVLink peer memory, and the interleaved schedule (several
chunks of blocks per rank, peer memory), on one model and one global batch.

    python -m torch.distributed.run --nproc-per-node 4 benchmarks/train_pp.py

The default model is a decoder of hidden size 2048, 16 layers, 16 heads, FFN 8192 (GELU, biases,
LayerNorm, sinusoidal positions, vocab 32000, about 0.94 B parameters), bf16, 8 micro-batches of
2 x 2048 tokens.  With P stages and M micro-batches the idle share of the 1F1B schedule is
(P - 1) / (M + P - 1); with v chunks per rank it is (P - 1) / (v M + P - 1).  Timed with CUDA
events on every rank, maximum over ranks; synthetic token ids, random-init weights."""
import argparse
import gc
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--chunks", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--modes", default="nccl,peer,interleaved")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29537")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.pp import InterleavedPipelineStage, PipelineStage
    cfg = DecoderConfig(hidden_dim=a.hidden, num_layers=a.layers, num_heads=a.heads,
                        intermediate_dim=a.ffn, vocab_size=32000, max_seq_len=a.seq)
    M, b, S = a.micro_batches, a.micro_batch, a.seq
    gen = torch.Generator().manual_seed(11)
    batch = torch.randint(0, cfg.vocab_size, (M, b, S + 1), generator=gen).to(dev)
    ids, tgt = batch[:, :, :-1].contiguous(), batch[:, :, 1:].contiguous()
    results = {}
    for mode in a.modes.split(","):
        if mode == "interleaved":
            if world < 2 or a.layers % (world * a.chunks):
                continue
            st = InterleavedPipelineStage(cfg, dist.group.WORLD, dev, micro_batches=M,
                                          chunks=a.chunks, seed=3)
        else:
            st = PipelineStage(cfg, dist.group.WORLD, dev, micro_batches=M, seed=3,
                               transport=mode if world > 1 else "nccl")
        for _ in range(a.warmup):
            loss = st.train_step(ids, tgt)
        dist.barrier()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            loss = st.train_step(ids, tgt)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        t = torch.tensor([e0.elapsed_time(e1) / a.steps, float(loss)], device=dev,
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[mode] = {"ms_per_step": round(t[0].item(), 3),
                         "tokens_per_s": round(M * b * S / t[0].item() * 1e3, 1),
                         "loss": round(t[1].item(), 4)}
        ring = getattr(st, "_ring", None)
        if ring is not None:
            ring.close()        # after the barrier above: nobody pushes into it any more
        del st, ring
        gc.collect()
        torch.cuda.empty_cache()
    if rank == 0:
        P = world
        print(json.dumps({
            "bench": "train_pp", "pp": P, "micro_batches": M, "micro_batch": [b, S],
            "model": {"hidden": a.hidden, "layers": a.layers, "heads": a.heads, "ffn": a.ffn},
            "idle_share_1f1b": round((P - 1) / (M + P - 1), 3),
            "idle_share_interleaved": round((P - 1) / (a.chunks * M + P - 1), 3),
            "chunks": a.chunks, **results}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
