"""Train the same small decoder under any parallelism strategy with one call.

    python examples/parallel_training.py                                   # one process
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/parallel_training.py --strategy tp                        # 2 ranks (CPU: Gloo)

``--strategy`` is one of dp, dp0 (replicated optimizer state), tp, pp, pp_interleaved, ep, cp,
ulysses, dp_tp and dp_pp (replicas of a two-rank tensor-parallel model / pipeline, four ranks or
more); the group size comes from the launcher.  Every rank is handed the same global batch and
``ParallelRun.step`` gives it the part its strategy needs.  The reference has no parallel training
(its training example is a toy regression, examples/training_example.rs)."""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--strategy", default="dp")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from coeus_b200.core.config import ParallelConfig
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.optim.lr import WarmupCosine
    from coeus_b200.train.launch import build_trainer
    from coeus_b200.train.trainer import TrainConfig
    world = int(os.environ.get("WORLD_SIZE", "1"))
    device = a.device
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if device.startswith("cuda"):
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            device = f"cuda:{local}"
            dist.init_process_group("nccl", device_id=torch.device(device))
        else:
            dist.init_process_group("gloo")
    moe = a.strategy == "ep"
    cfg = DecoderConfig(hidden_dim=128, num_layers=4, num_heads=2, intermediate_dim=256,
                        vocab_size=512, max_seq_len=64, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope",
                        **(dict(num_experts=4, top_k=2, capacity_factor=2.0) if moe else {}))
    par = {"dp": ParallelConfig(dp=world), "dp0": ParallelConfig(dp=world, zero_stage=0),
           "tp": ParallelConfig(tp=world), "pp": ParallelConfig(pp=world),
           "pp_interleaved": ParallelConfig(pp=world, pp_chunks=2),
           "ep": ParallelConfig(dp=world, ep=world), "cp": ParallelConfig(cp=world),
           "ulysses": ParallelConfig(cp=world, ulysses=True),
           "dp_tp": ParallelConfig(dp=world // 2, tp=2),        # four ranks or more
           "dp_pp": ParallelConfig(dp=world // 2, pp=2)}[a.strategy] if world > 1 \
        else ParallelConfig()
    run = build_trainer(cfg, par, device, TrainConfig(learning_rate=3e-3, grad_clip=1.0),
                        micro_batches=2, dtype=torch.bfloat16 if device.startswith("cuda")
                        else torch.float32,
                        schedule=WarmupCosine(3e-3, 2, a.steps, floor=3e-4))
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (4, 64), generator=g).to(device)
    tgt = torch.roll(ids, -1, 1)
    losses = [float(run.step(ids, tgt)) for _ in range(a.steps)]
    out = {"strategy": run.strategy, "world": world, "first": losses[0], "last": losses[-1]}
    if run.rank == world - 1:
        print(out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
