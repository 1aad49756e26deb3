#!/usr/bin/env python
"""Cost of the fused data-parallel step (reduce-scatter + AdamW + all-gather per bucket over
NVLink peer memory) of the Transformer-250M benchmark configuration, device-timed, maximum over
ranks:

* ``step_ms`` / ``single_ms``: a whole training step with and without data parallelism,
* ``exposed_tail_ms``: from the end of the last backward kernel to the end of the last bucket
  kernel (what the overlap with backward does not hide),
* ``buckets_alone_ms``: all bucket kernels back to back with no compute beside them, and what
  that is against the roofline: the slower of the NVLink bytes of one rank in one direction at
  the measured 770 GB/s and the HBM bytes of its shard update at the measured copy bandwidth.

    torchrun --nproc-per-node 8 benchmarks/dp_step.py [--clip 1.0]
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS, HBM_GBS = 770.0, 6550.0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--clip", type=float, default=None)
    ap.add_argument("--nvls", action="store_true",
                    help="reduce in the NVLink switch (multimem) instead of plain peer loads")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    import dataclasses
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.zero import ShardedDataParallel
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cfg = dataclasses.replace(DecoderConfig.transformer_250m(2048), num_layers=a.layers)
    batch = torch.randint(0, cfg.vocab_size, (8, 2049), device=dev)
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    out = {"ranks": world, "layers": a.layers, "grad_clip": a.clip, "nvls": a.nvls}
    # ---- one replica without data parallelism
    m0 = DecoderLM(cfg, device=dev, seed=0)
    t0 = Trainer(m0, TrainConfig(learning_rate=3e-4, grad_clip=a.clip))
    for _ in range(3):
        t0.train_step(x, y)
    out["single_ms"] = round(timed(lambda: t0.train_step(x, y), a.steps), 3)
    del t0, m0
    torch.cuda.empty_cache()
    # ---- the data-parallel step
    m = DecoderLM(cfg, device=dev, seed=0)
    dp = ShardedDataParallel(dist.group.WORLD, dev, nvls=a.nvls)
    tr = Trainer(m, TrainConfig(learning_rate=3e-4, grad_clip=a.clip), dp=dp)
    for _ in range(3):
        tr.train_step(x, y)
    out["step_ms"] = round(timed(lambda: tr.train_step(x, y), a.steps), 3)
    # exposed tail: end of backward on the main stream -> end of the bucket kernels
    tails = []
    for _ in range(a.steps):
        tr.train_step(x, y)
        eb = torch.cuda.Event(enable_timing=True)
        eb.record(torch.cuda.current_stream())          # after the last kernel of the step's compute
        ec = torch.cuda.Event(enable_timing=True)
        ec.record(dp.comm_stream)
        torch.cuda.synchronize()
        tails.append(max(0.0, eb.elapsed_time(ec)))
    t = torch.tensor([sum(tails) / len(tails)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out["exposed_tail_ms"] = round(float(t), 3)
    # ---- the bucket kernels alone
    triggers = [-1] + list(reversed(range(cfg.num_layers))) + [-2]

    def buckets_only():
        dp.set_grad_scale(1.0 / world)
        dp.begin_step()
        for trg in triggers:
            dp.on_layer_done(trg)
        dp.reduce_and_step(1.0 / world)
        torch.cuda.current_stream().wait_event(dp.done_event)
    buckets_only()
    alone = timed(buckets_only, a.steps)
    n = m.n_flat
    nvlink_bytes = (world - 1) / world * n * (4 + 2)           # fp32 gradients in, bf16 weights out
    hbm_bytes = n / world * (4 * world + 4 * 3 * 2 + 2 * world)  # read N grads, r/w p32 m v, write N bf16
    roof_ms = max(nvlink_bytes / (NVLINK_GBS * 1e6), hbm_bytes / (HBM_GBS * 1e6)) if world > 1 else \
        hbm_bytes / (HBM_GBS * 1e6)
    out.update({"buckets_alone_ms": round(alone, 3), "buckets": len(dp.buckets),
                "nvlink_mb_per_rank_per_direction": round(nvlink_bytes / 1e6, 1),
                "roofline_ms": round(roof_ms, 3), "fraction_of_roofline": round(roof_ms / alone, 3)})
    _lib.check_status(dev)
    if rank == 0:
        print(json.dumps(out))
    dp.finish()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
