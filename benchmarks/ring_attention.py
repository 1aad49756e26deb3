#!/usr/bin/env python
"""Context-parallel (ring) attention, forward + backward, against the single-GPU flash kernels on
the same amount of work.

One sequence of ``--seq`` tokens (default 32768) per batch element is split over the ranks
(zig-zag chunks, ``coeus_b200/parallel/cp.py``); every rank times the forward and backward ring
attention of its share: 16 heads x 64 by default, bf16, causal.  The comparator is what ONE GPU
needs for 1 / world of the whole causal attention without any exchange: the flash kernels on a
sequence of ``seq / sqrt(world)`` tokens (a causal problem with 1 / world of the score elements).

    python -m torch.distributed.run --nproc-per-node 8 benchmarks/ring_attention.py
    python -m torch.distributed.run --nproc-per-node 8 benchmarks/ring_attention.py --backend collective

Timed with CUDA events on every rank, maximum over ranks."""
import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dh", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--backend", default=None, choices=["p2p", "collective"])
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29545")
    if cuda:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.ops import _lib
    from coeus_b200.ops import attention as A
    from coeus_b200.parallel.cp import ContextParallel

    B, nh, dh, S = a.batch, a.heads, a.dh, a.seq
    H = nh * dh
    Sc = S // (2 * world)
    if Sc * 2 * world != S or Sc % 128:
        raise SystemExit("--seq must be a multiple of 256 * world size")
    dtype = torch.bfloat16 if cuda else torch.float32
    cp = ContextParallel(dist.group.WORLD, dev, backend=a.backend)
    gen = torch.Generator().manual_seed(17 + rank)
    qkv = torch.randn(2 * B * Sc, 3 * H, generator=gen).to(dtype).to(dev)
    do = torch.randn(2 * B * Sc, H, generator=gen).to(dtype).to(dev)

    def sync():
        dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        sync()
        if not cuda:
            import time
            t0 = time.perf_counter()
            for _ in range(a.iters):
                fn()
            return (time.perf_counter() - t0) * 1e3 / a.iters
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        sync()
        return e0.elapsed_time(e1) / a.iters

    o, lse = cp.attention_fwd(qkv, B, Sc, nh, dh)
    t_fwd = timed(lambda: cp.attention_fwd(qkv, B, Sc, nh, dh))
    t_bwd = timed(lambda: cp.attention_bwd(do, qkv, o, lse, B, Sc, nh, dh))
    if cuda:
        _lib.check_status(dev)

    # comparator: one GPU, no exchange, 1 / world of the causal score elements
    S1 = max(128, int(round(S / math.sqrt(world) / 128)) * 128)
    x = torch.randn(B * S1, 3 * H, generator=gen).to(dtype).to(dev)
    d1 = torch.randn(B * S1, H, generator=gen).to(dtype).to(dev)
    q, k, v = x[:, :H], x[:, H:2 * H], x[:, 2 * H:]
    o1, l1 = A.attention_fwd(q, k, v, B, S1, nh, dh)
    s_fwd = timed(lambda: A.attention_fwd(q, k, v, B, S1, nh, dh))
    s_bwd = timed(lambda: A.attention_bwd(d1, q, k, v, o1, l1, B, S1, nh, dh))

    t = torch.tensor([t_fwd, t_bwd, s_fwd, s_bwd], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        f, b, sf, sb = t.tolist()
        flops_fwd = 4.0 * B * nh * dh * S * S / 2 / world      # per rank, causal half
        scale = (S1 * S1) / (S * S / world)                     # comparator's share of that work
        print(json.dumps({
            "bench": "ring_attention", "cp": world, "backend": cp.backend, "seq": S, "batch": B,
            "heads": nh, "dh": dh, "chunk": Sc,
            "ring_fwd_ms": round(f, 3), "ring_bwd_ms": round(b, 3),
            "ring_fwd_tflops_per_gpu": round(flops_fwd / f / 1e9, 1),
            "ring_bwd_tflops_per_gpu": round(2.5 * flops_fwd / b / 1e9, 1),
            "single_gpu_seq": S1, "single_fwd_ms": round(sf, 3), "single_bwd_ms": round(sb, 3),
            "ring_over_single_fwd": round(f / (sf / scale), 3),
            "ring_over_single_bwd": round(b / (sb / scale), 3)}))
    sync()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
