#!/usr/bin/env python
"""Latency of the decode collective (all-reduce of ``[rows, H]`` bf16 + residual + RMSNorm) per
backend: ``nvls`` (reduced in the NVLink switch, ``multimem``), ``fused`` (plain peer loads) and
``nccl`` (library all-reduce + stand-alone kernels).  Device-timed over a CUDA-graph replay of
``--calls`` back-to-back calls, maximum over ranks.

    torchrun --nproc-per-node 8 benchmarks/allreduce_latency.py --rows 64 --hidden 2048
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--calls", type=int, default=48)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--backends", default="nvls,fused,nccl")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.allreduce import FusedAllReduce
    from coeus_b200.parallel.symm import multicast_supported
    out = {"rows": a.rows, "hidden": a.hidden, "ranks": world, "calls_per_graph": a.calls}
    scale = torch.ones(a.hidden, dtype=torch.bfloat16, device=dev)
    for backend in a.backends.split(","):
        if backend == "nvls" and not multicast_supported(dev):
            out["nvls"] = "unsupported"
            continue
        ar = FusedAllReduce(dist.group.WORLD, dev, a.rows, a.hidden, backend=backend)
        x0 = torch.randn(a.rows, a.hidden, device=dev).bfloat16()

        def run():
            x = x0
            for _ in range(a.calls):
                ar.next_part(a.rows).normal_()
                x, n = ar.reduce(a.rows, x, scale, None, True, 1e-5)
            return x
        # the partial is produced by a small kernel (normal_) each call, like the GEMM before it
        run()
        torch.cuda.synchronize()
        dist.barrier()
        use_graph = backend != "nccl"
        if use_graph:
            g = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                run()
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=s):
                    run()
            fn = g.replay
        else:
            fn = run
        # the same loop without the collective, to subtract the producer kernels
        def base():
            for _ in range(a.calls):
                ar.next_part(a.rows).normal_()
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        _lib.check_status(dev)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(a.iters):
            base()
        b1.record()
        torch.cuda.synchronize()
        out[backend] = {"us_per_call_incl_producer": round(float(t) * 1e3 / (a.iters * a.calls), 2),
                        "producer_us": round(b0.elapsed_time(b1) * 1e3 / (a.iters * a.calls), 2),
                        "graph": use_graph}
        dist.barrier()
        ar.close() if hasattr(ar, "close") else None
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
