#!/usr/bin/env python
"""Micro-benchmark of the fused compute+collective kernels against their NCCL compositions, with
the achieved fraction of the roofline of each.

    python -m torch.distributed.run --nproc-per-node 8 benchmarks/fused_collectives.py

Shapes are those of the 1.3B tensor-parallel configuration (32,768 tokens, hidden 2048, FFN 5504,
16 heads) at TP = world size.  Roofline time of an op = the slower of its FLOPs at the measured
GEMM peak and the bytes that must cross NVLink at the measured peer bandwidth (770 GB/s per
direction per GPU); ``frac`` = roofline time / measured time.  Also: latency of the one-shot
all-reduce (+residual+norm) of decode against ``all_reduce`` + separate kernels.  Times are CUDA
events per call after warm-up, maximum over ranks."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops_sustained"], "measured"
    return 1400.0, "fallback"


def timed(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29536")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.allreduce import FusedAllReduce
    from coeus_b200.parallel.tp import TensorParallel
    tf, src = peaks()
    T, H, I, tp = a.tokens, 2048, 5504, world
    Ts = T // tp
    fused = TensorParallel(dist.group.WORLD, dev, backend="fused")
    nccl = TensorParallel(dist.group.WORLD, dev, backend="nccl")
    rows = []

    def record(name, flops, link_bytes, t_f, t_n):
        roof = max(flops / (tf * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        rows.append({"op": name, "fused_ms": round(t_f, 4), "nccl_ms": round(t_n, 4),
                     "roofline_ms": round(roof, 4), "frac_of_roofline": round(roof / t_f, 3),
                     "bound": "nvlink" if link_bytes / (NVLINK_GBS * 1e9) > flops / (tf * 1e12)
                     else "compute"})

    bf = torch.bfloat16
    for name, K, N in (("ag_gemm_qkv", H, 3 * H // tp), ("ag_gemm_gate_up", H, 2 * I // tp)):
        w = (torch.randn(K, N, device=dev) * 0.02).to(bf)
        x_own = torch.randn(Ts, K, device=dev).to(bf)
        res = {}
        for tag, t in (("f", fused), ("n", nccl)):
            def call(t=t, site=name + tag):
                t.own_rows(site, T, K).copy_(x_own)
                t.ag_gemm(site, w)
            res[tag] = timed(call, a.iters, a.warmup, dev)
        record(name, 2.0 * T * N * K, (tp - 1) / tp * T * K * 2, res["f"], res["n"])
    for name, K, N in (("gemm_rs_oproj", H // tp, H), ("gemm_rs_down", I // tp, H)):
        w = (torch.randn(K, N, device=dev) * 0.02).to(bf)
        act = torch.randn(T, K, device=dev).to(bf)
        resid = torch.randn(Ts, N, device=dev).to(bf)
        res = {}
        for tag, t in (("f", fused), ("n", nccl)):
            res[tag] = timed(lambda t=t, site=name + tag: t.gemm_rs(site, act, w, resid),
                             a.iters, a.warmup, dev)
        record(name, 2.0 * T * N * K, (tp - 1) / tp * T * N * 2, res["f"], res["n"])
    # decode all-reduce: [64, 2048] bf16 partials + residual + RMSNorm
    B = 64
    scale = torch.ones(H, device=dev, dtype=bf)
    resid = torch.randn(B, H, device=dev).to(bf)
    part = torch.randn(B, H, device=dev).to(bf)
    res = {}
    for tag, backend in (("f", "fused"), ("n", "nccl")):
        ar = FusedAllReduce(dist.group.WORLD, dev, B, H, backend=backend)

        def call(ar=ar):
            ar.next_part(B).copy_(part)
            ar.reduce(B, resid, scale, None, True, 1e-6)
        res[tag] = timed(call, 50, 10, dev)
    rows.append({"op": "allreduce_resid_rmsnorm_64x2048", "fused_ms": round(res["f"], 4),
                 "nccl_ms": round(res["n"], 4),
                 "note": "latency-bound; includes the 256 KB copy into the partial buffer"})
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        print(json.dumps({"bench": "fused_collectives", "tp": tp, "tokens": T, "peaks": src,
                          "gemm_peak_tflops": tf, "nvlink_gbs": NVLINK_GBS, "rows": rows}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
