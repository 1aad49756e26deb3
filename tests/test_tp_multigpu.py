"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels over NVLink peer memory against the
NCCL-composed reference (all_gather + GEMM, GEMM + reduce_scatter)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.tp import TensorParallel
    fused = TensorParallel(dist.group.WORLD, dev, backend="fused")
    ref = TensorParallel(dist.group.WORLD, dev, backend="nccl")
    T, K, N = 512 * world, 256, 384
    Ts = T // world
    res = {}
    for it in range(3):   # repeated use exercises the epoch / reuse protocol
        torch.manual_seed(100 * it + rank)
        x_own = torch.randn(Ts, K, device=dev).bfloat16()
        torch.manual_seed(7)
        w = (torch.randn(K, N, device=dev) * 0.05).bfloat16()
        bias = torch.randn(N, device=dev).bfloat16()
        for tp, tag in ((fused, "f"), (ref, "r")):
            tp.own_rows("qkv", T, K).copy_(x_own)
            y, xg = tp.ag_gemm("qkv", w, bias)
            res[f"ag_{tag}{it}"] = y.float().cpu()
            res[f"xg_{tag}{it}"] = xg.float().cpu().clone()
        # row-parallel: every rank holds a different slice of the contraction dimension
        torch.manual_seed(200 * it + rank)
        a = torch.randn(T, K, device=dev).bfloat16()
        w2 = (torch.randn(K, N, device=dev) * 0.05).bfloat16()
        resid = torch.randn(Ts, N, device=dev).bfloat16()
        for tp, tag in ((fused, "f"), (ref, "r")):
            o = tp.gemm_rs("oproj", a, w2, resid)
            res[f"rs_{tag}{it}"] = o.float().cpu()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        out.put(res)
    dist.barrier()
    dist.destroy_process_group()


def test_fused_tp_kernels_match_nccl():
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else (4 if n >= 4 else 2)     # the largest power of two the box offers
    from mp_util import run_ranks
    res = run_ranks(_worker, world, ())[0]
    for it in range(3):
        assert torch.equal(res[f"xg_f{it}"], res[f"xg_r{it}"])          # the gather is bitwise
        assert torch.equal(res[f"ag_f{it}"], res[f"ag_r{it}"])          # same GEMM on same data
        d = (res[f"rs_f{it}"] - res[f"rs_r{it}"]).abs().max().item()
        assert d < 0.06 * res[f"rs_r{it}"].abs().max().item() + 0.05, d   # bf16 partial sums


def _model_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.tp import TensorParallel
    from coeus_b200.parallel.tp_model import TPDecoderLM, TPTrainer
    cfg = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=512,
                        vocab_size=2000, max_seq_len=256, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    full = DecoderLM(cfg, device=dev, seed=0)
    gen = torch.Generator().manual_seed(3)
    batch = torch.randint(0, cfg.vocab_size, (2, 257), generator=gen).to(dev)
    x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
    full.zero_grad()
    ref_loss = float(full.forward_loss(x, y))
    full.backward()
    res = {"ref": ref_loss}
    for backend in ("fused", "nccl"):
        tp = TensorParallel(dist.group.WORLD, dev, backend=backend)
        m = TPDecoderLM(cfg, tp, dev, full=full)
        m.zero_grad()
        res[backend] = float(m.forward_loss(x, y))
        m.backward()
        Hl = cfg.hidden_dim // world
        want = full.g["layers.0.attn.o_weights"][rank * Hl:(rank + 1) * Hl]
        got = m.g["layers.0.attn.o_weights"]
        res[backend + "_gerr"] = ((got - want).abs().max() / (want.abs().max() + 1e-9)).item()
        res[backend + "_embed"] = ((m.g["token_embed"] - full.g["token_embed"]).abs().max()
                                   / (full.g["token_embed"].abs().max() + 1e-9)).item()
        tr = TPTrainer(m)
        losses = [float(tr.train_step(x, y)) for _ in range(4)]
        res[backend + "_train"] = losses
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        out.put(res)
    dist.barrier()
    dist.destroy_process_group()


def test_tp_model_matches_single_gpu():
    from mp_util import run_ranks
    res = run_ranks(_model_worker, 2, ())[0]
    for b in ("fused", "nccl"):
        assert abs(res[b] - res["ref"]) < 0.03, res
        assert res[b + "_gerr"] < 0.06 and res[b + "_embed"] < 0.06, res
        assert res[b + "_train"][-1] < res[b + "_train"][0], res
