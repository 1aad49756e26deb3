"""Mixture-of-experts on the GPU: routing/permutation kernels against their PyTorch restatement,
the single-rank MoE decoder against the fp32 CPU model, and (two or more GPUs) the expert GEMMs
with the exchange fused in against the all-to-all composition."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def test_routing_and_permutation_kernels():
    from coeus_b200.ops import moe as M
    dev = torch.device("cuda")
    torch.manual_seed(0)
    T, E, K, H = 1000, 8, 2, 256
    C = 256
    logits = torch.randn(T, E, device=dev)
    got = M.route(logits, K, C)
    ref = M.route(logits.cpu(), K, C)
    names = ("expert", "weight", "probs", "slot", "counts")
    for n, g, r in zip(names, got, ref):
        if g.dtype.is_floating_point:
            assert (g.cpu() - r).abs().max() < 1e-5, n
        else:
            assert torch.equal(g.cpu().long(), r.long()), n
    expert, w, _, slot, _ = got
    x = torch.randn(T, H, device=dev).bfloat16()
    send = torch.zeros(E * C, H, device=dev, dtype=torch.bfloat16)
    M.gather_rows(x, expert, slot, send, C, scale=w)
    send_ref = torch.zeros(E * C, H)
    M.gather_rows(x.float().cpu(), expert.cpu(), slot.cpu(), send_ref, C, scale=w.cpu())
    assert (send.float().cpu() - send_ref).abs().max() < 2e-2
    ret = torch.randn(E * C, H, device=dev).bfloat16()
    resid = torch.randn(T, H, device=dev).bfloat16()
    out = M.combine_rows(ret, expert, slot, C, w, resid)
    out_ref = M.combine_rows(ret.float().cpu(), expert.cpu(), slot.cpu(), C, w.cpu(), resid.float().cpu())
    assert (out.float().cpu() - out_ref).abs().max() < 5e-2
    dots = M.pair_dot(x, ret, expert, slot, C)
    dots_ref = M.pair_dot(x.float().cpu(), ret.float().cpu(), expert.cpu(), slot.cpu(), C)
    assert (dots.cpu() - dots_ref).abs().max() < 1e-2 * dots_ref.abs().max()


def _cfg():
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=384,
                         vocab_size=512, max_seq_len=128, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope", num_experts=8, top_k=2, capacity_factor=2.0)


def test_moe_decoder_matches_cpu_model():
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    torch.manual_seed(0)
    cfg = _cfg()
    gpu = DecoderLM(cfg, device="cuda", seed=3)
    cpu = DecoderLM(cfg, device="cpu", dtype=torch.float32, seed=3)
    cpu.p32.copy_(gpu.p16.float().cpu())     # the bf16-rounded weights on both sides
    cpu.sync_working_copy()
    ids = torch.randint(0, cfg.vocab_size, (4, 128))
    tgt = torch.randint(0, cfg.vocab_size, (4, 128))
    gpu.zero_grad(); cpu.zero_grad()
    lg = gpu.forward_loss(ids.cuda(), tgt.cuda()); gpu.backward()
    lc = cpu.forward_loss(ids, tgt); cpu.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    assert abs(float(lg) - float(lc)) < 3e-2
    # bf16 rounding may flip the second expert of a few near-tied tokens; compare in aggregate
    for name in ("layers.1.moe.experts.down_weights", "layers.0.moe.experts.gate_up_weights",
                 "layers.0.moe.router_weights", "layers.0.attn.qkv_weights", "token_embed"):
        a, b = gpu.g[name].cpu().flatten(), cpu.g[name].flatten()
        cos = torch.dot(a, b) / (a.norm() * b.norm() + 1e-30)
        assert cos > 0.98, (name, float(cos))


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
    from coeus_b200.parallel.ep import ExpertParallel, MoEFFN
    H, I, E, K, T = 256, 384, 8, 2, 1024
    res = {}
    layers = {}
    for backend in ("fused", "nccl"):
        epx = ExpertParallel(dist.group.WORLD, dev, backend=backend)
        layers[backend] = MoEFFN(H, I, E, K, 1.5, epx, seed=11)
    for it in range(3):      # repeated use exercises the epoch / buffer reuse protocol
        torch.manual_seed(50 * it + rank)
        x = torch.randn(T, H, device=dev).bfloat16()
        resid = torch.randn(T, H, device=dev).bfloat16()
        dout = (torch.randn(T, H, device=dev) * 0.1).bfloat16()
        for backend, m in layers.items():
            m.zero_grad()
            o = m.forward(x, resid)
            dx = m.backward(dout)
            res[f"{backend}{it}"] = dict(o=o.float().cpu(), dx=dx.float().cpu(),
                                         **{k: v.float().cpu().clone() for k, v in m.g.items()})
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        out.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_fused_expert_exchange_matches_all_to_all():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 4 if torch.cuda.device_count() >= 4 else 2
    from mp_util import run_ranks
    res = run_ranks(_worker, world, ())[0]
    for it in range(3):
        f, n = res[f"fused{it}"], res[f"nccl{it}"]
        assert torch.equal(f["o"], n["o"])       # same GEMMs on the same rows
        assert torch.equal(f["dx"], n["dx"])
        for k in ("router", "gate_up", "down"):
            assert (f[k] - n[k]).abs().max() <= 1e-3 * n[k].abs().max() + 1e-6, k
