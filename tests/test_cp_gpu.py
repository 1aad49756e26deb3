"""Sequence parallelism on GPUs: ring-attention helper kernels against their PyTorch restatement,
chunked attention on one GPU against the plain model, and (two GPUs) the peer-to-peer transports
of ring attention and Ulysses against the collective ones."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def test_ring_helper_kernels():
    from coeus_b200.ops import ring as R
    dev = torch.device("cuda")
    torch.manual_seed(0)
    B, S, nh, dh = 2, 96, 4, 64
    H = nh * dh
    o_acc = torch.randn(B * S, H, device=dev)
    lse_acc = torch.randn(B, nh, S, device=dev)
    o_p = torch.randn(B * S, H, device=dev).bfloat16()
    lse_p = torch.randn(B, nh, S, device=dev)
    ref_o, ref_l = o_acc.cpu().clone(), lse_acc.cpu().clone()
    R.merge_partial(ref_o, ref_l, o_p.cpu(), lse_p.cpu(), B, S, nh, dh, first=False)
    R.merge_partial(o_acc, lse_acc, o_p, lse_p, B, S, nh, dh, first=False)
    assert (o_acc.cpu() - ref_o).abs().max() < 1e-4
    assert (lse_acc.cpu() - ref_l).abs().max() < 1e-4
    R.merge_partial(o_acc, lse_acc, o_p, lse_p, B, S, nh, dh, first=True)
    assert torch.equal(o_acc.cpu(), o_p.float().cpu()) and torch.equal(lse_acc.cpu(), lse_p.cpu())
    acc = torch.randn(100, 3 * H, device=dev)
    x = torch.randn(100, H, device=dev).bfloat16()
    want = acc[:, H:2 * H].cpu() + x.float().cpu()
    R.accum_rows(acc[:, H:2 * H], x)
    assert (acc[:, H:2 * H].cpu() - want).abs().max() < 1e-6
    dst = torch.empty(100, 3 * H, device=dev, dtype=torch.bfloat16)
    R.cast_rows(acc[:, :H], dst[:, H:2 * H], 0.5)
    assert (dst[:, H:2 * H].float().cpu() - (acc[:, :H] * 0.5).bfloat16().float().cpu()).abs().max() == 0
    a = torch.randn(4096, device=dev)
    b = torch.randn(4096, device=dev)
    want = (a + b).cpu()
    R.peer_add_f32(a.data_ptr(), b)
    assert (a.cpu() - want).abs().max() < 1e-6


def _cfg(S):
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=512,
                         vocab_size=512, max_seq_len=S, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope")


def _cos(a, b):
    a, b = a.flatten().float(), b.flatten().float()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))


def test_chunked_attention_on_one_gpu_matches_plain_model():
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.cp import ContextParallel
    torch.manual_seed(0)
    S = 512
    cp = ContextParallel(None, "cuda")
    plain = DecoderLM(_cfg(S), "cuda", seed=2)
    ring = DecoderLM(_cfg(S), "cuda", seed=2, cp=cp)
    ids = torch.randint(0, 512, (2, S), device="cuda")
    tgt = torch.randint(0, 512, (2, S), device="cuda")
    plain.zero_grad(); ring.zero_grad()
    l0 = plain.forward_loss(ids, tgt); plain.backward()
    l1 = ring.forward_loss(cp.shard(ids), cp.shard(tgt)); ring.backward()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    assert abs(float(l0) - float(l1)) < 2e-2
    for name in ("layers.0.attn.qkv_weights", "layers.1.attn.o_weights", "token_embed"):
        assert _cos(plain.g[name], ring.g[name]) > 0.995, name


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
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.cp import ContextParallel
    from coeus_b200.parallel.ulysses import UlyssesParallel
    S = 1024
    torch.manual_seed(3)
    ids = torch.randint(0, 512, (2, S), device=dev)
    tgt = torch.randint(0, 512, (2, S), device=dev)
    res = {}
    for kind, cls in (("ring", ContextParallel), ("ulysses", UlyssesParallel)):
        for backend in ("p2p", "collective"):
            sp = cls(dist.group.WORLD, dev, backend=backend)
            m = DecoderLM(_cfg(S), dev, seed=2, cp=sp)
            for it in range(2):     # second pass exercises buffer reuse
                m.zero_grad()
                loss = m.forward_loss(sp.shard(ids), sp.shard(tgt))
                m.backward()
            dist.all_reduce(m.g32)
            lt = loss.clone()
            dist.all_reduce(lt)
            res[f"{kind}:{backend}"] = (float(lt) / world, m.g32.float().cpu() / world)
    plain = DecoderLM(_cfg(S), dev, seed=2)
    plain.zero_grad()
    l0 = plain.forward_loss(ids, tgt)
    plain.backward()
    res["plain"] = (float(l0), plain.g32.float().cpu())
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        out.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_sequence_parallel_transports_on_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    from mp_util import run_ranks
    res = run_ranks(_worker, world, ())[0]
    l0, g0 = res["plain"]
    for key in ("ring:p2p", "ring:collective", "ulysses:p2p", "ulysses:collective"):
        l, g = res[key]
        assert abs(l - l0) < 2e-2, key
        assert _cos(g, g0) > 0.995, key
    assert _cos(res["ring:p2p"][1], res["ring:collective"][1]) > 0.9999
    assert torch.equal(res["ulysses:p2p"][1], res["ulysses:collective"][1]) or \
        _cos(res["ulysses:p2p"][1], res["ulysses:collective"][1]) > 0.9999
