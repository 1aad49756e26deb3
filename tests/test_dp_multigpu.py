"""Sharded data parallelism on real GPUs: the fused reduce-scatter + AdamW + all-gather kernel
over NVLink peer memory against the same step done with NCCL collectives."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.models.config import DecoderConfig

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

CFG = DecoderConfig(hidden_dim=256, num_layers=2, num_heads=4, intermediate_dim=1024,
                    vocab_size=2048, max_seq_len=256)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, backend, out, clip=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.ops import _lib
    from coeus_b200.parallel.zero import ShardedDataParallel
    from coeus_b200.train.trainer import TrainConfig, Trainer
    model = DecoderLM(CFG, device=dev, seed=0)
    nvls = backend == "p2p-nvls"      # the same kernel reading through the NVLink multicast mapping
    dp = ShardedDataParallel(dist.group.WORLD, dev, backend="p2p" if nvls else backend, nvls=nvls)
    tr = Trainer(model, TrainConfig(learning_rate=1e-3, grad_clip=clip), dp=dp)
    gen = torch.Generator().manual_seed(100 + rank)
    batch = torch.randint(0, CFG.vocab_size, (2, 129), generator=gen).to(dev)
    losses = [float(tr.train_step(batch[:, :-1], batch[:, 1:])) for _ in range(4)]
    full = dp.gather_master()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        out.put((losses, full.cpu(), model.p16.float().cpu()))
    dist.barrier()
    dist.destroy_process_group()


def _run(backend, world=2, clip=None):
    from mp_util import run_ranks

    res = run_ranks(_worker_clip if clip is not None else _worker, world,
                    (backend, clip) if clip is not None else (backend,))[0]
    return res


def _worker_clip(rank, world, port, backend, clip, out):
    _worker(rank, world, port, backend, out, clip)


def test_fused_kernel_matches_nccl_collectives():
    l_ref, m_ref, p_ref = _run("collective")
    l_p2p, m_p2p, p_p2p = _run("p2p")
    assert l_p2p[-1] < l_p2p[0]
    for a, b in zip(l_ref, l_p2p):
        assert abs(a - b) < 0.05
    d = (m_ref - m_p2p).abs()
    # Adam amplifies rounding noise on (near-)zero gradients (e.g. the key bias), so compare by
    # the fraction of entries that moved apart
    assert (d > 5e-4).float().mean() < 0.01, d.max()
    assert (p_ref - p_p2p).abs().max() < 0.05


def test_switch_reduced_kernel_matches_nccl_collectives():
    """The bucket kernel with multimem.ld_reduce / multimem.st (NVLink multicast) against the
    collective path; falls back to plain peer loads by itself where multicast is unsupported."""
    l_ref, m_ref, p_ref = _run("collective")
    l_mc, m_mc, p_mc = _run("p2p-nvls")
    for a, b in zip(l_ref, l_mc):
        assert abs(a - b) < 0.05
    d = (m_ref - m_mc).abs()
    assert (d > 5e-4).float().mean() < 0.01, d.max()
    assert (p_ref - p_mc).abs().max() < 0.05


def test_gradient_clipping_in_the_fused_step_matches_collectives():
    """With a clip threshold far below the gradient norm the split kernel (reduce-scatter + sum of
    squares, then AdamW + all-gather with the coefficient) must follow the NCCL path."""
    l_ref, m_ref, _ = _run("collective", clip=0.05)
    l_p2p, m_p2p, _ = _run("p2p", clip=0.05)
    for a, b in zip(l_ref, l_p2p):
        assert abs(a - b) < 0.05
    d = (m_ref - m_p2p).abs()
    assert (d > 5e-4).float().mean() < 0.01, d.max()
