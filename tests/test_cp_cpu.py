"""Context parallelism (ring attention, zig-zag chunks) on CPU: the chunked attention on one
rank, and two Gloo ranks, against the ordinary model on the whole sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.parallel.cp import ContextParallel


def _cfg(pos="rope"):
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=48,
                         vocab_size=96, max_seq_len=32, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos=pos)


def test_pairs_are_balanced():
    class Fake(ContextParallel):
        def __init__(self, rank, cp):
            self.rank, self.cp = rank, cp
    for cp in (2, 4, 8):
        for r in range(cp):
            f = Fake(r, cp)
            for s in range(cp):
                pairs = f._pairs(s)
                if s == r:
                    assert sorted(pairs) == [(0, 0, True), (1, 0, False), (1, 1, True)]
                else:
                    assert len(pairs) == 2 and not any(c for _, _, c in pairs)


@pytest.mark.parametrize("pos", ["rope", "sinusoidal"])
def test_single_rank_chunked_attention_matches_plain_model(pos):
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(0)
    cfg = _cfg(pos)
    cp = ContextParallel(None, "cpu")
    plain = DecoderLM(cfg, "cpu", seed=2, dtype=torch.float32)
    ring = DecoderLM(cfg, "cpu", seed=2, dtype=torch.float32, cp=cp)
    ids = torch.randint(0, 96, (3, 32))
    tgt = torch.randint(0, 96, (3, 32))
    plain.zero_grad(); ring.zero_grad()
    l0 = plain.forward_loss(ids, tgt); plain.backward()
    l1 = ring.forward_loss(cp.shard(ids), cp.shard(tgt)); ring.backward()
    assert abs(float(l0) - float(l1)) < 1e-5
    assert (plain.g32 - ring.g32).abs().max() < 1e-5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ids, tgt, out, kind="ring"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel.ulysses import UlyssesParallel
    cp = (ContextParallel if kind == "ring" else UlyssesParallel)(dist.group.WORLD, "cpu")
    m = DecoderLM(_cfg(), "cpu", seed=2, dtype=torch.float32, cp=cp)
    m.zero_grad()
    loss = m.forward_loss(cp.shard(ids), cp.shard(tgt))
    m.backward()
    dist.all_reduce(m.g32)
    m.g32 /= world
    lt = loss.clone()
    dist.all_reduce(lt)
    out.put((rank, float(lt) / world, m.g32.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,kind", [(2, "ring"), (4, "ring"), (2, "ulysses")])
def test_sequence_parallel_ranks_match_plain_model(world, kind):
    from coeus_b200.models.decoder import DecoderLM
    torch.manual_seed(1)
    ids = torch.randint(0, 96, (2, 32))
    tgt = torch.randint(0, 96, (2, 32))
    plain = DecoderLM(_cfg(), "cpu", seed=2, dtype=torch.float32)
    plain.zero_grad()
    l0 = float(plain.forward_loss(ids, tgt))
    plain.backward()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ids, tgt, q, kind)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, loss, g in res:
        assert abs(loss - l0) < 1e-5
        assert (torch.from_numpy(g) - plain.g32).abs().max() < 1e-5
