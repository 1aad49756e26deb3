"""Sharded data parallelism on CPU ranks (Gloo, world size 2): the sharding plan tiles the flat
buffer exactly, and two ranks with half the batch each reproduce one rank with the whole batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.models.config import DecoderConfig
from coeus_b200.models.decoder import DecoderLM, ParamLayout
from coeus_b200.parallel.plans import build_buckets, moment_offsets, shard_table
from coeus_b200.train.trainer import TrainConfig, Trainer

CFG = DecoderConfig(hidden_dim=128, num_layers=2, num_heads=2, intermediate_dim=256,
                    vocab_size=512, max_seq_len=64)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_shards_tile_the_flat_buffer(world):
    layout = ParamLayout(DecoderConfig.transformer_250m())
    n = layout.padded_total(8 * 1024)
    buckets = build_buckets(layout, n)
    covered = sorted((s, e) for r, lst in shard_table(buckets, world).items()
                     for _, s, e in lst if e > s)
    pos = 0
    for s, e in covered:
        assert s == pos and s % 8 == 0
        pos = e
    assert pos == n
    triggers = [b.trigger for b in buckets]
    assert triggers[0] == -1 and triggers[-1] == -2
    assert triggers[1:-2] == list(reversed(range(layout.cfg.num_layers)))
    for r in range(world):
        offs, total = moment_offsets(buckets, r, world)
        assert len(offs) == len(buckets) and total >= sum(
            b.shard(r, world)[1] - b.shard(r, world)[0] for b in buckets)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.zero import ShardedDataParallel
    torch.manual_seed(0)
    model = DecoderLM(CFG, device="cpu", seed=0)
    dp = ShardedDataParallel(dist.group.WORLD, "cpu")
    tr = Trainer(model, TrainConfig(learning_rate=1e-2), dp=dp)
    per = batch.shape[0] // world
    mine = batch[rank * per:(rank + 1) * per]
    losses = [float(tr.train_step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    full = dp.gather_master()
    if rank == 0:
        out.put((losses, full.clone(), model.p16.float().clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_match_one_rank():
    torch.manual_seed(0)
    batch = torch.randint(0, CFG.vocab_size, (4, 33))
    ref = DecoderLM(CFG, device="cpu", seed=0)
    tr = Trainer(ref, TrainConfig(learning_rate=1e-2))
    ref_losses = [float(tr.train_step(batch[:, :-1], batch[:, 1:])) for _ in range(3)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    losses, master, p16 = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # The parameters must agree.  The key bias (and through it a few key-projection weights) has
    # an analytically zero gradient (softmax ignores a shift of all keys); Adam turns its rounding
    # noise into +-lr steps, so those entries are compared by the fraction that moved apart.
    for s in ref.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        d = (master[sl] - ref.p32[sl]).abs()
        if "qkv" in s.name:
            assert (d > 1e-3).float().mean() < 0.3, s.name
        else:
            assert d.max() < 2e-3, (s.name, d.max())
            assert (p16[sl] - ref.p16[sl].float()).abs().max() < 2e-2, s.name
    assert losses[2] < losses[0] and ref_losses[2] < ref_losses[0]


def test_backward_reports_every_bucket_trigger_in_order():
    """The data-parallel buckets hang on these callbacks: head (-1), the layers from last to
    first, then -2 once the embedding gradient is complete."""
    import torch
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    cfg = DecoderConfig(hidden_dim=32, num_layers=3, num_heads=2, intermediate_dim=64,
                        vocab_size=64, max_seq_len=16)
    m = DecoderLM(cfg, "cpu", dtype=torch.float32)
    ids = torch.randint(0, 64, (2, 16))
    m.zero_grad()
    m.forward_loss(ids, ids)
    seen = []
    embed_done_at_minus2 = []

    def hook(t):
        seen.append(t)
        if t == -2:
            embed_done_at_minus2.append(float(m.g["token_embed"].abs().sum()) > 0)

    m.backward(on_layer_done=hook)
    assert seen == [-1, 2, 1, 0, -2]
    assert embed_done_at_minus2 == [True]
    assert m._saved is None


def _worker_replicated(rank, world, port, batch, tmp, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coeus_b200.parallel.dp import ReplicatedDataParallel
    model = DecoderLM(CFG, device="cpu", seed=0)
    dp = ReplicatedDataParallel(dist.group.WORLD, "cpu", overlap=(rank >= 0))
    tr = Trainer(model, TrainConfig(learning_rate=1e-2), dp=dp)
    per = batch.shape[0] // world
    mine = batch[rank * per:(rank + 1) * per]
    losses = [float(tr.train_step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    tr.save_checkpoint(tmp)
    if rank == 0:
        out.put((losses, dp.gather_master().numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_replicated_data_parallel_matches_one_rank(tmp_path):
    """The all-reduce comparator: two ranks on half the batch each equal one rank on all of it,
    and the checkpoint rank 0 writes loads into a single-replica trainer."""
    from mp_util import run_ranks
    torch.manual_seed(0)
    batch = torch.randint(0, CFG.vocab_size, (4, 33))
    ref = DecoderLM(CFG, device="cpu", seed=0)
    tr = Trainer(ref, TrainConfig(learning_rate=1e-2))
    ref_losses = [float(tr.train_step(batch[:, :-1], batch[:, 1:])) for _ in range(3)]
    losses, full = run_ranks(_worker_replicated, 2, (batch, str(tmp_path)))[0]
    # each rank's loss is over its own half; the mean of the first step's halves is not
    # available here, so compare weights (and that the loss falls)
    assert losses[-1] < losses[0]
    # bf16 working precision: Adam turns rounding differences of the two reduction orders into
    # fractions of a step (lr = 1e-2)
    assert (torch.from_numpy(full) - ref.p32).abs().max() < 4e-3
    other = Trainer(DecoderLM(CFG, device="cpu", seed=5), TrainConfig(learning_rate=1e-2))
    meta = other.load_checkpoint(str(tmp_path))
    assert int(meta["train_step"]) == 3
    assert torch.equal(other.model.p32, torch.from_numpy(full))
    assert len(ref_losses) == 3


def test_symmetric_heap_offset_allocator():
    from coeus_b200.parallel.symm import OffsetAllocator
    a = OffsetAllocator(4096, alignment=256)
    x, y, z = a.alloc(100), a.alloc(300), a.alloc(256)
    assert (x, y, z) == (0, 256, 768) and a.used() == 1024
    a.release(y)
    assert a.alloc(512) == 256                      # first fit reuses the hole exactly
    a.release(x)
    a.release(256)
    assert a.free[0] == [0, 768]                    # neighbours coalesce
    w = a.alloc(3072)
    assert w == 1024 and a.peak == 3072 + 256
    with pytest.raises(Exception):
        a.alloc(1024)
    a.release(z)
    a.release(w)
    assert a.free == [[0, 4096]] and a.used() == 0
    # the same call sequence gives the same offsets on every "rank"
    b, c = OffsetAllocator(1 << 20), OffsetAllocator(1 << 20)
    seq = [1000, 70000, 5, 4096]
    assert [b.alloc(n) for n in seq] == [c.alloc(n) for n in seq]
