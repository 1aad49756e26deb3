"""``build_trainer``: one call from a ParallelConfig to a running trainer, for every strategy, on
two Gloo ranks; the first-step loss is the single-rank loss of the same global batch and the
loss falls."""
import os

import pytest
import torch
import torch.distributed as dist

from coeus_b200.core.config import ParallelConfig
from coeus_b200.models.config import DecoderConfig
from coeus_b200.train.launch import build_trainer
from coeus_b200.train.trainer import TrainConfig


def _cfg(moe=False, layers=2):
    kw = dict(num_experts=4, top_k=2, capacity_factor=4.0, aux_loss_coef=0.0) if moe else {}
    return DecoderConfig(hidden_dim=32, num_layers=layers, num_heads=2, intermediate_dim=64,
                         vocab_size=96, max_seq_len=16, use_bias=False, activation="swiglu",
                         norm="rmsnorm", pos="rope", **kw)


def _tc(clip=None):
    return TrainConfig(learning_rate=0.05, eps=1.0, weight_decay=0.0, grad_clip=clip)


def _batch():
    torch.manual_seed(0)
    return torch.randint(0, 96, (4, 16)), torch.randint(0, 96, (4, 16))


def _worker(rank, world, port, kind, out, clip=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if kind == "dp0":
        par = ParallelConfig(dp=world, zero_stage=0)
    elif kind == "pp_interleaved":
        par = ParallelConfig(pp=world, pp_chunks=2)
    elif kind == "ulysses":
        par = ParallelConfig(cp=world, ulysses=True)
    else:
        par = ParallelConfig(**{kind: world})
    if kind == "ep":
        par = ParallelConfig(dp=world, ep=world)
    from coeus_b200.optim.lr import Constant
    run = build_trainer(_cfg(moe=(kind == "ep"), layers=4 if kind == "pp_interleaved" else 2),
                        par, "cpu", _tc(clip), micro_batches=2, seed=3,
                        dtype=torch.float32, schedule=Constant(0.05))
    ids, tgt = _batch()
    losses = [float(run.step(ids, tgt)) for _ in range(4)]
    opt = run.trainer.opt if hasattr(run.trainer, "opt") else run.trainer.opts[0]
    dp = getattr(run.trainer, "dp", None)
    lr_now = dp.opt_cfg.lr if dp is not None else opt.learning_rate()
    assert abs(lr_now - 0.05) < 1e-12
    t = torch.tensor(losses)
    if kind in ("dp", "dp0", "ep", "cp", "ulysses"):       # each rank reports the loss of its own part
        dist.all_reduce(t)
        t /= world
    out.put((rank, run.strategy, t.tolist()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["dp", "dp0", "tp", "pp", "pp_interleaved", "ep", "cp", "ulysses"])
def test_every_strategy_through_the_launcher(kind):
    from mp_util import run_ranks
    ids, tgt = _batch()
    single = build_trainer(_cfg(moe=(kind == "ep"), layers=4 if kind == "pp_interleaved" else 2),
                           ParallelConfig(), "cpu", _tc(), seed=3, dtype=torch.float32)
    assert single.strategy == "single"
    ref = [float(single.step(ids, tgt)) for _ in range(4)]
    res = {r[0]: r for r in run_ranks(_worker, 2, (kind,), results=2)}
    want = {"ulysses": "cp", "dp0": "dp", "pp_interleaved": "pp"}.get(kind, kind)
    assert res[0][1] == want
    got = res[1][2]          # rank 1 is the last pipeline stage; the others agree on all ranks
    tol = 2e-2 if kind == "ep" else 1e-4     # capacity slots differ between 1 and 2 ranks
    assert abs(got[0] - ref[0]) < tol, (got, ref)
    assert got[-1] < got[0]
    if kind != "ep":
        assert abs(got[-1] - ref[-1]) < 5e-3


def _worker_clip(rank, world, port, kind, clip, out):
    _worker(rank, world, port, kind, out, clip)


@pytest.mark.parametrize("kind", ["dp", "tp", "pp", "pp_interleaved", "cp"])
def test_gradient_clipping_uses_the_global_norm_in_every_strategy(kind):
    """With eps = 1 the AdamW update depends on the gradient scale, so a run clipped at a small
    threshold only follows the clipped single-rank run if every rank clips by the norm of ALL
    gradients (sharded, staged or replicated)."""
    from mp_util import run_ranks
    ids, tgt = _batch()
    layers = 4 if kind == "pp_interleaved" else 2
    ref, free = [], []
    for clip, dst in ((0.02, ref), (None, free)):
        single = build_trainer(_cfg(layers=layers), ParallelConfig(), "cpu", _tc(clip), seed=3,
                               dtype=torch.float32)
        dst += [float(single.step(ids, tgt)) for _ in range(4)]
    assert abs(ref[-1] - free[-1]) > 0.02          # the threshold is active
    res = {r[0]: r for r in run_ranks(_worker_clip, 2, (kind, 0.02), results=2)}
    got = res[1][2]
    assert abs(got[-1] - ref[-1]) < 3e-3, (got, ref, free)


def _worker_2d(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    run = build_trainer(_cfg(), ParallelConfig(dp=2, tp=2), "cpu", _tc(), seed=3,
                        dtype=torch.float32)
    ids, tgt = _batch()
    t = torch.tensor([float(run.step(ids, tgt)) for _ in range(4)])
    dist.all_reduce(t)               # two replicas x two ranks, each reporting its replica's loss
    out.put((rank, run.strategy, (t / world).tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_replicas_of_a_tensor_parallel_model():
    from mp_util import run_ranks
    ids, tgt = _batch()
    single = build_trainer(_cfg(), ParallelConfig(), "cpu", _tc(), seed=3, dtype=torch.float32)
    ref = [float(single.step(ids, tgt)) for _ in range(4)]
    res = run_ranks(_worker_2d, 4, (), results=4)
    for _, strategy, got in res:
        assert strategy == "dp+tp"
        assert abs(got[0] - ref[0]) < 1e-4 and abs(got[-1] - ref[-1]) < 5e-3, (got, ref)


def _worker_dp_pp(rank, world, port, chunks, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    run = build_trainer(_cfg(layers=4), ParallelConfig(dp=2, pp=2, pp_chunks=chunks), "cpu",
                        _tc(0.02 if chunks == 1 else None), micro_batches=2, seed=3,
                        dtype=torch.float32)
    ids, tgt = _batch()
    losses = [float(run.step(ids, tgt)) for _ in range(3)]
    # a checkpoint written by the first replica, loaded by both: the next step is the same
    import tempfile
    box = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    run.trainer.save_checkpoint(box[0])
    dist.barrier()
    assert sorted(f for f in os.listdir(box[0]) if f.startswith("part")) == \
        ["part0.safetensors", "part1.safetensors"]
    nxt = float(run.step(ids, tgt))
    run.trainer.load_checkpoint(box[0])
    again = float(run.step(ids, tgt))
    assert abs(again - nxt) < 1e-6
    t = torch.tensor(losses + [nxt])
    dist.all_reduce(t)               # the last stage of each replica reports its replica's loss
    out.put((rank, run.strategy, (t / 2).tolist()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 2])
def test_data_parallel_replicas_of_a_pipeline(chunks):
    """Two pipelines of two stages side by side (plain with gradient clipping by the global
    norm, and interleaved): the same losses as one rank on the whole batch."""
    from mp_util import run_ranks
    ids, tgt = _batch()
    single = build_trainer(_cfg(layers=4), ParallelConfig(), "cpu",
                           _tc(0.02 if chunks == 1 else None), seed=3, dtype=torch.float32)
    ref = [float(single.step(ids, tgt)) for _ in range(4)]
    res = run_ranks(_worker_dp_pp, 4, (chunks,), results=4)
    for _, strategy, got in res:
        assert strategy == "dp+pp"
        assert abs(got[0] - ref[0]) < 1e-4 and abs(got[-1] - ref[-1]) < 5e-3, (got, ref)


def test_launcher_rejects_products_and_wrong_sizes():
    with pytest.raises(Exception):
        build_trainer(_cfg(), ParallelConfig(pp=2, tp=2), "cpu")
    with pytest.raises(Exception):
        build_trainer(_cfg(), ParallelConfig(tp=2), "cpu")      # no process group of 2 here
    with pytest.raises(Exception):
        build_trainer(_cfg(), ParallelConfig(zero_stage=3), "cpu")


def test_pipeline_transport_is_a_checked_option():
    from coeus_b200.foundation.error import ConfigError
    assert ParallelConfig(pp=2).pp_transport == "auto"
    ParallelConfig(pp=2, pp_transport="peer").validate()
    with pytest.raises(ConfigError):
        ParallelConfig(pp=2, pp_transport="smoke signals").validate()
