"""Failure detection and elastic recovery with CPU ranks only: a rank leaves between steps, the
others notice through heartbeats, regroup to the smaller world and continue from the sharded
checkpoint.  Also the host fault injector and the step watchdog."""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coeus_b200.parallel.health import FaultInjector, InjectedFault, StepWatchdog


def test_fault_injector_fires_on_the_named_occurrence():
    inj = FaultInjector("after_bucket:3,before_step")
    inj.reach("after_bucket"); inj.reach("after_bucket")
    with pytest.raises(InjectedFault) as e:
        inj.reach("after_bucket")
    assert e.value.point == "after_bucket" and e.value.count == 3
    inj.reach("after_bucket")                       # only the third time
    with pytest.raises(InjectedFault):
        inj.reach("before_step")
    FaultInjector("").reach("anything")


def test_step_watchdog_flags_outliers():
    w = StepWatchdog(factor=3.0, warmup=3)
    assert not any(w.observe(t) for t in (1.0, 1.1, 0.9, 1.0, 1.2))
    assert w.observe(5.0)
    assert w.outliers == 1


def _cfg():
    from coeus_b200.models.config import DecoderConfig
    return DecoderConfig(hidden_dim=32, num_layers=2, num_heads=2, intermediate_dim=64,
                         vocab_size=64, max_seq_len=16, use_bias=True)


def _batch(step, rank, world):
    g = torch.Generator().manual_seed(100 + step)
    b = torch.randint(0, 64, (12, 17), generator=g)
    n = 12 // world
    return b[rank * n:(rank + 1) * n, :-1].contiguous(), b[rank * n:(rank + 1) * n, 1:].contiguous()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, pg_port, store_port, ckpt, out):
    from datetime import timedelta
    from coeus_b200.foundation.error import CommError
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.parallel import health
    from coeus_b200.parallel.zero import ShardedDataParallel
    from coeus_b200.train.trainer import TrainConfig, Trainer
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0),
                          timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", store=dist.PrefixStore("gen0", store), rank=rank,
                            world_size=world)
    hb = health.Heartbeat(store, rank, world, interval_s=0.05, timeout_s=1.0).start()
    m = DecoderLM(_cfg(), "cpu", seed=1, dtype=torch.float32)
    tr = Trainer(m, TrainConfig(learning_rate=1e-2), dp=ShardedDataParallel(dist.group.WORLD, "cpu"))
    for s in range(2):
        tr.train_step(*_batch(s, rank, world))
    tr.save_checkpoint(ckpt, data_cursor=2)
    if rank == world - 1:
        # this rank "fails": it leaves between steps with nothing in flight and stops beating
        hb.stop()
        out.put((rank, "left", None))
        return
    # survivors: the next step starts with a liveness check on the host
    deadline = time.monotonic() + 20
    detected = None
    while time.monotonic() < deadline:
        try:
            hb.require_alive()
        except CommError as e:
            detected = e
            break
        time.sleep(0.1)
    assert detected is not None
    dead = hb.dead_peers()
    alive = health.agree_on_survivors(store, rank, world, dead, generation=1)
    dist.destroy_process_group()
    new_rank, new_world = health.regroup(store, rank, alive, generation=1)
    m2 = DecoderLM(_cfg(), "cpu", seed=1, dtype=torch.float32)
    tr2 = Trainer(m2, TrainConfig(learning_rate=1e-2),
                  dp=ShardedDataParallel(dist.group.WORLD, "cpu"))
    meta = tr2.load_checkpoint(ckpt)
    for s in range(meta["train_step"], 4):
        tr2.train_step(*_batch(s, new_rank, new_world))
    full = tr2.dp.gather_master()
    out.put((rank, "survived", (alive, new_world, tr2.step_index, full.numpy().copy())))
    dist.barrier()
    hb.stop()
    dist.destroy_process_group()


def test_rank_loss_is_detected_and_training_continues_on_fewer_ranks(tmp_path):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    pg_port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, pg_port, store_port, str(tmp_path / "ck"), q))
             for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r = q.get(timeout=180)
        res[r[0]] = r
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[2][1] == "left"
    for r in (0, 1):
        alive, new_world, steps, _ = res[r][2]
        assert alive == [0, 1] and new_world == 2 and steps == 4
    assert (torch.from_numpy(res[0][2][3]) - torch.from_numpy(res[1][2][3])).abs().max() == 0
