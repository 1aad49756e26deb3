"""One entry point from a :class:`coeus_b200.core.config.ParallelConfig` to a ready trainer.

``build_trainer`` reads which strategy the configuration asks for, builds the communication state
and the (sharded) model of that strategy over the given process group, and returns a
:class:`ParallelRun` whose ``step(ids, targets)`` takes the *global* batch on every rank and feeds
each rank the part its strategy wants (a slice of sequences for data and expert parallelism, the
whole batch for tensor parallelism, micro-batches for a pipeline, zig-zag chunks of every sequence
for context parallelism).  One strategy spans the group, with one product: data parallelism over replicas of a
tensor-parallel model (``dp x tp``, ranks ``[d * tp, (d + 1) * tp)`` forming replica ``d``);
other products are rejected with a configuration error rather than half-supported.  The reference is a
single process (no parallelism of any kind in its sources).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from ..core.config import ParallelConfig
from ..foundation.error import ConfigError
from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM
from .trainer import TrainConfig, Trainer


@dataclass
class ParallelRun:
    strategy: str                       # single | dp | tp | pp | ep | cp
    trainer: Any
    model: Any
    rank: int
    world: int
    _feed: Callable

    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """``ids`` / ``targets``: the global ``[B, S]`` batch, identical on every rank.  Returns
        this rank's loss (pipeline: the last stage holds it, the others return zeros)."""
        return self._feed(ids, targets)


def build_trainer(cfg: DecoderConfig, parallel: ParallelConfig, device,
                  train_cfg: Optional[TrainConfig] = None, group=None, micro_batches: int = 1,
                  seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                  recompute: bool = False, schedule=None) -> ParallelRun:
    """``schedule`` (an object with ``at(step) -> lr``, :mod:`coeus_b200.optim.lr`) drives the
    learning rate of whichever trainer is built."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    parallel.validate()
    active = [k for k in ("dp", "tp", "pp", "ep", "cp") if getattr(parallel, k) > 1]
    if parallel.ep > 1 and parallel.dp == parallel.ep:
        active = [k for k in active if k != "dp"]    # the expert group is the data group
    if active == ["dp", "tp"]:
        return _build_dp_tp(cfg, parallel, device, train_cfg or TrainConfig(), group, world, rank,
                            seed, dtype, recompute, schedule)
    if active == ["dp", "pp"]:
        return _build_dp_pp(cfg, parallel, device, train_cfg or TrainConfig(), group, world, rank,
                            seed, dtype, schedule, micro_batches)
    if len(active) > 1:
        raise ConfigError.conflict(active[0], active[1],
                                   "one parallelism strategy spans the process group at a time")
    strategy = active[0] if active else "single"
    if strategy != "single" and getattr(parallel, strategy) != world:
        raise ConfigError.invalid(strategy, getattr(parallel, strategy),
                                  f"must equal the size of the process group ({world})")
    if strategy != "single" and group is None:
        group = dist.group.WORLD
    device = torch.device(device)
    tc = train_cfg or TrainConfig()
    cpu = device.type != "cuda"
    if tc.grad_accum > 1 and strategy in ("tp", "pp", "ep"):
        raise ConfigError.invalid("grad_accum", tc.grad_accum,
                                  "Gradient accumulation is built into the plain and "
                                  "data-parallel trainers; a pipeline accumulates over its "
                                  "micro_batches")

    if strategy == "single":
        model = DecoderLM(cfg, device, seed=seed, dtype=dtype, recompute=recompute)
        tr = Trainer(model, tc, schedule=schedule)
        return ParallelRun(strategy, tr, model, rank, world, tr.train_step)

    if strategy == "dp":
        model = DecoderLM(cfg, device, seed=seed, dtype=dtype, recompute=recompute)
        if parallel.zero_stage == 0:
            from ..parallel.dp import ReplicatedDataParallel
            dp_obj = ReplicatedDataParallel(group, device)
        else:
            from ..parallel.zero import ShardedDataParallel
            dp_obj = ShardedDataParallel(group, device,
                                         backend="collective" if cpu else parallel.dp_backend)
        tr = Trainer(model, tc, dp=dp_obj, schedule=schedule)

        def feed(ids, targets):
            per = ids.shape[0] // world
            sl = slice(rank * per, (rank + 1) * per)
            return tr.train_step(ids[sl].contiguous(), targets[sl].contiguous())
        return ParallelRun(strategy, tr, model, rank, world, feed)

    if strategy == "tp":
        from ..parallel.tp import TensorParallel
        from ..parallel.tp_model import TPDecoderLM, TPTrainer
        tp = TensorParallel(group, device)
        model = TPDecoderLM(cfg, tp, device, seed=seed, dtype=dtype, recompute=recompute)
        tr = TPTrainer(model, tc.adamw(), schedule=schedule)
        return ParallelRun(strategy, tr, model, rank, world, tr.train_step)

    if strategy == "pp":
        from ..parallel.pp import InterleavedPipelineStage, PipelineStage
        transport = None if parallel.pp_transport == "auto" else parallel.pp_transport
        if parallel.pp_chunks > 1:
            st = InterleavedPipelineStage(cfg, group, device, micro_batches,
                                          chunks=parallel.pp_chunks, seed=seed, dtype=dtype,
                                          train_cfg=tc, schedule=schedule, transport=transport)
        else:
            st = PipelineStage(cfg, group, device, micro_batches, seed=seed, dtype=dtype,
                               train_cfg=tc, schedule=schedule, transport=transport or "nccl")

        def feed(ids, targets):
            M = micro_batches
            b = ids.shape[0] // M
            return st.train_step(ids.reshape(M, b, -1), targets.reshape(M, b, -1))
        return ParallelRun(strategy, st, getattr(st, "model", None) or st.models[0], rank, world,
                           feed)

    if strategy == "ep":
        from ..parallel.ep import ExpertParallel, ExpertParallelTrainer
        epx = ExpertParallel(group, device)
        model = DecoderLM(cfg, device, seed=seed, dtype=dtype, epx=epx, recompute=recompute)
        tr = ExpertParallelTrainer(model, tc, schedule=schedule)

        def feed(ids, targets):
            per = ids.shape[0] // world
            sl = slice(rank * per, (rank + 1) * per)
            return tr.train_step(ids[sl].contiguous(), targets[sl].contiguous())
        return ParallelRun(strategy, tr, model, rank, world, feed)

    # context parallelism: every rank sees its chunks of every sequence; gradients are summed over
    # the group exactly like data-parallel replicas
    from ..parallel.zero import ShardedDataParallel
    if parallel.ulysses:
        from ..parallel.ulysses import UlyssesParallel
        cp = UlyssesParallel(group, device)
    else:
        from ..parallel.cp import ContextParallel
        cp = ContextParallel(group, device)
    model = DecoderLM(cfg, device, seed=seed, dtype=dtype, cp=cp, recompute=recompute)
    backend = "collective" if cpu else parallel.dp_backend
    tr = Trainer(model, tc, dp=ShardedDataParallel(group, device, backend=backend),
                 schedule=schedule)

    def feed_cp(ids, targets):
        return tr.train_step(cp.shard(ids), cp.shard(targets))
    return ParallelRun("cp", tr, model, rank, world, feed_cp)


def _build_dp_tp(cfg, parallel, device, tc, group, world, rank, seed, dtype, recompute, schedule):
    """Replicas of a tensor-parallel model: ``tp`` consecutive ranks share a model, ranks with the
    same position in their replica average gradients."""
    from ..parallel.tp import TensorParallel
    from ..parallel.tp_model import TPDecoderLM, TPTrainer
    dp, tp = parallel.dp, parallel.tp
    if tc.grad_accum > 1:
        raise ConfigError.invalid("grad_accum", tc.grad_accum,
                                  "Not built for replicas of a tensor-parallel model")
    if dp * tp != world:
        raise ConfigError.invalid("dp*tp", dp * tp, f"must equal the size of the process group ({world})")
    ranks = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
    d_idx, t_idx = rank // tp, rank % tp
    tp_group = dp_group = None
    # every rank creates every group, in the same order
    for d in range(dp):
        g = dist.new_group([ranks[d * tp + t] for t in range(tp)])
        if d == d_idx:
            tp_group = g
    for t in range(tp):
        g = dist.new_group([ranks[d * tp + t] for d in range(dp)])
        if t == t_idx:
            dp_group = g
    device = torch.device(device)
    model = TPDecoderLM(cfg, TensorParallel(tp_group, device), device, seed=seed, dtype=dtype,
                        recompute=recompute)
    tr = TPTrainer(model, tc.adamw(), dp_group=dp_group, schedule=schedule)

    def feed(ids, targets):
        per = ids.shape[0] // dp
        sl = slice(d_idx * per, (d_idx + 1) * per)
        return tr.train_step(ids[sl].contiguous(), targets[sl].contiguous())
    return ParallelRun("dp+tp", tr, model, rank, world, feed)


def _build_dp_pp(cfg, parallel, device, tc, group, world, rank, seed, dtype, schedule,
                 micro_batches):
    """Replicas of a pipeline: ``pp`` consecutive ranks form a pipeline, ranks that hold the same
    stage in different replicas average their gradients.  Every replica is fed its own part of
    the batch, cut into ``micro_batches`` micro-batches."""
    from ..parallel.pp import InterleavedPipelineStage, PipelineStage
    dp, pp = parallel.dp, parallel.pp
    if tc.grad_accum > 1:
        raise ConfigError.invalid("grad_accum", tc.grad_accum,
                                  "A pipeline accumulates over its micro_batches")
    if dp * pp != world:
        raise ConfigError.invalid("dp*pp", dp * pp, f"must equal the size of the process group ({world})")
    ranks = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
    d_idx, p_idx = rank // pp, rank % pp
    pp_group = dp_group = None
    # every rank creates every group, in the same order
    for d in range(dp):
        g = dist.new_group([ranks[d * pp + p] for p in range(pp)])
        if d == d_idx:
            pp_group = g
    for p in range(pp):
        g = dist.new_group([ranks[d * pp + p] for d in range(dp)])
        if p == p_idx:
            dp_group = g
    transport = None if parallel.pp_transport == "auto" else parallel.pp_transport
    if parallel.pp_chunks > 1:
        st = InterleavedPipelineStage(cfg, pp_group, device, micro_batches,
                                      chunks=parallel.pp_chunks, seed=seed, dtype=dtype,
                                      train_cfg=tc, schedule=schedule, transport=transport,
                                      dp_group=dp_group)
    else:
        st = PipelineStage(cfg, pp_group, device, micro_batches, seed=seed, dtype=dtype,
                           train_cfg=tc, schedule=schedule, transport=transport or "nccl",
                           dp_group=dp_group)

    def feed(ids, targets):
        per = ids.shape[0] // dp
        sl = slice(d_idx * per, (d_idx + 1) * per)
        M = micro_batches
        b = per // M
        return st.train_step(ids[sl].reshape(M, b, -1), targets[sl].reshape(M, b, -1))
    return ParallelRun("dp+pp", st, getattr(st, "model", None) or st.models[0], rank, world, feed)
