"""Replicated data parallelism: every rank keeps the full optimizer state, gradients are
all-reduced bucket by bucket while the backward pass is still running.

This is the plain comparator of :class:`coeus_b200.parallel.zero.ShardedDataParallel` (same
bucket plan, same hooks, library collectives, nothing sharded); it is what a stock
data-parallel wrapper does and costs ``world`` times the optimizer memory and update work of the
sharded step.  The reference is a single process and has no data parallelism.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..optim.adamw import AdamW, AdamWConfig
from .plans import Bucket, build_buckets


class ReplicatedDataParallel:
    """Drop-in for the ``dp`` argument of :class:`coeus_b200.train.trainer.Trainer`."""

    def __init__(self, group, device, overlap: bool = True) -> None:
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.overlap = overlap
        self.backend = "allreduce"
        self.sharded = False        # the trainer writes single-replica checkpoints from rank 0
        self.model = None
        self._grad_scale = 1.0
        self._pending: List = []

    # ------------------------------------------------------------------ set-up
    def attach(self, model, opt_cfg: AdamWConfig) -> None:
        self.model = model
        self.opt_cfg = opt_cfg
        self.buckets: List[Bucket] = build_buckets(model.layout, model.n_flat)
        self.by_trigger = {}
        for b in self.buckets:
            self.by_trigger.setdefault(b.trigger, []).append(b)
        self.opt = AdamW(opt_cfg, 0, model.n_flat, model.layout.decay_end, self.device)
        self.step_no = 0
        dist.broadcast(model.p32, src=dist.get_global_rank(self.group, 0), group=self.group)
        model.sync_working_copy()
        self.comm_stream = (torch.cuda.Stream(device=self.device)
                            if self.device.type == "cuda" else None)

    # ------------------------------------------------------------------ step protocol
    def set_grad_scale(self, s: float) -> None:
        self._grad_scale = s

    def begin_step(self) -> None:
        self.step_no += 1
        self._pending = []

    def _reduce(self, b: Bucket) -> None:
        g = self.model.g32[b.start:b.end]
        if self.comm_stream is None:
            self._pending.append(dist.all_reduce(g, group=self.group, async_op=True))
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            dist.all_reduce(g, group=self.group)

    def on_layer_done(self, trigger: int) -> None:
        if not self.overlap:
            return
        for b in self.by_trigger.get(trigger, []):
            self._reduce(b)

    def reduce_and_step(self, grad_scale: float) -> None:
        """Finish the all-reduces, then the same full AdamW step on every rank."""
        if not self.overlap:
            for b in self.buckets:
                self._reduce(b)
        for w in self._pending:
            w.wait()
        self._pending = []
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        m = self.model
        self.opt.cfg = self.opt_cfg          # a schedule may have changed the learning rate
        self.opt.step(m.p32, m.g32, m.p16, grad_scale)

    def finish(self) -> None:
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def gather_master(self) -> torch.Tensor:
        """Every rank holds the full master weights already."""
        self.finish()
        return self.model.p32.clone()
