"""Trainer: one object that owns the model, the optimizer state and the data-parallel plan and
runs whole training steps.

It keeps the shape of the reference's ``TrainableModel`` trait (``train_step``,
``update_parameters``, ``compute_loss``, ``is_training``, ``set_training``;
src/core/model.rs:107-131) and of its example loop (examples/training_example.rs:257-276), and
supplies what the reference leaves out: a real backward pass, AdamW, and sharded data
parallelism over NVLink.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..foundation.error import ProcessingError
from ..models.decoder import DecoderLM
from ..optim.adamw import AdamW, AdamWConfig


@dataclass
class TrainConfig:
    """Counterpart of the reference's ``TrainingConfig{learning_rate, batch_size, epochs}``
    (src/domain/training/mod.rs:14-20) with the fields a real step needs."""

    learning_rate: float = 3e-4
    batch_size: int = 8
    epochs: int = 1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    grad_clip: Optional[float] = None
    grad_accum: int = 1

    def adamw(self) -> AdamWConfig:
        return AdamWConfig(self.learning_rate, self.beta1, self.beta2, self.eps,
                           self.weight_decay, self.grad_clip)


class Trainer:
    def __init__(self, model: DecoderLM, cfg: Optional[TrainConfig] = None, dp=None,
                 schedule=None) -> None:
        """``dp`` is a :class:`coeus_b200.parallel.zero.ShardedDataParallel` (or ``None`` for a
        single replica); ``schedule`` an object with ``at(step) -> lr``
        (:mod:`coeus_b200.optim.lr`) applied before every optimizer step."""
        self.model = model
        self.cfg = cfg or TrainConfig()
        self.dp = dp
        self.schedule = schedule
        self._micro = 0
        self._training = True
        self.step_index = 0
        self.listeners: List[Callable[[dict], None]] = []
        if dp is None:
            self.opt = AdamW(self.cfg.adamw(), 0, model.n_flat, model.layout.decay_end,
                             model.device)
        else:
            dp.attach(model, self.cfg.adamw())
            self.opt = dp.opt

    # ---- TrainableModel surface
    def is_training(self) -> bool:
        return self._training

    def set_training(self, training: bool) -> None:
        self._training = training

    def compute_loss(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        return self.model.forward_loss(ids, targets)

    def evaluate(self, batches) -> Dict[str, float]:
        """Mean next-token loss and perplexity over ``(ids, targets)`` batches without touching
        gradients or optimizer state (token-weighted; averaged over the data-parallel group when
        there is one)."""
        import math
        m = self.model
        tot = torch.zeros(2, dtype=torch.float64, device=m.device)
        was_training, m.train_mode = getattr(m, "train_mode", True), False   # no dropout
        for ids, targets in batches:
            n = int((targets >= 0).sum())
            loss = m.forward_loss(ids, targets)
            m._saved = None                       # nothing is kept for a backward pass
            tot[0] += float(loss) * targets.numel()
            tot[1] += n
        if self.dp is not None and self.dp.world > 1:
            import torch.distributed as dist
            dist.all_reduce(tot, group=self.dp.group)
        m.train_mode = was_training
        mean = float(tot[0] / tot[1].clamp_min(1))
        return {"loss": mean, "perplexity": math.exp(min(mean, 80.0)), "tokens": int(tot[1])}

    def update_parameters(self, grad_scale: float = 1.0) -> None:
        m = self.model
        if self.dp is None:
            self.opt.step(m.p32, m.g32, m.p16, grad_scale)
        else:
            self.dp.reduce_and_step(grad_scale)

    def _set_lr(self, lr: float) -> None:
        if self.dp is None:
            self.opt.set_learning_rate(lr)
        else:
            self.dp.opt_cfg.lr = lr

    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Forward and backward for one micro-batch per rank and, on every ``grad_accum``-th call,
        the optimizer update (gradients of the calls in between are summed, each scaled by
        ``1 / grad_accum``); returns the rank-local mean loss as a device scalar."""
        m = self.model
        world = 1 if self.dp is None else self.dp.world
        accum = max(1, self.cfg.grad_accum)
        first, last = self._micro == 0, self._micro == accum - 1
        if first:
            if self.schedule is not None:
                self._set_lr(self.schedule.at(self.step_index))
            if self.dp is not None:
                self.dp.set_grad_scale(1.0 / world)
                self.dp.begin_step()
            m.zero_grad()
        T = ids.numel()
        loss = m.forward_loss(ids, targets, grad_scale=1.0 / (T * accum))
        # the bucket reductions of the data-parallel plan start only in the last micro-step
        hook = self.dp.on_layer_done if (self.dp is not None and last) else None
        m.backward(on_layer_done=hook)
        self._micro = (self._micro + 1) % accum
        if last:
            self.update_parameters(1.0 / world)
            self.step_index += 1
            m.dropout_step = self.step_index      # the next step draws new dropout masks
        return loss

    # ---- Checkpoint trait (src/core/traits.rs:181-189)
    def state_dict(self) -> Dict[str, object]:
        return {"p32": self.model.p32, "opt": self.opt.state_dict(), "step": self.step_index}

    def checkpoint(self) -> bytes:
        """Single-replica training state as one byte string: a JSON header line, then the fp32
        master weights and the two Adam moments (``Checkpoint::checkpoint``,
        src/core/traits.rs:181-189).  Sharded runs use :meth:`save_checkpoint`."""
        import json
        if self.dp is not None:
            raise ProcessingError.unsupported(
                "Trainer.checkpoint() under data parallelism", "use save_checkpoint(directory)")
        m = self.model
        head = {"n_flat": m.n_flat, "opt_step": self.opt.step_count, "train_step": self.step_index,
                "micro": self._micro, "config": m.cfg.to_dict()}
        parts = [json.dumps(head).encode() + b"\n"]
        for t in (m.p32, self.opt.m, self.opt.v):
            parts.append(t.detach().cpu().numpy().tobytes())
        return b"".join(parts)

    def restore(self, checkpoint: bytes) -> None:
        """Inverse of :meth:`checkpoint` (``Checkpoint::restore``)."""
        import json

        import numpy as np
        m = self.model
        nl = checkpoint.index(b"\n")
        head = json.loads(checkpoint[:nl].decode())
        n = int(head["n_flat"])
        if n != m.n_flat or len(checkpoint) != nl + 1 + 12 * n:
            raise ProcessingError.invalid_input(
                f"checkpoint holds {n} parameters, the model {m.n_flat}")
        body = np.frombuffer(checkpoint, dtype=np.float32, count=3 * n, offset=nl + 1)
        for j, t in enumerate((m.p32, self.opt.m, self.opt.v)):
            t.copy_(torch.from_numpy(body[j * n:(j + 1) * n].copy()))
        m.sync_working_copy()
        self.opt.step_count = int(head["opt_step"])
        self.step_index = int(head["train_step"])
        self._micro = int(head.get("micro", 0))

    # ---- sharded checkpoints (resume on any number of ranks)
    def _sharded(self) -> bool:
        """Whether optimizer state is split over the data-parallel ranks (else every rank holds
        all of it and rank 0 writes the checkpoint of a single replica)."""
        return self.dp is not None and getattr(self.dp, "sharded", True)

    def _owned_segments(self):
        m = self.model
        if not self._sharded():
            return [(0, m.n_flat)]
        return [b.shard(self.dp.rank, self.dp.world) for b in self.dp.buckets]

    def _moment_view(self, name: str, s: int, e: int) -> torch.Tensor:
        """The ``[s, e)`` slice of Adam's ``m`` or ``v`` (flat coordinates)."""
        if not self._sharded():
            return getattr(self.opt, name)[s:e]
        for b, off in zip(self.dp.buckets, self.dp.moffs):
            bs, be = b.shard(self.dp.rank, self.dp.world)
            if bs <= s and e <= be:
                return getattr(self.opt, name)[off + s - bs: off + e - bs]
        raise KeyError(f"range [{s}, {e}) is not owned by this rank")

    def save_checkpoint(self, directory: str, data_cursor: int = 0, background: bool = False) -> None:
        """Write this rank's shard (fp32 master weights and Adam moments of the ranges it owns)
        and, on rank 0, the manifest.  ``background=True`` returns once the device-to-host copies
        are enqueued; :meth:`wait_checkpoint` finishes the job."""
        import random

        import torch.distributed as dist

        from ..checkpoint import sharded as S
        m = self.model
        if self.dp is not None:
            self.dp.finish()
        if self.dp is not None and not self._sharded():
            # replicated state: rank 0 writes the checkpoint of one replica, the others wait
            if self.dp.rank != 0:
                dist.barrier(group=self.dp.group)
                return
            rank, world = 0, 1
        else:
            rank = 0 if self.dp is None else self.dp.rank
            world = 1 if self.dp is None else self.dp.world

        def fetch(name, s, e):
            return m.p32[s:e] if name == "p32" else self._moment_view(name, s, e)

        meta = {"config": m.cfg.to_dict(), "n_flat": m.n_flat, "data_cursor": data_cursor,
                "opt_step": self.opt.step_count, "train_step": self.step_index,
                "python_rng": repr(random.getstate()[1][:4])}
        barrier = (lambda: dist.barrier(group=self.dp.group)) if self._sharded() else None
        if background and self.dp is not None and not self._sharded():
            background = False       # one writer; the other ranks are already at the barrier
        if background:
            if not hasattr(self, "_ckpt_writer"):
                self._ckpt_writer = S.AsyncWriter()
            self._ckpt_pending = (directory, world, self.step_index, meta, barrier, rank)
            S.save_shard(directory, rank, world, self._owned_segments(), fetch, self.step_index,
                         meta, writer=self._ckpt_writer)
        else:
            S.save_shard(directory, rank, world, self._owned_segments(), fetch, self.step_index,
                         meta, barrier=barrier)
        if self.dp is not None and not self._sharded():
            dist.barrier(group=self.dp.group)
        for fn in self.listeners:
            fn({"event": "PersistenceEvent::Saved", "path": directory, "step": self.step_index})

    def wait_checkpoint(self) -> None:
        """Finish a background save: join the writer, then write the manifest on rank 0."""
        from ..checkpoint import sharded as S
        pend = getattr(self, "_ckpt_pending", None)
        if pend is None:
            return
        directory, world, step, meta, barrier, rank = pend
        self._ckpt_writer.wait()
        if barrier is not None:
            barrier()
        if rank == 0:
            S.finalize_manifest(directory, world, step, meta)
        if barrier is not None:
            barrier()
        self._ckpt_pending = None

    def load_checkpoint(self, directory: str) -> dict:
        """Restore weights (all of them, every rank needs the full working copy) and the Adam
        moments of the ranges this rank owns now, whatever the world size at save time was."""
        from ..checkpoint import sharded as S
        m = self.model

        def put_w(name, s, e, t):
            m.p32[s:e].copy_(t)

        def put_m(name, s, e, t):
            self._moment_view(name, s, e).copy_(t)

        man = S.load_ranges(directory, [(0, m.n_flat)], put_w, state_names=("p32",))
        S.load_ranges(directory, self._owned_segments(), put_m, verify=False, state_names=("m", "v"))
        m.sync_working_copy()
        meta = man["meta"]
        self.opt.step_count = int(meta["opt_step"])
        self.step_index = int(meta["train_step"])
        return meta
