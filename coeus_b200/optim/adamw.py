"""AdamW over a flat fp32 master buffer (``csrc/elementwise.cu: adamw_kernel``).

The reference declares the optimizer only as data (``OptimizerState`` in src/core/model.rs:652-667
and ``Optimizer::Adam{beta1,beta2}`` in src/domain/training/mod.rs:23-27; its example never applies
the Adam state, examples/training_example.rs:206-213).  This is the update rule behind those
names: decoupled weight decay on the ``[0, decay_end)`` range of the flat buffer (the matrices),
none on the rest (biases and norm scales), bias-corrected moments, one pass that also refreshes
the bf16 working copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import elementwise as E


@dataclass
class AdamWConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    grad_clip: Optional[float] = None


class AdamW:
    """Optimizer state for the index range ``[start, end)`` of a flat parameter buffer (the whole
    buffer on one GPU, this rank's shard under sharded data parallelism)."""

    def __init__(self, cfg: AdamWConfig, start: int, end: int, decay_end: int, device) -> None:
        self.cfg = cfg
        self.start, self.end, self.decay_end = start, end, decay_end
        n = end - start
        self.m = torch.zeros(n, dtype=torch.float32, device=device)
        self.v = torch.zeros(n, dtype=torch.float32, device=device)
        self.step_count = 0
        # ``norm_hook(g32, sumsq)``: turns this rank's sum of squared gradients into the global one
        # in place (tensor / pipeline / expert parallelism, where ranks hold different tensors)
        self.norm_hook = None
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=device)

    # OptimizerState trait (src/core/model.rs:652-667)
    def get_step(self) -> int:
        return self.step_count

    def increment_step(self) -> None:
        self.step_count += 1

    def learning_rate(self) -> float:
        return self.cfg.lr

    def set_learning_rate(self, lr: float) -> None:
        self.cfg.lr = lr

    def reset(self) -> None:
        self.m.zero_()
        self.v.zero_()
        self.step_count = 0

    def _ranges(self):
        """(global_start, global_end, weight_decay) pieces of this optimizer's range."""
        s, e, d = self.start, self.end, self.decay_end
        if s < min(e, d):
            yield s, min(e, d), self.cfg.weight_decay
        if max(s, d) < e:
            yield max(s, d), e, 0.0

    def compute_clip(self, g32: torch.Tensor, grad_scale: float) -> None:
        """Global-norm clipping coefficient from this range's gradients (single rank)."""
        self.sumsq.zero_()
        E.sumsq_into(g32[self.start:self.end], self.sumsq)
        if self.norm_hook is not None:      # model-parallel trainers complete the sum over ranks
            self.norm_hook(g32, self.sumsq)
        E.clip_coef_from_sumsq(self.sumsq, grad_scale, self.cfg.grad_clip, self.clip_coef,
                               self.grad_norm)

    def step(self, p32: torch.Tensor, g32: torch.Tensor, p16: Optional[torch.Tensor],
             grad_scale: float = 1.0) -> None:
        """One update of ``p32[start:end]`` from ``g32[start:end]``; refreshes ``p16``."""
        c = self.cfg
        self.step_count += 1
        if c.grad_clip is not None:
            self.compute_clip(g32, grad_scale)
        for s, e, wd in self._ranges():
            lo, hi = s - self.start, e - self.start
            E.adamw_step(p32[s:e], self.m[lo:hi], self.v[lo:hi], g32[s:e],
                         None if p16 is None else p16[s:e], lr=c.lr, beta1=c.beta1,
                         beta2=c.beta2, eps=c.eps, weight_decay=wd, step=self.step_count,
                         grad_scale=grad_scale,
                         clip_coef=self.clip_coef if c.grad_clip is not None else None)

    def state_dict(self) -> Dict[str, object]:
        return {"m": self.m, "v": self.v, "step": self.step_count, "start": self.start,
                "end": self.end}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
