"""Plain SGD with momentum (``Optimizer::SGD{momentum}``, src/domain/training/mod.rs:23-27; the
update rule the reference's training example applies by hand, examples/training_example.rs:206-213)."""
from __future__ import annotations

from typing import Optional

import torch


class SGD:
    def __init__(self, lr: float = 0.01, momentum: float = 0.0) -> None:
        self.lr, self.momentum = lr, momentum
        self.buf: Optional[torch.Tensor] = None
        self.step_count = 0

    def get_step(self) -> int:
        return self.step_count

    def increment_step(self) -> None:
        self.step_count += 1

    def learning_rate(self) -> float:
        return self.lr

    def set_learning_rate(self, lr: float) -> None:
        self.lr = lr

    def reset(self) -> None:
        self.buf = None
        self.step_count = 0

    def step(self, p32: torch.Tensor, g32: torch.Tensor, p16: Optional[torch.Tensor] = None,
             grad_scale: float = 1.0) -> None:
        self.step_count += 1
        g = g32 * grad_scale
        if self.momentum:
            if self.buf is None:
                self.buf = torch.zeros_like(p32)
            self.buf.mul_(self.momentum).add_(g)
            g = self.buf
        p32.add_(g, alpha=-self.lr)
        if p16 is not None:
            p16.copy_(p32)
