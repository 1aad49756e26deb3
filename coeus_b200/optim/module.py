"""AdamW for ``torch.nn.Module`` models (the autograd layers of :mod:`coeus_b200.nn`): the
module's parameters are re-pointed at views of ONE flat working buffer, fp32 master weights and
moments live beside it, and a step is one pass of the flat AdamW kernel (master update + working
copy refresh) after the gradients have been gathered into a flat fp32 buffer.  The reference's
``OptimizerState`` (src/core/model.rs:652-667) is state only; its examples update parameters in
plain loops (examples/training_example.rs:206-213)."""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

from .adamw import AdamW, AdamWConfig


class ModuleAdamW:
    def __init__(self, module: torch.nn.Module, cfg: Optional[AdamWConfig] = None,
                 no_decay: Optional[Callable[[str, torch.nn.Parameter], bool]] = None,
                 group=None) -> None:
        """``no_decay(name, param)`` selects parameters without weight decay (default: vectors,
        i.e. biases and norm scales).  ``group``: data-parallel process group; the flat gradient
        buffer is averaged over it with one all-reduce per step and the replicas start from the
        first rank's weights."""
        self.cfg = cfg or AdamWConfig()
        no_decay = no_decay or (lambda name, p: p.dim() < 2)
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("the module has no trainable parameters")
        dev, dt = named[0][1].device, named[0][1].dtype
        decay = [(n, p) for n, p in named if not no_decay(n, p)]
        plain = [(n, p) for n, p in named if no_decay(n, p)]
        self.params: List[Tuple[str, torch.nn.Parameter, int]] = []
        off = 0
        for part in (decay, plain):
            for n, p in part:
                self.params.append((n, p, off))
                off += (p.numel() + 7) // 8 * 8          # the kernel works on 16-byte groups
            if part is decay:
                self.decay_end = off
        self.n = max(off, 8)
        self.p32 = torch.zeros(self.n, dtype=torch.float32, device=dev)
        self.p16 = torch.zeros(self.n, dtype=dt, device=dev)
        self.g32 = torch.zeros(self.n, dtype=torch.float32, device=dev)
        for _, p, o in self.params:
            self.p32[o:o + p.numel()].copy_(p.detach().reshape(-1))
            self.p16[o:o + p.numel()].copy_(p.detach().reshape(-1))
            p.data = self.p16[o:o + p.numel()].view(p.shape)   # the module now reads the flat copy
        self.opt = AdamW(self.cfg, 0, self.n, self.decay_end, dev)
        self.group = group
        self.world = 1
        if group is not None:
            import torch.distributed as dist
            self.world = dist.get_world_size(group)
            dist.broadcast(self.p32, src=dist.get_global_rank(group, 0), group=group)
            self.p16.copy_(self.p32)

    def zero_grad(self) -> None:
        for _, p, _ in self.params:
            p.grad = None

    def set_learning_rate(self, lr: float) -> None:
        self.opt.set_learning_rate(lr)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.g32.zero_()
        for _, p, o in self.params:
            if p.grad is not None:
                self.g32[o:o + p.numel()].copy_(p.grad.reshape(-1))
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(self.g32, group=self.group)
        self.opt.step(self.p32, self.g32, self.p16, grad_scale / self.world)

    @property
    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step (when ``grad_clip`` is set)."""
        return self.opt.grad_norm
