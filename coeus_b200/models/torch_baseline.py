"""Comparator arm: the same decoder on stock PyTorch (cuBLAS GEMMs, SDPA attention, fused torch
AdamW, ``DistributedDataParallel`` over NCCL).  Parameters are resident in bf16 by default, so no
step pays for casting weights (and the optimizer updates bf16 directly, without the fp32 master
copy this framework keeps: the comparator does strictly less work per step);
``resident="fp32"`` selects fp32 parameters under bf16 autocast instead.  None of this
framework's kernels are used here; it exists to be measured against."""
from __future__ import annotations

import torch
import torch.nn as nn

from . import torch_reference as R
from .config import DecoderConfig
from .decoder import ParamLayout


class TorchDecoder(nn.Module):
    def __init__(self, cfg: DecoderConfig, device, resident: str = "bf16") -> None:
        super().__init__()
        self.cfg = cfg
        self.resident = resident
        self.params = nn.ParameterDict()
        gen = torch.Generator(device=device)
        gen.manual_seed(0)
        for s in ParamLayout(cfg).specs:
            t = torch.empty(s.shape, dtype=torch.float32, device=device)
            if s.kind in ("weight", "embed"):
                t.normal_(0.0, cfg.init_std, generator=gen)
            elif s.kind == "scale":
                t.fill_(1.0)
            else:
                t.zero_()
            if resident == "bf16":
                t = t.to(torch.bfloat16)
            self.params[s.name.replace(".", "__")] = nn.Parameter(t)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        named = {k.replace("__", "."): v for k, v in self.params.items()}
        if self.resident == "bf16":
            return R.forward_loss(named, self.cfg, ids, targets)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return R.forward_loss(named, self.cfg, ids, targets)


class TorchBaseline:
    def __init__(self, cfg: DecoderConfig, device, world: int, resident: str = "bf16") -> None:
        self.module = TorchDecoder(cfg, device, resident)
        self.model = self.module
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            self.model = DDP(self.module, device_ids=[device.index], gradient_as_bucket_view=True)
        self.opt = torch.optim.AdamW(self.module.parameters(), lr=3e-4, betas=(0.9, 0.95),
                                     eps=1e-8, weight_decay=0.1, fused=True)

    def step(self, batch: torch.Tensor) -> torch.Tensor:
        self.opt.zero_grad(set_to_none=True)
        loss = self.model(batch[:, :-1], batch[:, 1:])
        loss.backward()
        self.opt.step()
        return loss.detach()
