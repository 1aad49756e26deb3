"""Train the decoder as a ``torch.nn.Module``: autograd over the framework's kernels and the flat
AdamW kernel behind the module's parameters.

    python examples/autograd_training.py --steps 30

The explicit :class:`coeus_b200.models.decoder.DecoderLM` (no autograd graph, flat buffers, fused
data-parallel step) is what the benchmarks use; this is the path for models assembled from the
``coeus_b200.nn`` layers.  The reference's training example is a toy regression with hand-written
gradients (examples/training_example.rs:64-103)."""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.nn import TransformerLM
    from coeus_b200.optim.adamw import AdamWConfig
    from coeus_b200.optim.lr import WarmupCosine
    from coeus_b200.optim.module import ModuleAdamW
    cfg = DecoderConfig(hidden_dim=128, num_layers=2, num_heads=2, intermediate_dim=256,
                        vocab_size=256, max_seq_len=64, use_bias=False, activation="swiglu",
                        norm="rmsnorm", pos="rope")
    net = TransformerLM(cfg, device=a.device)
    opt = ModuleAdamW(net, AdamWConfig(lr=3e-3, weight_decay=0.01, grad_clip=1.0))
    sched = WarmupCosine(3e-3, 3, a.steps, floor=3e-4)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 256, (4, 64), generator=g).to(a.device)
    tgt = torch.roll(ids, -1, 1)
    losses = []
    for step in range(a.steps):
        opt.set_learning_rate(sched.at(step))
        opt.zero_grad()
        loss = net(ids, tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    out = {"first": losses[0], "last": losses[-1], "grad_norm": float(opt.grad_norm)}
    print(out)
    return out


if __name__ == "__main__":
    main()
