#!/usr/bin/env python
"""Two training loops.

1. The reference's toy (examples/training_example.rs): a sine predictor implementing the
   ``TrainableModel`` trait with ``MSELoss``, batches of 16 from the iterator adapters, ten epochs.
2. What the reference has no code for: a decoder language model trained with the framework's
   trainer (forward, backward, AdamW on the kernels; ``--device cuda`` for the GPU path)."""
import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from coeus_b200.prelude import Iter, MSELoss, TrainableModel


class SinePredictor(TrainableModel):
    """y = a * sin(b * x + c) fitted by gradient descent on (a, b, c)."""

    def __init__(self) -> None:
        self.params = [0.5, 0.8, 0.1]
        self._training = True
        self.loss = MSELoss()

    def name(self) -> str:
        return "sine-predictor"

    def config(self):
        return None

    def num_parameters(self) -> int:
        return 3

    def forward(self, xs):
        a, b, c = self.params
        return [a * math.sin(b * x + c) for x in xs]

    def compute_loss(self, data) -> float:
        xs, ys = data
        return self.loss.compute(self.forward(xs), ys)

    def train_step(self, data, lr: float) -> float:
        xs, ys = data
        a, b, c = self.params
        pred = self.forward(xs)
        g = self.loss.gradient(pred, ys)
        ga = sum(gi * math.sin(b * x + c) for gi, x in zip(g, xs))
        gb = sum(gi * a * math.cos(b * x + c) * x for gi, x in zip(g, xs))
        gc = sum(gi * a * math.cos(b * x + c) for gi, x in zip(g, xs))
        self.update_parameters([lr * ga, lr * gb, lr * gc])
        return self.loss.compute(pred, ys)

    def update_parameters(self, gradients) -> None:
        self.params = [p - g for p, g in zip(self.params, gradients)]

    def is_training(self) -> bool:
        return self._training

    def set_training(self, training: bool) -> None:
        self._training = training


def toy(epochs: int = 10) -> list:
    xs = [i * 0.02 for i in range(320)]
    ys = [math.sin(x) for x in xs]
    model = SinePredictor()
    history = []
    for _ in range(epochs):
        tot, n = 0.0, 0
        for batch in Iter(list(zip(xs, ys))).batch(16, 16):
            bx, by = [p[0] for p in batch], [p[1] for p in batch]
            tot += model.train_step((bx, by), 0.02)
            n += 1
        history.append(tot / n)
    return history


def language_model(device: str = "cpu", steps: int = 20) -> list:
    from coeus_b200.models.config import DecoderConfig
    from coeus_b200.models.decoder import DecoderLM
    from coeus_b200.train.trainer import TrainConfig, Trainer
    cuda = device == "cuda"
    cfg = DecoderConfig(hidden_dim=128 if cuda else 32, num_layers=2, num_heads=2,
                        intermediate_dim=256 if cuda else 64, vocab_size=256, max_seq_len=64)
    model = DecoderLM(cfg, device, seed=0, dtype=torch.bfloat16 if cuda else torch.float32)
    trainer = Trainer(model, TrainConfig(learning_rate=3e-3))
    gen = torch.Generator().manual_seed(0)
    data = torch.randint(0, 256, (8, 65), generator=gen).to(device)      # one batch, memorised
    x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
    return [float(trainer.train_step(x, y)) for _ in range(steps)]


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=20)
    a = ap.parse_args(argv)
    h = toy()
    print("toy: loss %.4f -> %.4f" % (h[0], h[-1]))
    lm = language_model(a.device, a.steps)
    print("language model: loss %.3f -> %.3f" % (lm[0], lm[-1]))
    return {"toy": h, "lm": lm}


if __name__ == "__main__":
    main()
