#!/usr/bin/env python
"""Linear noise schedule, a deterministic DDPM-style sampler and a toy denoiser over a slice view
(counterpart of examples/diffusion_example.rs)."""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import DiffusionSampler, NoiseSchedule, SliceView


class LinearNoiseSchedule(NoiseSchedule):
    def __init__(self, steps: int = 50, beta_start: float = 1e-4, beta_end: float = 0.02) -> None:
        self.betas = [beta_start + (beta_end - beta_start) * i / max(1, steps - 1) for i in range(steps)]
        self.alpha_bars, acc = [], 1.0
        for b in self.betas:
            acc *= 1.0 - b
            self.alpha_bars.append(acc)

    def num_steps(self) -> int:
        return len(self.betas)

    def beta(self, timestep: int) -> float:
        return self.betas[timestep]

    def alpha_bar(self, timestep: int) -> float:
        return self.alpha_bars[timestep]


class DDPMSampler(DiffusionSampler):
    """Posterior mean step with a seeded pseudo-noise term, so runs repeat exactly."""

    def sample_step(self, current, predicted_noise, timestep, noise_schedule):
        beta, ab = noise_schedule.beta(timestep), noise_schedule.alpha_bar(timestep)
        alpha = 1.0 - beta
        out = []
        for i, (x, e) in enumerate(zip(current, predicted_noise)):
            mean = (x - beta / math.sqrt(1.0 - ab) * e) / math.sqrt(alpha)
            noise = math.sin(12.9898 * (i + 1) + 78.233 * timestep) if timestep > 0 else 0.0
            out.append(mean + math.sqrt(beta) * 0.1 * noise)
        return out

    def is_deterministic(self) -> bool:
        return True


def toy_denoiser(x, timestep: int, target):
    """Predicts the noise as the offset from a known clean signal (stands in for a network)."""
    return [xi - ti for xi, ti in zip(x, target)]


def main(steps: int = 50) -> dict:
    sched = LinearNoiseSchedule(steps)
    sampler = DDPMSampler()
    target = [math.sin(0.3 * i) for i in range(16)]
    x = [math.cos(1.7 * i) * 2.0 for i in range(16)]
    start = sum((a - b) ** 2 for a, b in zip(x, target)) / 16
    for t in reversed(range(sched.num_steps())):
        x = sampler.sample_step(x, toy_denoiser(x, t, target), t, sched)
    end = sum((a - b) ** 2 for a, b in zip(x, target)) / 16
    view = SliceView.new(x)
    print(f"mse to the clean signal: {start:.3f} -> {end:.5f}")
    return {"start_mse": start, "end_mse": end, "alpha_bar_last": sched.alpha_bar(steps - 1),
            "deterministic": sampler.is_deterministic(), "view_len": len(view)}


if __name__ == "__main__":
    print(main())
