"""Flow-matching Euler scheduler with the resolution-dependent time shift (src/models/flux/scheduler.rs)."""
from __future__ import annotations

import math

import torch


def empirical_mu(image_seq_len: int, num_steps: int) -> float:
    """The shift parameter as a linear fit in the number of image tokens, blended between the 10-step and 200-step fits by the
    step count; long sequences use the 200-step line alone."""
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return a2 * image_seq_len + b2
    m200, m10 = a2 * image_seq_len + b2, a1 * image_seq_len + b1
    a = (m200 - m10) / 190.0
    return a * num_steps + (m200 - 200.0 * a)


class FlowMatchEuler:
    """``sigmas = shift(linspace(1, 1 / N, N))`` with ``shift(s) = e^mu / (e^mu + (1 / s - 1))``, a terminal 0 appended; one step is
    ``x <- x + (sigma_next - sigma) * v``.  The model is queried at ``t = sigma``."""

    def __init__(self, num_steps: int, image_seq_len: int, mu: float | None = None):
        mu = empirical_mu(image_seq_len, num_steps) if mu is None else mu
        s = torch.linspace(1.0, 1.0 / num_steps, num_steps, dtype=torch.float64)
        s = math.exp(mu) / (math.exp(mu) + (1.0 / s - 1.0))
        self.sigmas = torch.cat([s, torch.zeros(1, dtype=torch.float64)]).float()
        self.num_steps, self.index = num_steps, 0

    @property
    def t(self) -> float:
        return float(self.sigmas[self.index])

    def step(self, velocity, sample):
        dt = self.sigmas[self.index + 1] - self.sigmas[self.index]
        self.index += 1
        return sample + dt.to(sample.dtype) * velocity
