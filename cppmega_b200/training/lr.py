"""Learning-rate schedules: constant, linear warm-up + cosine / linear / WSD decay."""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class LRSchedule:
    lr: float = 1e-4
    min_lr: float = 0.0
    warmup_steps: int = 0
    decay_steps: int = 0            # 0 -> constant after warm-up
    style: str = "cosine"           # constant | cosine | linear | wsd
    wsd_decay_fraction: float = 0.1

    def __call__(self, step: int) -> float:
        if self.warmup_steps > 0 and step < self.warmup_steps:
            return self.lr * (step + 1) / self.warmup_steps
        if self.style == "constant" or self.decay_steps <= 0:
            return self.lr
        t = min(max(step - self.warmup_steps, 0), self.decay_steps) / self.decay_steps
        if self.style == "cosine":
            return self.min_lr + 0.5 * (self.lr - self.min_lr) * (1.0 + math.cos(math.pi * t))
        if self.style == "linear":
            return self.lr + (self.min_lr - self.lr) * t
        if self.style == "wsd":
            start = 1.0 - self.wsd_decay_fraction
            if t < start:
                return self.lr
            return self.lr + (self.min_lr - self.lr) * (t - start) / max(self.wsd_decay_fraction, 1e-12)
        raise ValueError(f"unknown lr style {self.style!r}")
