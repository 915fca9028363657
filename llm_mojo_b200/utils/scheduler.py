"""Learning-rate schedules: cosine, linear, constant, WSD (``llmm/scheduler.mojo:25-113``)."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, scheduler_type: str, learning_rate: float, warmup_steps: int,
                 train_num_batches: int, final_learning_rate_fraction: float):
        if scheduler_type not in ("cosine", "linear", "constant", "wsd"):
            raise ValueError(f"Invalid scheduler type: {scheduler_type}")
        self.scheduler_type = scheduler_type
        self.learning_rate = learning_rate
        self.warmup_steps = warmup_steps
        self.train_num_batches = train_num_batches
        self.final_learning_rate_fraction = final_learning_rate_fraction

    def _warm(self, step: int) -> float:
        return self.learning_rate * (step + 1) / self.warmup_steps

    def get_learning_rate(self, step: int) -> float:
        lr, frac = self.learning_rate, self.final_learning_rate_fraction
        if self.scheduler_type == "constant":
            return lr
        if step < self.warmup_steps:
            return self._warm(step)
        min_lr = lr * frac
        if self.scheduler_type == "wsd":
            decay_point = self.train_num_batches * 4 // 5
            if step < decay_point:
                return lr
            ratio = (step - decay_point) / (self.train_num_batches - decay_point)
            return min_lr + (1.0 - math.sqrt(ratio)) * (lr - min_lr)
        ratio = (step - self.warmup_steps) / (self.train_num_batches - self.warmup_steps)
        if self.scheduler_type == "linear":
            return min_lr + ratio * (lr - min_lr)
        coeff = 0.5 * (1.0 + math.cos(math.pi * ratio))
        return min_lr + coeff * (lr - min_lr)
