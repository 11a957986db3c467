"""Learning-rate schedulers (crates/incin-core/src/optim/scheduler.rs:9-134): ConstantLR, LinearLR,
CosineAnnealingLR, StepLR.  A scheduler maps a step index to a learning rate and pushes it into the
optimiser; its state (the step counter) is part of the trainer checkpoint here."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, optimizer, base_lr: float | None = None):
        self.optimizer = optimizer
        self.base_lr = float(base_lr if base_lr is not None else optimizer.lr)
        self.last_step = 0

    def lr_at(self, step: int) -> float:
        raise NotImplementedError

    def step(self) -> float:
        self.last_step += 1
        lr = self.lr_at(self.last_step)
        self.optimizer.set_lr(lr)
        return lr

    def state_dict(self) -> dict:
        return {"last_step": self.last_step, "base_lr": self.base_lr}

    def load_state_dict(self, sd: dict) -> None:
        self.last_step, self.base_lr = int(sd["last_step"]), float(sd["base_lr"])
        self.optimizer.set_lr(self.lr_at(self.last_step))


class ConstantLR(LRScheduler):
    def lr_at(self, step):
        return self.base_lr


class LinearLR(LRScheduler):
    """Linear ramp from ``start_factor * base`` to ``end_factor * base`` over ``total_steps`` (warm-up / decay)."""

    def __init__(self, optimizer, start_factor: float = 0.0, end_factor: float = 1.0, total_steps: int = 100, base_lr=None):
        super().__init__(optimizer, base_lr)
        self.start_factor, self.end_factor, self.total_steps = start_factor, end_factor, max(1, total_steps)

    def lr_at(self, step):
        t = min(step, self.total_steps) / self.total_steps
        return self.base_lr * (self.start_factor + (self.end_factor - self.start_factor) * t)


class CosineAnnealingLR(LRScheduler):
    def __init__(self, optimizer, t_max: int, eta_min: float = 0.0, base_lr=None):
        super().__init__(optimizer, base_lr)
        self.t_max, self.eta_min = max(1, t_max), eta_min

    def lr_at(self, step):
        t = min(step, self.t_max)
        return self.eta_min + (self.base_lr - self.eta_min) * 0.5 * (1.0 + math.cos(math.pi * t / self.t_max))


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1, base_lr=None):
        super().__init__(optimizer, base_lr)
        self.step_size, self.gamma = max(1, step_size), gamma

    def lr_at(self, step):
        return self.base_lr * self.gamma ** (step // self.step_size)
