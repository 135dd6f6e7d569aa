"""Learning-rate schedulers (crates/optim/src/lr_scheduler.rs): nine standalone schedules with the interface
get_lr(step) / current_lr() / step() / reset() / name().  `attach(optimizer)` couples one to an optimizer's lr."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self):
        self._step = 0
        self._opt = None

    def get_lr(self, step: int) -> float:
        raise NotImplementedError

    def current_lr(self) -> float:
        return self.get_lr(self._step)

    def step(self) -> float:
        self._step += 1
        lr = self.current_lr()
        if self._opt is not None:
            self._opt.set_lr(lr)
        return lr

    def reset(self) -> None:
        self._step = 0

    def name(self) -> str:
        return type(self).__name__

    def attach(self, optimizer):
        self._opt = optimizer
        optimizer.set_lr(self.current_lr())
        return self


class ConstantLR(LRScheduler):
    def __init__(self, lr: float):
        super().__init__()
        self.lr = lr

    def get_lr(self, step):
        return self.lr


class LinearWarmup(LRScheduler):
    def __init__(self, initial_lr: float, peak_lr: float, warmup_steps: int):
        super().__init__()
        self.initial, self.peak, self.warmup = initial_lr, peak_lr, max(1, warmup_steps)

    def get_lr(self, step):
        if step >= self.warmup:
            return self.peak
        return self.initial + (self.peak - self.initial) * step / self.warmup


class CosineAnnealingLR(LRScheduler):
    def __init__(self, initial_lr: float, min_lr: float, total_steps: int):
        super().__init__()
        self.initial, self.min, self.total = initial_lr, min_lr, max(1, total_steps)

    def get_lr(self, step):
        t = min(step, self.total) / self.total
        return self.min + 0.5 * (self.initial - self.min) * (1 + math.cos(math.pi * t))


class WarmupCosine(LRScheduler):
    def __init__(self, peak_lr: float, min_lr: float, warmup_steps: int, total_steps: int, initial_lr: float = 0.0):
        super().__init__()
        self.peak, self.min, self.warmup, self.total, self.initial = peak_lr, min_lr, warmup_steps, total_steps, initial_lr

    def with_initial_lr(self, lr: float):
        self.initial = lr
        return self

    def get_lr(self, step):
        if self.warmup > 0 and step < self.warmup:
            return self.initial + (self.peak - self.initial) * step / self.warmup
        span = max(1, self.total - self.warmup)
        t = min(max(step - self.warmup, 0), span) / span
        return self.min + 0.5 * (self.peak - self.min) * (1 + math.cos(math.pi * t))


class StepDecay(LRScheduler):
    def __init__(self, initial_lr: float, factor: float, step_size: int):
        super().__init__()
        self.initial, self.factor, self.step_size = initial_lr, factor, max(1, step_size)

    def get_lr(self, step):
        return self.initial * (self.factor ** (step // self.step_size))


class ExponentialLR(LRScheduler):
    def __init__(self, initial_lr: float, decay_rate: float):
        super().__init__()
        self.initial, self.rate = initial_lr, decay_rate

    def get_lr(self, step):
        return self.initial * math.exp(-self.rate * step)


class PlateauLR(LRScheduler):
    """Reduce on plateau: `report_loss` drives it; lr is multiplied by `factor` after `patience` non-improving
    reports, never below `min_lr`, with an optional cooldown."""

    def __init__(self, initial_lr: float, min_lr: float = 0.0, factor: float = 0.5, patience: int = 5, cooldown: int = 0,
                 threshold: float = 1e-4):
        super().__init__()
        self.initial = self.lr = initial_lr
        self.min, self.factor, self.patience, self.cooldown, self.threshold = min_lr, factor, patience, cooldown, threshold
        self.best = float("inf")
        self.bad = 0
        self.cool = 0

    def report_loss(self, loss: float) -> float:
        if loss < self.best - self.threshold:
            self.best, self.bad = loss, 0
        elif self.cool > 0:
            self.cool -= 1
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.lr = max(self.min, self.lr * self.factor)
                self.bad, self.cool = 0, self.cooldown
        if self._opt is not None:
            self._opt.set_lr(self.lr)
        return self.lr

    def get_lr(self, step):
        return self.lr

    def reset(self):
        super().reset()
        self.lr, self.best, self.bad, self.cool = self.initial, float("inf"), 0, 0


class OneCycleLR(LRScheduler):
    """Linear rise from max/10 to max over the first half, cosine fall back to max/10 over the second."""

    def __init__(self, max_lr: float, total_steps: int):
        super().__init__()
        self.max, self.total = max_lr, max(2, total_steps)
        self.min = max_lr / 10.0

    def get_lr(self, step):
        half = self.total // 2
        if step <= half:
            return self.min + (self.max - self.min) * step / half
        t = min(step - half, self.total - half) / (self.total - half)
        return self.min + 0.5 * (self.max - self.min) * (1 + math.cos(math.pi * t))


class PolynomialLR(LRScheduler):
    def __init__(self, initial_lr: float, min_lr: float, total_steps: int, power: float = 1.0):
        super().__init__()
        self.initial, self.min, self.total, self.power = initial_lr, min_lr, max(1, total_steps), power

    def get_lr(self, step):
        t = min(step, self.total) / self.total
        return self.min + (self.initial - self.min) * (1 - t) ** self.power
