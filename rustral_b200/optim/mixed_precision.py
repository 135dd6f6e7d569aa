"""Mixed-precision training: dynamic loss scaling and an optimizer wrapper with fp32 master weights
(crates/optim/src/mixed_precision.rs).

Differences from the reference, on purpose: gradients are UNSCALED (divided by the loss scale) before the inner
step (the reference multiplies them); the overflow check runs on the device; bf16 parameters keep fp32 master
weights as well (the reference skips them for bf16).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch

from .. import ops
from .optimizers import Adam, Optimizer


class DType(enum.Enum):
    FLOAT32 = "f32"
    FLOAT16 = "f16"
    BFLOAT16 = "bf16"


class LossScaleScheduler:
    """scale 1024, x2 every 2000 clean steps, x0.5 on overflow, floor 1."""

    def __init__(self, initial_scale: float = 1024.0, min_scale: float = 1.0, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000, max_scale: float = 2.0 ** 24):
        self.scale = initial_scale
        self.min_scale, self.max_scale = min_scale, max_scale
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self.good_steps = 0
        self.overflows = 0

    def step(self, has_overflow: bool) -> bool:
        """Returns True when the optimizer step must be skipped."""
        if has_overflow:
            self.scale = max(self.min_scale, self.scale * self.backoff_factor)
            self.good_steps = 0
            self.overflows += 1
            return True
        self.good_steps += 1
        if self.good_steps >= self.growth_interval:
            self.scale = min(self.max_scale, self.scale * self.growth_factor)
            self.good_steps = 0
        return False


@dataclass
class MixedPrecisionStats:
    dtype: str
    bytes_per_param: int
    master_bytes_per_param: int
    speedup_estimate: float

    @classmethod
    def for_dtype(cls, dt: DType):
        if dt is DType.FLOAT32:
            return cls("f32", 4, 0, 1.0)
        return cls(dt.value, 2, 4, 2.0)


class MixedPrecisionOptimizer(Optimizer):
    def __init__(self, inner: Optimizer | None = None, dtype: DType = DType.BFLOAT16,
                 loss_scale: LossScaleScheduler | None = None, check_overflow: bool = True):
        self.inner = inner or Adam()
        self.dtype = dtype
        self.loss_scale = loss_scale or LossScaleScheduler(1.0 if dtype is DType.BFLOAT16 else 1024.0)
        self.check_overflow = check_overflow
        self.skipped_steps = 0
        self.lr = self.inner.lr

    def set_lr(self, lr):
        self.lr = self.inner.lr = lr

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.loss_scale.scale

    def step(self, params, gradients=None, ctx=None) -> bool:
        """Returns False when the step was skipped because of an overflow."""
        params = list(params)
        grads = {}
        found = torch.zeros((), dtype=torch.int32, device=params[0].tensor.device)
        inv = 1.0 / self.loss_scale.scale
        for p in params:
            g = self.inner._grad_of(p, gradients)
            if g is None:
                continue
            if self.check_overflow:
                ops.sumsq(g, found_inf=found)
            grads[p.id] = g if inv == 1.0 else ops.scalar_op("mul_scalar", g, inv)
        overflow = bool(int(found)) if self.check_overflow else False
        if self.loss_scale.step(overflow):
            self.skipped_steps += 1
            return False
        self.inner.step(params, grads, ctx)
        return True
