"""Optimizers, learning-rate schedules and mixed-precision wrappers."""
from .optimizers import Optimizer, Sgd, Adam, AdamW, AdamState, AdamCheckpoint, Gradient, OptimError, MissingState
from .lr_scheduler import (LRScheduler, ConstantLR, LinearWarmup, CosineAnnealingLR, WarmupCosine, StepDecay,
                           ExponentialLR, PlateauLR, OneCycleLR, PolynomialLR)
from .mixed_precision import MixedPrecisionOptimizer, LossScaleScheduler, MixedPrecisionStats, DType

__all__ = [n for n in dir() if not n.startswith("_")]
