"""LayerNorm, RMSNorm, BatchNorm (crates/nn/src/normalization.rs:10-310)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, ShapeMismatch


@dataclass
class LayerNormConfig:
    normalized_shape: int
    eps: float = 1e-5


class LayerNorm(Module, Trainable, Saveable):
    """Population variance, eps inside the square root; gamma starts at ones and beta at zeros (the reference
    draws gamma from uniform(-1, 1), crates/nn/src/normalization.rs:48-53, which is not what a LayerNorm wants)."""

    def __init__(self, config: LayerNormConfig, weight: Parameter, bias: Parameter):
        self.config = config
        self.weight, self.bias = weight, bias

    @classmethod
    def new(cls, backend, dim: int, eps: float = 1e-5):
        return cls(LayerNormConfig(dim, eps), backend.constant_parameter("weight", (dim,), 1.0),
                   backend.constant_parameter("bias", (dim,), 0.0))

    def forward(self, x, ctx: ForwardCtx):
        if x.shape[-1] != self.config.normalized_shape:
            raise ShapeMismatch((self.config.normalized_shape,), x.shape[-1:], "LayerNorm input")
        with ctx.profile("layer_norm", x.shape):
            return ops.layer_norm(x, self.weight.tensor, self.bias.tensor, self.config.eps)


class RMSNorm(Module, Trainable, Saveable):
    """y = x / sqrt(mean(x^2) + eps) * weight (Llama-style; absent from the reference, needed by its 8B config)."""

    def __init__(self, dim: int, weight: Parameter, eps: float = 1e-5):
        self.dim, self.eps = dim, eps
        self.weight = weight

    @classmethod
    def new(cls, backend, dim: int, eps: float = 1e-5):
        return cls(dim, backend.constant_parameter("weight", (dim,), 1.0), eps)

    def forward(self, x, ctx: ForwardCtx):
        with ctx.profile("rms_norm", x.shape):
            return ops.rms_norm(x, self.weight.tensor, self.eps)


@dataclass
class BatchNormConfig:
    num_features: int
    eps: float = 1e-5
    momentum: float = 0.1


class BatchNorm(Module, Trainable, Saveable):
    """Batch statistics in training, running statistics in inference; input [N, C] or [N, C, H, W].
    (The reference normalises with batch statistics in both modes, crates/nn/src/normalization.rs:206-310.)"""

    def __init__(self, config: BatchNormConfig, weight: Parameter, bias: Parameter):
        self.config = config
        self.weight, self.bias = weight, bias
        dev, dt = weight.tensor.device, torch.float32
        self._running_mean = torch.zeros(config.num_features, device=dev, dtype=dt)
        self._running_var = torch.ones(config.num_features, device=dev, dtype=dt)

    @classmethod
    def new(cls, backend, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        return cls(BatchNormConfig(num_features, eps, momentum), backend.constant_parameter("weight", (num_features,), 1.0),
                   backend.constant_parameter("bias", (num_features,), 0.0))

    def forward(self, x, ctx: ForwardCtx):
        c = self.config.num_features
        if x.dim() not in (2, 4) or x.shape[1] != c:
            raise ShapeMismatch(("N", c), x.shape, "BatchNorm input")
        dims = (0,) if x.dim() == 2 else (0, 2, 3)
        shape = (1, c) if x.dim() == 2 else (1, c, 1, 1)
        xf = x.float()
        if ctx.is_training():
            mean = xf.mean(dims)
            var = xf.var(dims, unbiased=False)
            with torch.no_grad():
                m = self.config.momentum
                self._running_mean.mul_(1 - m).add_(mean.detach(), alpha=m)
                self._running_var.mul_(1 - m).add_(var.detach(), alpha=m)
        else:
            mean, var = self._running_mean, self._running_var
        y = (xf - mean.reshape(shape)) * torch.rsqrt(var.reshape(shape) + self.config.eps)
        y = y * self.weight.tensor.float().reshape(shape) + self.bias.tensor.float().reshape(shape)
        return y.to(x.dtype)
