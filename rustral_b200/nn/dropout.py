"""Mode-gated inverted dropout (crates/nn/src/dropout.rs:17-75)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module


@dataclass
class DropoutConfig:
    p: float = 0.1

    def __post_init__(self):
        self.p = min(max(float(self.p), 0.0), 1.0)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        y, mask = ops.dropout(x, p, True, seed=seed, offset=offset, return_mask=True)
        ctx.save_for_backward(mask)
        ctx.p = p
        return y

    @staticmethod
    def backward(ctx, dy):
        (mask,) = ctx.saved_tensors
        return ops.binary("mul", dy.contiguous(), (mask.to(dy.dtype) * (1.0 / (1.0 - ctx.p))).contiguous()), None, None, None


class Dropout(Module):
    """Active only when ``ctx.is_training()``; the Philox stream is keyed by (ctx.seed, a per-call offset)."""

    def __init__(self, config: DropoutConfig | float = 0.1):
        self.config = config if isinstance(config, DropoutConfig) else DropoutConfig(config)

    def forward(self, x, ctx: ForwardCtx):
        p = self.config.p
        if not ctx.is_training() or p <= 0.0:
            return x
        if p >= 1.0:
            return x * 0
        return _DropoutFn.apply(x, p, ctx.seed, ctx.next_rng_offset((x.numel() + 3) // 4))
