"""Losses: MSE, cross-entropy (per-row softmax), BCE-with-logits (crates/nn/src/loss.rs:19-219)."""
from __future__ import annotations

import torch

from .. import ops
from ..core import ShapeMismatch


class MSELoss:
    def forward(self, pred, target):
        if pred.shape != target.shape:
            raise ShapeMismatch(pred.shape, target.shape, "MSELoss")
        d = pred.float() - target.float()
        return (d * d).mean()

    __call__ = forward


class CrossEntropyLoss:
    """Mean over rows of -log softmax(logits)[target]; softmax is per row."""

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index

    def forward_indices(self, logits, targets, n_valid=None):
        return ops.cross_entropy(logits, torch.as_tensor(targets, dtype=torch.int64, device=logits.device), n_valid,
                                 self.ignore_index)

    def forward(self, logits, onehot):
        """One-hot (or soft) targets of the same shape as the logits."""
        if logits.shape != onehot.shape:
            raise ShapeMismatch(logits.shape, onehot.shape, "CrossEntropyLoss")
        lp = ops.log_softmax(logits.float() if not logits.is_cuda else logits)
        return -(lp.float() * onehot.float()).sum(-1).mean()

    __call__ = forward_indices


class BCEWithLogitsLoss:
    """max(x,0) - x*y + log(1 + exp(-|x|)), averaged."""

    def forward(self, logits, targets):
        if logits.shape != targets.shape:
            raise ShapeMismatch(logits.shape, targets.shape, "BCEWithLogitsLoss")
        x, y = logits.float(), targets.float()
        return (torch.clamp(x, min=0) - x * y + torch.log1p(torch.exp(-x.abs()))).mean()

    __call__ = forward
