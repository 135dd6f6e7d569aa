"""Label heads (crates/nn/src/readout.rs:16-46, multi_readout.rs:11-131)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Saveable, Trainable
from ..symbolic import LabelPrediction, Vocabulary
from .linear import LinearBuilder


@dataclass
class ReadoutConfig:
    """crates/nn/src/readout.rs:11-17."""
    hidden_dim: int
    labels: int


@dataclass
class BinaryPrediction:
    """crates/nn/src/multi_readout.rs:115-122."""
    logit: float
    probability: float
    predicted: bool


@dataclass
class LabelBinaryPrediction:
    """One label's decision in a multi-label prediction (crates/nn/src/multi_readout.rs:23-34)."""
    label: str
    id: int
    logit: float
    probability: float
    predicted: bool


class Readout(Module, Trainable, Saveable):
    """Linear projection onto a label vocabulary; `predict` returns the arg-max label."""

    def __init__(self, labels: Vocabulary, projection):
        self._labels = labels
        self.projection = projection

    @classmethod
    def new(cls, backend, labels: Vocabulary, in_dim: int, seed: int = 42):
        return cls(labels, LinearBuilder(in_dim, len(labels)).with_bias().seed(seed).build(backend))

    def logits(self, x, ctx: ForwardCtx):
        return self.projection(x, ctx)

    forward = logits

    def probabilities(self, x, ctx: ForwardCtx):
        return ops.softmax(self.logits(x, ctx))

    def predict(self, x, ctx: ForwardCtx) -> list:
        p = self.probabilities(x, ctx).detach().float().cpu().reshape(-1, len(self._labels))
        idx = p.argmax(-1)
        return [LabelPrediction(self._labels.token(int(i)), int(i), float(p[r, i])) for r, i in enumerate(idx)]


class MultiReadout(Module, Trainable, Saveable):
    """One independent sigmoid head per label (multi-label classification)."""

    def __init__(self, labels: list, heads: list, threshold: float = 0.5):
        self._labels = list(labels)
        self.heads = heads
        self.threshold = threshold

    @classmethod
    def new(cls, backend, labels, in_dim: int, seed: int = 42, threshold: float = 0.5):
        heads = [LinearBuilder(in_dim, 1).with_bias().seed(seed + 2 * i).build(backend) for i in range(len(labels))]
        return cls(labels, heads, threshold)

    def forward(self, x, ctx: ForwardCtx):
        """Sigmoid scores [batch, num_labels]."""
        return torch.sigmoid(torch.cat([h(x, ctx) for h in self.heads], -1).float())

    def predict(self, x, ctx: ForwardCtx) -> list:
        s = self.forward(x, ctx).detach().cpu()
        return [[LabelPrediction(self._labels[j], j, float(row[j])) for j in range(len(self._labels)) if row[j] >= self.threshold]
                for row in s]

    def predict_all(self, x, ctx: ForwardCtx) -> list:
        """Every label's logit, probability and decision for every row (the reference's `predict_with_details`)."""
        logits = torch.cat([h(x, ctx) for h in self.heads], -1).float().detach().cpu()
        probs = torch.sigmoid(logits)
        return [[LabelBinaryPrediction(self._labels[j], j, float(lr[j]), float(pr[j]), bool(pr[j] >= self.threshold))
                 for j in range(len(self._labels))] for lr, pr in zip(logits, probs)]

    def top_k(self, x, ctx: ForwardCtx, k: int) -> list:
        s = self.forward(x, ctx).detach().cpu()
        out = []
        for row in s:
            vals, idx = row.topk(min(k, len(self._labels)))
            out.append([LabelPrediction(self._labels[int(j)], int(j), float(v)) for v, j in zip(vals, idx)])
        return out


class BinaryReadout(Module, Trainable, Saveable):
    def __init__(self, projection, threshold: float = 0.5):
        self.projection = projection
        self.threshold = threshold

    @classmethod
    def new(cls, backend, in_dim: int, seed: int = 42, threshold: float = 0.5):
        return cls(LinearBuilder(in_dim, 1).with_bias().seed(seed).build(backend), threshold)

    def forward(self, x, ctx: ForwardCtx):
        return torch.sigmoid(self.projection(x, ctx).float())[..., 0]

    def predict(self, x, ctx: ForwardCtx) -> list:
        return [bool(v >= self.threshold) for v in self.forward(x, ctx).detach().cpu().reshape(-1)]

    def predict_detailed(self, x, ctx: ForwardCtx) -> list:
        logits = self.projection(x, ctx).float().detach().cpu().reshape(-1)
        return [BinaryPrediction(float(l), float(torch.sigmoid(l)), bool(torch.sigmoid(l) >= self.threshold)) for l in logits]
