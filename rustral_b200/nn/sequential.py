"""Sequential2 / chain: parameter names first. / second. (crates/nn/src/sequential.rs:5-77)."""
from __future__ import annotations

from ..core import ForwardCtx, Module, Saveable, Trainable


class Sequential2(Module, Trainable, Saveable):
    def __init__(self, first, second):
        self.first, self.second = first, second

    def forward(self, x, ctx: ForwardCtx):
        return self.second(self.first(x, ctx), ctx)


def chain(a, b) -> Sequential2:
    return Sequential2(a, b)


class Sequential(Module, Trainable, Saveable):
    """N-ary variant: names layers.{i}."""

    def __init__(self, *layers):
        self.layers = list(layers)

    def forward(self, x, ctx: ForwardCtx):
        for l in self.layers:
            x = l(x, ctx)
        return x
