"""Module contracts (crates/core/src/module.rs:8-91).

A module is an object with ``forward(input, ctx)``; trainable modules enumerate their parameters with
stable hierarchical names through ``visit_parameters``.  Names are the checkpoint keys.
"""
from __future__ import annotations

from typing import Callable, Iterator

import torch

from .context import ForwardCtx
from .parameter import Parameter


class Module:
    """Base class: ``forward(input, ctx) -> output``; ``__call__`` forwards to it."""

    def forward(self, x, ctx: ForwardCtx):
        raise NotImplementedError

    def __call__(self, x, ctx: ForwardCtx | None = None):
        if ctx is None:
            ctx = ForwardCtx.inference()
        return self.forward(x, ctx)


class NamedParameters:
    """Mixin: enumerate parameters as (name, Parameter) with stable hierarchical names.

    Default implementation walks instance attributes in definition order: ``Parameter`` attributes are
    leaves, ``NamedParameters`` attributes and lists of them are sub-trees (``layers.0.attn.wq.weight``).
    A class can pin the order / names by overriding ``_children``.
    """

    def _children(self):
        for k, v in self.__dict__.items():
            if k.startswith("_"):
                continue
            if isinstance(v, (Parameter, NamedParameters)):
                yield k, v
            elif isinstance(v, (list, tuple)) and v and all(isinstance(e, (Parameter, NamedParameters)) for e in v):
                yield k, list(v)

    def visit_parameters(self, f: Callable[[str, Parameter], None], prefix: str = "") -> None:
        for name, child in self._children():
            if isinstance(child, Parameter):
                f(prefix + name, child)
            elif isinstance(child, list):
                for i, e in enumerate(child):
                    if isinstance(e, Parameter):
                        f(f"{prefix}{name}.{i}", e)
                    else:
                        e.visit_parameters(f, f"{prefix}{name}.{i}.")
            else:
                child.visit_parameters(f, prefix + name + ".")

    def visit_parameters_mut(self, f: Callable[[str, Parameter], None], prefix: str = "") -> None:
        self.visit_parameters(f, prefix)

    def named_parameters(self) -> list:
        out = []
        self.visit_parameters(lambda n, p: out.append((n, p)))
        return out


class Trainable(NamedParameters):
    def parameters(self) -> list:
        """Every parameter once, in first-appearance order.  A parameter shared by two sub-modules (tied embeddings, one
        layer used twice) has two names in `named_parameters()` but is one entry here, so that an optimizer steps it once."""
        seen, out = set(), []
        for _, p in self.named_parameters():
            if id(p) not in seen:
                seen.add(id(p))
                out.append(p)
        return out

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.zero_grad()

    def to(self, *args, **kw):
        for p in self.parameters():
            p.to(*args, **kw)
        return self


class StatefulModule:
    """Modules with a recurrent state (LSTM/GRU cells): ``initial_state(batch)``."""

    def initial_state(self, batch: int, ctx: ForwardCtx):
        raise NotImplementedError


class Saveable(NamedParameters):
    """state_dict / load_state_dict keyed by the NamedParameters paths; loading is strict."""

    def state_dict(self) -> dict:
        return {n: p.tensor.detach().clone() for n, p in self.named_parameters()}

    def load_state_dict(self, state: dict, strict: bool = True) -> None:
        from .errors import SerializationError, ShapeMismatch
        mine = dict(self.named_parameters())
        if strict:
            missing = [k for k in mine if k not in state]
            extra = [k for k in state if k not in mine]
            if missing:
                raise SerializationError(f"missing keys in state dict: {missing}")
            if extra:
                raise SerializationError(f"unexpected keys in state dict: {extra}")
        staged = []
        for k, p in mine.items():
            if k not in state:
                continue
            t = state[k]
            if tuple(t.shape) != p.shape:
                raise ShapeMismatch(p.shape, t.shape, k)
            staged.append((p, t))
        for p, t in staged:   # nothing is mutated until everything validated
            p.set_(t)


def collect_named_parameters(model: NamedParameters) -> list:
    return model.named_parameters()


def collect_named_parameter_ids(model: NamedParameters) -> dict:
    return {n: int(p.id) for n, p in model.named_parameters()}
