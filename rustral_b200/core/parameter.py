"""Parameters with process-unique ids (crates/core/src/parameter.rs:12-130)."""
from __future__ import annotations

import itertools
import threading

import torch

_next_id = itertools.count(1)
_id_lock = threading.Lock()


class ParameterId(int):
    """Process-local unique id.  Checkpoints key state by parameter NAME, never by this id."""

    @staticmethod
    def fresh() -> "ParameterId":
        with _id_lock:
            return ParameterId(next(_next_id))


class Parameter:
    """A named trainable tensor.  `tensor` is a leaf with requires_grad=True."""

    __slots__ = ("id", "name", "tensor")

    def __init__(self, name: str, tensor: torch.Tensor, requires_grad: bool = True):
        self.id = ParameterId.fresh()
        self.name = name
        t = tensor.detach()
        t.requires_grad_(requires_grad and t.is_floating_point())
        self.tensor = t

    @classmethod
    def with_tensor(cls, other: "Parameter", tensor: torch.Tensor) -> "Parameter":
        """Same id and name, new storage (used by optimizers that return updated copies)."""
        p = cls.__new__(cls)
        p.id, p.name = other.id, other.name
        t = tensor.detach()
        t.requires_grad_(other.tensor.requires_grad)
        p.tensor = t
        return p

    @property
    def shape(self):
        return tuple(self.tensor.shape)

    def numel(self) -> int:
        return self.tensor.numel()

    @property
    def grad(self):
        return self.tensor.grad

    def zero_grad(self):
        self.tensor.grad = None

    def set_(self, tensor: torch.Tensor) -> None:
        """Overwrite the value in place (shape-checked)."""
        if tuple(tensor.shape) != self.shape:
            from .errors import ShapeMismatch
            raise ShapeMismatch(self.shape, tensor.shape, self.name)
        with torch.no_grad():
            self.tensor.copy_(tensor.to(self.tensor.dtype))

    def to(self, *args, **kw) -> "Parameter":
        rg = self.tensor.requires_grad
        self.tensor = self.tensor.detach().to(*args, **kw).requires_grad_(rg)
        return self

    def __repr__(self):
        return f"Parameter(id={int(self.id)}, name={self.name!r}, shape={self.shape}, dtype={self.tensor.dtype})"


class ParameterRef:
    """Borrowed view of a parameter: (id, name)."""

    __slots__ = ("id", "name")

    def __init__(self, p: Parameter):
        self.id, self.name = p.id, p.name


class ParameterGroup:
    """Parameters that share optimizer hyper-parameters."""

    def __init__(self, name: str, params=None, **hyper):
        self.name = name
        self.params: list[Parameter] = list(params or [])
        self.hyper = dict(hyper)

    def add(self, p: Parameter) -> None:
        self.params.append(p)

    def __iter__(self):
        return iter(self.params)

    def __len__(self):
        return len(self.params)

    def numel(self) -> int:
        return sum(p.numel() for p in self.params)
