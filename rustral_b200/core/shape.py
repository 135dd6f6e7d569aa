"""Validated shapes and the shape policy (crates/core/src/shape.rs:6-57, shape_policy.rs:8)."""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .errors import InvalidShape


@dataclass(frozen=True)
class Shape:
    """A non-empty shape whose dimensions are all non-zero."""
    dims: tuple

    def __init__(self, dims):
        dims = tuple(int(d) for d in dims)
        if len(dims) == 0:
            raise InvalidShape("shape must have at least one dimension")
        if any(d <= 0 for d in dims):
            raise InvalidShape(f"shape dimensions must be positive, got {dims}")
        object.__setattr__(self, "dims", dims)

    @property
    def rank(self) -> int:
        return len(self.dims)

    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def __iter__(self):
        return iter(self.dims)

    def __len__(self):
        return len(self.dims)

    def __getitem__(self, i):
        return self.dims[i]


class ShapePolicy(enum.Enum):
    """How much shapes may vary between steps; decides CUDA-graph capture and arena pooling."""
    STATIC = "static"
    DYNAMIC_BOUNDED = "dynamic_bounded"
    DYNAMIC_UNBOUNDED = "dynamic_unbounded"

    def supports_cuda_graph_capture(self) -> bool:
        return self is ShapePolicy.STATIC

    def prefers_arena_pool(self) -> bool:
        return self in (ShapePolicy.STATIC, ShapePolicy.DYNAMIC_BOUNDED)


class ShapeExt:
    """Element count of a plain shape sequence (crates/core/src/shape.rs:41-50): `ShapeExt.elem_count((2, 3, 4)) == 24`;
    the empty shape is a scalar and counts one element."""

    @staticmethod
    def elem_count(shape) -> int:
        n = 1
        for d in shape:
            n *= int(d)
        return n


class TensorShape:
    """Anything that can report its shape (crates/core/src/shape.rs:57-60).  `TensorShape.shape_of(x)` reads it from
    tensors, parameters, arrays and `Shape` objects alike."""

    @staticmethod
    def shape_of(x) -> tuple:
        if isinstance(x, Shape):
            return x.dims
        t = getattr(x, "tensor", x)
        shp = getattr(t, "shape", None)
        if shp is None:
            raise TypeError(f"{type(x).__name__} has no shape")
        return tuple(int(d) for d in shp)
