"""ForwardCtx: the explicit per-call context (crates/core/src/context.rs:12-109)."""
from __future__ import annotations

import enum
import itertools
import threading

from .shape import ShapePolicy

_run_ids = itertools.count(1)
_run_lock = threading.Lock()


class Mode(enum.Enum):
    TRAIN = "train"
    INFERENCE = "inference"


class RunId(int):
    @staticmethod
    def fresh() -> "RunId":
        with _run_lock:
            return RunId(next(_run_ids))


class ForwardCtx:
    """Carries the backend, the Train/Inference mode, a run id, an optional OperationProfiler and the shape policy.

    Modules never consult global state for any of these: dropout reads ``ctx.is_training()``, profiled ops
    record into ``ctx.profiler``.
    """

    def __init__(self, backend=None, mode: Mode = Mode.INFERENCE, profiler=None,
                 shape_policy: ShapePolicy = ShapePolicy.DYNAMIC_UNBOUNDED, seed: int = 0):
        if backend is None:
            from .backend import default_backend
            backend = default_backend()
        self.backend = backend
        self.mode = mode
        self.run_id = RunId.fresh()
        self.profiler = profiler
        self.shape_policy = shape_policy
        self.seed = seed
        self._rng_offset = 0

    @classmethod
    def train(cls, backend=None, **kw) -> "ForwardCtx":
        return cls(backend, Mode.TRAIN, **kw)

    @classmethod
    def inference(cls, backend=None, **kw) -> "ForwardCtx":
        return cls(backend, Mode.INFERENCE, **kw)

    def is_training(self) -> bool:
        return self.mode is Mode.TRAIN

    def with_profiler(self, profiler) -> "ForwardCtx":
        self.profiler = profiler
        return self

    def with_shape_policy(self, policy: ShapePolicy) -> "ForwardCtx":
        self.shape_policy = policy
        return self

    def next_rng_offset(self, n: int) -> int:
        """Reserves `n` counter values of the dropout generator; each dropout call gets a fresh range."""
        off = self._rng_offset
        self._rng_offset += n
        return off

    def profile(self, name: str, shape=None):
        """Context manager recording one operation into the profiler (no-op without one)."""
        if self.profiler is None:
            return _NULL_GUARD
        return self.profiler.guard(name, shape=shape)


class _NullGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL_GUARD = _NullGuard()
