"""TensorPool: shape-keyed reuse of scratch tensors (crates/core/src/tensor_pool.rs:34-260).

On CUDA the torch caching allocator already recycles blocks; the pool matters for (a) static-shape steps that are
captured into CUDA graphs, where buffers must keep their addresses, and (b) the CPU backend.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class PoolStrategy(enum.Enum):
    STANDARD = "standard"
    TRAINING_ARENA = "training_arena"      # everything handed out in a step returns at begin_step()
    INFERENCE_REUSE = "inference_reuse"    # buffers return as soon as released


class TensorPool:
    def __init__(self, strategy: PoolStrategy = PoolStrategy.STANDARD, max_per_shape: int = 10, max_total: int = 100,
                 min_elems: int = 100, max_elems: int = 1 << 20):
        self.strategy = strategy
        self.max_per_shape, self.max_total = max_per_shape, max_total
        self.min_elems, self.max_elems = min_elems, max_elems
        self._free: dict = {}
        self._lent: list = []
        self.hits = self.misses = 0

    def _key(self, shape, dtype, device):
        return (tuple(shape), dtype, str(device))

    def _poolable(self, numel: int) -> bool:
        return self.min_elems <= numel <= self.max_elems or self.strategy is PoolStrategy.TRAINING_ARENA

    def acquire(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        key = self._key(shape, dtype, device)
        lst = self._free.get(key)
        if lst:
            self.hits += 1
            t = lst.pop()
        else:
            self.misses += 1
            t = torch.empty(tuple(shape), dtype=dtype, device=device)
        if self.strategy is PoolStrategy.TRAINING_ARENA:
            self._lent.append((key, t))
        return t

    def release(self, t: torch.Tensor) -> None:
        if not self._poolable(t.numel()):
            return
        key = self._key(t.shape, t.dtype, t.device)
        lst = self._free.setdefault(key, [])
        if len(lst) < self.max_per_shape and self.total_free() < self.max_total:
            lst.append(t)

    def begin_step(self) -> None:
        """Arena strategy: everything lent during the previous step becomes reusable."""
        for key, t in self._lent:
            self._free.setdefault(key, []).append(t)
        self._lent.clear()

    def total_free(self) -> int:
        return sum(len(v) for v in self._free.values())

    def clear(self) -> None:
        self._free.clear()
        self._lent.clear()

    def pool_stats(self) -> "PoolStats":
        """Contents of the free lists (crates/core/src/tensor_pool.rs:193-236); `stats()` has the hit counters."""
        n = sum(len(v) for v in self._free.values())
        nbytes = sum(t.numel() * t.element_size() for v in self._free.values() for t in v)
        return PoolStats(n, nbytes, sum(1 for v in self._free.values() if v), self.max_per_shape, self.max_total)

    def print_stats(self, file=None) -> None:
        import sys
        st, out = self.pool_stats(), file or sys.stdout
        print("Tensor pool statistics:", file=out)
        print(f"  total tensors: {st.total_tensors}\n  total memory: {st.total_memory_bytes / 1e6:.2f} MB\n"
              f"  unique shapes: {st.unique_shapes}\n  max per shape: {st.max_size_per_shape}\n  max total: {st.max_total_tensors}", file=out)

    def stats(self) -> dict:
        tot = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "hit_rate": self.hits / tot if tot else 0.0,
                "free": self.total_free(), "strategy": self.strategy.value}


@dataclass
class PoolStats:
    total_tensors: int
    total_memory_bytes: int
    unique_shapes: int
    max_size_per_shape: int
    max_total_tensors: int


class PooledTensor:
    """Context manager that returns its tensor to the pool on exit."""

    def __init__(self, pool: TensorPool, shape, dtype=torch.float32, device="cpu"):
        self.pool = pool
        self.tensor = pool.acquire(shape, dtype, device)

    def __enter__(self):
        return self.tensor

    def __exit__(self, *a):
        self.pool.release(self.tensor)
        return False


def pool_from_env():
    """RUSTRAL_POOL=1 enables a pool; RUSTRAL_POOL_STRATEGY picks the strategy (wikitext2_lm.rs:563-570)."""
    import os
    if os.environ.get("RUSTRAL_POOL", "0") not in ("1", "true"):
        return None
    name = os.environ.get("RUSTRAL_POOL_STRATEGY", "standard").lower()
    strat = {"standard": PoolStrategy.STANDARD, "training_arena": PoolStrategy.TRAINING_ARENA, "arena": PoolStrategy.TRAINING_ARENA,
             "inference_reuse": PoolStrategy.INFERENCE_REUSE}.get(name, PoolStrategy.STANDARD)
    return TensorPool(strat)
