"""MemoryProfiler: tagged allocation events, peak tracking, OOM-risk prediction, leak detection, timeline export
(crates/core/src/memory_profiler.rs:52-393).  On CUDA, `sample_device()` also records the allocator's counters."""
from __future__ import annotations

import enum
import json
import time
from dataclasses import dataclass, field

import torch


@dataclass
class AllocationEvent:
    t: float
    kind: str          # "alloc" | "free" | "sample"
    tag: str
    nbytes: int
    handle: int


class OOMRisk:
    LOW, MEDIUM, HIGH, CRITICAL = "low", "medium", "high", "critical"


class OomRisk(enum.Enum):
    """The four risk levels as an enumeration (crates/core/src/memory_profiler.rs:345-362); `predict_oom_risk` returns the
    plain strings, `OomRisk(value)` turns one into a member."""
    LOW = "low"
    MEDIUM = "medium"
    HIGH = "high"
    CRITICAL = "critical"

    def as_str(self) -> str:
        return self.value


@dataclass
class MemorySnapshot:
    """State of the profiler at one moment (crates/core/src/memory_profiler.rs:43-50).  Also answers the dictionary keys
    `label`, `t`, `current`, `peak`, `by_tag`."""
    timestamp: float
    total_allocated: int
    peak_allocated: int
    num_allocations: int
    by_tag: dict
    label: str = ""

    def __getitem__(self, key):
        return {"label": self.label, "t": self.timestamp, "current": self.total_allocated, "peak": self.peak_allocated,
                "by_tag": self.by_tag, "num_allocations": self.num_allocations}[key]


@dataclass
class MemorySummary:
    """Totals since the profiler was created (crates/core/src/memory_profiler.rs:325-336, 365-372)."""
    current_bytes: int
    peak_bytes: int
    total_allocations: int
    total_deallocations: int
    active_count: int
    duration: float


class MemoryProfiler:
    def __init__(self, capacity_bytes: int | None = None):
        self.events: list = []
        self.active: dict = {}          # handle -> (tag, nbytes, t)
        self.by_tag: dict = {}
        self.current = 0
        self.peak = 0
        self._next = 1
        if capacity_bytes is None and torch.cuda.is_available():
            capacity_bytes = torch.cuda.get_device_properties(0).total_memory
        self.capacity_bytes = capacity_bytes or (1 << 62)
        self.snapshots: list = []
        self._t0 = time.time()

    def alloc(self, tag: str, nbytes: int) -> int:
        h = self._next
        self._next += 1
        now = time.time()
        self.active[h] = (tag, nbytes, now)
        self.by_tag[tag] = self.by_tag.get(tag, 0) + nbytes
        self.current += nbytes
        self.peak = max(self.peak, self.current)
        self.events.append(AllocationEvent(now, "alloc", tag, nbytes, h))
        return h

    def free(self, handle: int) -> None:
        rec = self.active.pop(handle, None)
        if rec is None:
            return
        tag, nbytes, _ = rec
        self.by_tag[tag] -= nbytes
        self.current -= nbytes
        self.events.append(AllocationEvent(time.time(), "free", tag, nbytes, handle))

    def track_tensor(self, tag: str, t: torch.Tensor) -> "AllocationTracker":
        return AllocationTracker(self, tag, t.numel() * t.element_size())

    def sample_device(self, tag: str = "device") -> int:
        """Records torch's allocated bytes on the current CUDA device as a sample event."""
        n = torch.cuda.memory_allocated() if torch.cuda.is_available() else 0
        self.events.append(AllocationEvent(time.time(), "sample", tag, n, 0))
        self.peak = max(self.peak, n)
        return n

    def snapshot(self, label: str = "") -> dict:
        s = MemorySnapshot(time.time(), self.current, self.peak, len(self.active), dict(self.by_tag), label)
        self.snapshots.append(s)
        return s

    def summary(self) -> MemorySummary:
        allocs = sum(1 for e in self.events if e.kind == "alloc")
        frees = sum(1 for e in self.events if e.kind == "free")
        return MemorySummary(self.current, self.peak, allocs, frees, allocs - frees, time.time() - self._t0)

    def reset(self) -> None:
        """Forgets events, live allocations and peaks; the clock of `summary().duration` restarts."""
        self.events.clear(); self.active.clear(); self.by_tag.clear(); self.snapshots.clear()
        self.current = self.peak = 0
        self._t0 = time.time()

    def predict_oom_risk(self, planned_bytes: int = 0) -> str:
        """< 0.5 low, < 0.75 medium, < 0.9 high, else critical (fraction of capacity after the planned allocation)."""
        frac = (self.current + planned_bytes) / self.capacity_bytes
        if frac < 0.5:
            return OOMRisk.LOW
        if frac < 0.75:
            return OOMRisk.MEDIUM
        if frac < 0.9:
            return OOMRisk.HIGH
        return OOMRisk.CRITICAL

    def find_leaks(self, older_than_s: float = 0.0) -> list:
        now = time.time()
        return [(h, tag, n) for h, (tag, n, t) in self.active.items() if now - t >= older_than_s]

    def export_timeline(self, path: str | None = None) -> str:
        text = json.dumps([e.__dict__ for e in self.events])
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text


class AllocationTracker:
    """Context manager / RAII handle for one tracked allocation."""

    def __init__(self, profiler: MemoryProfiler, tag: str, nbytes: int):
        self.p = profiler
        self.h = profiler.alloc(tag, nbytes)

    def release(self):
        if self.h:
            self.p.free(self.h)
            self.h = 0

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.release()
        return False


_global = None


def global_profiler() -> MemoryProfiler:
    global _global
    if _global is None:
        _global = MemoryProfiler()
    return _global


def track_tensor(tag: str, t: torch.Tensor) -> AllocationTracker:
    return global_profiler().track_tensor(tag, t)
