"""Timeline profiler with Chrome-trace export and a bandwidth calculator
(crates/wgpu-backend/src/profiler.rs:91-456: GpuProfiler, export_chrome_trace :219, ScopedEvent :335,
BandwidthCalculator :362).

The reference stamps events with host timestamps around wgpu submissions.  Here an event on a CUDA device is bracketed
by CUDA events on the current stream, so the exported duration is device time; on the CPU it is wall-clock time.
The export is the Chrome trace-event JSON ("ph": "X" complete events plus "i" instants for memory samples) that
chrome://tracing and Perfetto read.
"""
from __future__ import annotations

import json
import time
from contextlib import contextmanager
from dataclasses import dataclass, field

import torch


@dataclass
class ProfileEvent:
    name: str
    category: str
    start_us: float            # host timestamp of the start (trace position)
    duration_us: float         # device time on CUDA, wall-clock on CPU
    args: dict = field(default_factory=dict)


@dataclass
class MemoryEvent:
    timestamp_us: float
    allocated_bytes: int
    reserved_bytes: int


class GpuProfiler:
    def __init__(self, device=None, enabled: bool = True):
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.enabled = enabled
        self.events: list = []
        self.memory_events: list = []
        self._pending: list = []           # (ProfileEvent, start CUDA event, end CUDA event)
        self._t0 = time.perf_counter()

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    @contextmanager
    def scope(self, name: str, category: str = "kernel", **args):
        """`with profiler.scope("gemm", bytes=...)`: the ScopedEvent / profile_scope! of the reference."""
        if not self.enabled:
            yield
            return
        start = self._now_us()
        if self.device.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                ev = ProfileEvent(name, category, start, 0.0, dict(args))
                self._pending.append((ev, e0, e1))
        else:
            try:
                yield
            finally:
                self.events.append(ProfileEvent(name, category, start, self._now_us() - start, dict(args)))

    def record_memory(self) -> None:
        if not self.enabled:
            return
        if self.device.type == "cuda":
            self.memory_events.append(MemoryEvent(self._now_us(), torch.cuda.memory_allocated(self.device),
                                                  torch.cuda.memory_reserved(self.device)))
        else:
            self.memory_events.append(MemoryEvent(self._now_us(), 0, 0))

    def resolve(self) -> None:
        """Reads back the device durations of finished scopes (synchronises the device once)."""
        if self._pending:
            torch.cuda.synchronize(self.device)
            for ev, e0, e1 in self._pending:
                ev.duration_us = e0.elapsed_time(e1) * 1e3
                self.events.append(ev)
            self._pending = []

    def summary(self) -> dict:
        self.resolve()
        out: dict = {}
        for e in self.events:
            s = out.setdefault(e.name, {"count": 0, "total_us": 0.0, "max_us": 0.0})
            s["count"] += 1
            s["total_us"] += e.duration_us
            s["max_us"] = max(s["max_us"], e.duration_us)
        for s in out.values():
            s["mean_us"] = s["total_us"] / s["count"]
        return out

    def profile_summary(self) -> "ProfileSummary":
        """Totals per category (crates/wgpu-backend/src/profiler.rs:196-216); `summary()` above is per event name."""
        self.resolve()
        cats: dict = {}
        for e in self.events:
            t, n = cats.get(e.category, (0.0, 0))
            cats[e.category] = (t + e.duration_us, n + 1)
        peak = max((m.allocated_bytes for m in self.memory_events), default=0)
        cur = self.memory_events[-1].allocated_bytes if self.memory_events else 0
        return ProfileSummary(len(self.events) + len(self._pending), len(self.events), peak, cur, cats)

    def export_chrome_trace(self, path: str | None = None) -> str:
        self.resolve()
        trace = [{"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.duration_us, "pid": 0,
                  "tid": 0 if e.category != "transfer" else 1, "args": e.args} for e in self.events]
        trace += [{"name": "memory", "ph": "i", "ts": m.timestamp_us, "pid": 0, "tid": 2, "s": "g",
                   "args": {"allocated_bytes": m.allocated_bytes, "reserved_bytes": m.reserved_bytes}}
                  for m in self.memory_events]
        text = json.dumps({"traceEvents": trace, "displayTimeUnit": "ms"})
        if path is not None:
            with open(path, "w") as f:
                f.write(text)
        return text

    def clear(self) -> None:
        self.events, self.memory_events, self._pending = [], [], []


@dataclass
class ProfileSummary:
    total_events: int
    completed_events: int
    total_memory_allocated: int          # peak of the recorded memory samples
    current_memory: int
    category_times: dict                 # category -> (total microseconds, count)


def export_chrome_trace(profiler: GpuProfiler, path: str | None = None) -> str:
    return profiler.export_chrome_trace(path)


class BandwidthCalculator:
    """GB/s of an operation from its bytes and duration, and the fraction of a peak (default: the copy bandwidth
    measured on B200, 6549.8 GB/s)."""

    def __init__(self, peak_gbs: float = 6549.8):
        self.peak_gbs = peak_gbs

    @staticmethod
    def gbs(nbytes: float, duration_us: float) -> float:
        return nbytes / (duration_us * 1e-6) / 1e9 if duration_us > 0 else 0.0

    def utilization(self, nbytes: float, duration_us: float) -> float:
        return self.gbs(nbytes, duration_us) / self.peak_gbs

    @staticmethod
    def elementwise_bytes(numel: int, inputs: int = 2, outputs: int = 1, elem_bytes: int = 2) -> int:
        return numel * (inputs + outputs) * elem_bytes

    @staticmethod
    def matmul_bytes(m: int, n: int, k: int, elem_bytes: int = 2) -> int:
        return (m * k + k * n + m * n) * elem_bytes
