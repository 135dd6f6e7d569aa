"""Scalar / histogram logging (crates/metrics/src/lib.rs): console logger, JSONL writer, fan-out logger, progress bar."""
from __future__ import annotations

import json
import os
import sys
import threading
import time
from dataclasses import dataclass


@dataclass
class ScalarMetric:
    name: str
    value: float
    step: int
    timestamp: float


@dataclass
class HistogramMetric:
    name: str
    counts: list
    edges: list
    step: int
    timestamp: float


class MetricsBackend:
    def log_scalar(self, m: ScalarMetric) -> None:
        raise NotImplementedError

    def log_histogram(self, m: HistogramMetric) -> None:
        pass

    def flush(self) -> None:
        pass

    def name(self) -> str:
        return type(self).__name__


class ConsoleLogger(MetricsBackend):
    """Buffers scalars and prints `[step N] k=v, ...` lines (flushes every `flush_every` scalars)."""

    def __init__(self, flush_every: int = 10, file=None):
        self.flush_every, self.file = flush_every, file or sys.stdout
        self._buf: list = []

    def log_scalar(self, m):
        self._buf.append(m)
        if len(self._buf) >= self.flush_every:
            self.flush()

    def flush(self):
        by_step: dict = {}
        for m in self._buf:
            by_step.setdefault(m.step, []).append(m)
        for step in sorted(by_step):
            print(f"[step {step}] " + ", ".join(f"{m.name}={m.value:.6g}" for m in by_step[step]), file=self.file)
        self._buf.clear()


class TensorBoardWriter(MetricsBackend):
    """JSON-lines event file `<log_dir>/<run_name>.jsonl` ({"type":"scalar",name,value,step,timestamp}); histograms
    are written too (the reference drops them)."""

    def __init__(self, log_dir: str, run_name: str = "run"):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, run_name + ".jsonl")
        self._f = open(self.path, "a", encoding="utf-8")

    def log_scalar(self, m):
        self._f.write(json.dumps({"type": "scalar", "name": m.name, "value": m.value, "step": m.step,
                                  "timestamp": m.timestamp}) + "\n")

    def log_histogram(self, m):
        self._f.write(json.dumps({"type": "histogram", "name": m.name, "counts": m.counts, "edges": m.edges,
                                  "step": m.step, "timestamp": m.timestamp}) + "\n")

    def flush(self):
        self._f.flush()


class MetricsLogger:
    def __init__(self, backends=None):
        self.backends = list(backends or [])
        self.current_step = 0
        self._lock = threading.Lock()

    def add_backend(self, b: MetricsBackend) -> None:
        self.backends.append(b)

    def log_scalar(self, name: str, value: float) -> None:
        self.log_scalar_with_step(name, value, self.current_step)

    def log_scalar_with_step(self, name: str, value: float, step: int) -> None:
        m = ScalarMetric(name, float(value), step, time.time())
        with self._lock:
            for b in self.backends:
                b.log_scalar(m)

    def log_histogram(self, name: str, values, bins: int = 30) -> None:
        import numpy as np
        counts, edges = np.histogram(np.asarray(values, dtype=np.float64), bins=bins)
        m = HistogramMetric(name, counts.tolist(), edges.tolist(), self.current_step, time.time())
        with self._lock:
            for b in self.backends:
                b.log_histogram(m)

    def step(self) -> None:
        self.current_step += 1

    def set_step(self, s: int) -> None:
        self.current_step = s

    def flush(self) -> None:
        for b in self.backends:
            b.flush()

    def log_training_summary(self, epoch: int, loss: float, accuracy: float | None = None, lr: float | None = None) -> None:
        self.log_scalar_with_step("train/loss", loss, epoch)
        if accuracy is not None:
            self.log_scalar_with_step("train/accuracy", accuracy, epoch)
        if lr is not None:
            self.log_scalar_with_step("train/lr", lr, epoch)
        self.flush()


ThreadSafeMetricsLogger = MetricsLogger     # the logger serialises backend calls itself


class ProgressBar:
    def __init__(self, total: int, width: int = 30, file=None):
        self.total, self.width, self.file = max(1, total), width, file or sys.stderr
        self.n = 0
        self.t0 = time.time()

    def update(self, n: int = 1, suffix: str = "") -> None:
        self.n = min(self.total, self.n + n)
        fill = int(self.width * self.n / self.total)
        rate = self.n / max(1e-9, time.time() - self.t0)
        print(f"\r[{'#' * fill}{'.' * (self.width - fill)}] {self.n}/{self.total} {rate:.1f}/s {suffix}", end="", file=self.file)
        if self.n == self.total:
            print(file=self.file)


def create_logger(log_dir: str | None = None, run_name: str = "run", console: bool = True) -> MetricsLogger:
    l = MetricsLogger()
    if console:
        l.add_backend(ConsoleLogger())
    if log_dir:
        l.add_backend(TensorBoardWriter(log_dir, run_name))
    return l
