"""Terminal training dashboard (crates/tui/src/lib.rs:135-1015): loss sparkline, throughput, memory / OOM risk, leak
warnings.  Plain ANSI text (no curses dependency); `TuiMetricsBackend` plugs it into MetricsLogger and
`run_dashboard` refreshes it from a background thread (crates/runtime/src/tui_hook.rs)."""
from __future__ import annotations

import sys
import threading
import time
from dataclasses import dataclass, field

from ..metrics import MetricsBackend

_BARS = " ▁▂▃▄▅▆▇█"


def sparkline(values, width: int = 40) -> str:
    vals = list(values)[-width:]
    if not vals:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    return "".join(_BARS[1 + int((v - lo) / span * (len(_BARS) - 2))] for v in vals)


@dataclass
class EpochSnapshot:
    epoch: int
    loss: float
    accuracy: float | None = None
    examples_per_sec: float = 0.0

    def push_to_dashboard(self, dash: "TrainingDashboard") -> None:
        dash.push_epoch(self)


@dataclass
class TrainingDashboard:
    title: str = "rustral-b200"
    losses: list = field(default_factory=list)
    accuracies: list = field(default_factory=list)
    throughput: float = 0.0
    memory_used: int = 0
    memory_capacity: int = 0
    warnings: list = field(default_factory=list)
    epoch: int = 0
    _lock: threading.Lock = field(default_factory=threading.Lock, repr=False)

    def push_epoch(self, s: EpochSnapshot) -> None:
        with self._lock:
            self.epoch = s.epoch
            self.losses.append(s.loss)
            if s.accuracy is not None:
                self.accuracies.append(s.accuracy)
            self.throughput = s.examples_per_sec

    def push_scalar(self, name: str, value: float) -> None:
        with self._lock:
            if "loss" in name:
                self.losses.append(value)
            elif "acc" in name:
                self.accuracies.append(value)

    def set_memory(self, used: int, capacity: int) -> None:
        with self._lock:
            self.memory_used, self.memory_capacity = used, capacity

    def oom_risk(self) -> str:
        if not self.memory_capacity:
            return "unknown"
        f = self.memory_used / self.memory_capacity
        return "low" if f < 0.5 else "medium" if f < 0.75 else "high" if f < 0.9 else "critical"

    def warn(self, msg: str) -> None:
        with self._lock:
            self.warnings.append(msg)
            self.warnings = self.warnings[-5:]


class DashboardRenderer:
    def __init__(self, dash: TrainingDashboard, file=None, ansi: bool = True):
        self.dash, self.file, self.ansi = dash, file or sys.stderr, ansi

    def render_text(self) -> str:
        d = self.dash
        with d._lock:
            lines = [f"== {d.title} == epoch {d.epoch}"]
            if d.losses:
                lines.append(f"loss {d.losses[-1]:.4f}  {sparkline(d.losses)}")
            if d.accuracies:
                lines.append(f"acc  {d.accuracies[-1]:.4f}  {sparkline(d.accuracies)}")
            lines.append(f"throughput {d.throughput:.1f}/s")
            if d.memory_capacity:
                lines.append(f"memory {d.memory_used / 2**30:.2f} / {d.memory_capacity / 2**30:.2f} GiB  OOM risk: {d.oom_risk()}")
            lines += [f"! {w}" for w in d.warnings]
        return "\n".join(lines)

    def draw(self) -> None:
        text = self.render_text()
        if self.ansi:
            self.file.write("\x1b[2J\x1b[H")
        self.file.write(text + "\n")
        self.file.flush()


class TuiMetricsBackend(MetricsBackend):
    def __init__(self, dash: TrainingDashboard):
        self.dash = dash

    def log_scalar(self, m) -> None:
        self.dash.push_scalar(m.name, m.value)


_global_dash = None
_global_thread = None


def init_global_dashboard(title: str = "rustral-b200", refresh_s: float = 0.5, file=None) -> TrainingDashboard:
    """Starts the render thread once per process; returns the shared dashboard."""
    global _global_dash, _global_thread
    if _global_dash is None:
        _global_dash = TrainingDashboard(title)
        _global_thread = run_dashboard(_global_dash, refresh_s, file)
    return _global_dash


def run_dashboard(dash: TrainingDashboard, refresh_s: float = 0.5, file=None, stop_event: threading.Event | None = None):
    r = DashboardRenderer(dash, file)
    stop = stop_event or threading.Event()

    def loop():
        while not stop.wait(refresh_s):
            try:
                import torch
                if torch.cuda.is_available():
                    free, total = torch.cuda.mem_get_info()
                    dash.set_memory(total - free, total)
            except Exception:   # noqa: BLE001 - the dashboard must never take training down
                pass
            r.draw()

    t = threading.Thread(target=loop, daemon=True)
    t.stop_event = stop
    t.start()
    return t
