"""Terminal training dashboard (crates/tui/src/lib.rs:71-1015).

Four panes drawn with box characters and ANSI colours (no curses / ratatui dependency):

* progress  epoch and batch bars, step, elapsed time, ETA, throughput
* metrics   latest loss / accuracy / learning rate with sparklines over a rolling window
* memory    used / peak / available with a bar and the OOM-risk level, per-tag breakdown, allocation counts
* warnings  leak reports (fed from `MemoryProfiler.find_leaks`), NaN losses, OOM risk, free-form events

`DashboardRenderer` draws frames, reads the keyboard without blocking when standard input is a terminal (`q` quits,
`p` pauses / resumes drawing, `c` clears the leak list) and can run as a loop on the calling or on a background
thread; `TuiMetricsBackend` plugs the dashboard into `MetricsLogger`; `dump_metrics` writes the state as JSON."""
from __future__ import annotations

import enum
import json
import math
import os
import sys
import threading
import time
from dataclasses import dataclass, field

from ..metrics import MetricsBackend

_BARS = " ▁▂▃▄▅▆▇█"
_COLORS = {"green": "\x1b[32m", "yellow": "\x1b[33m", "red": "\x1b[31m", "bright_red": "\x1b[91m", "cyan": "\x1b[36m",
           "bold": "\x1b[1m", "reset": "\x1b[0m"}


def sparkline(values, width: int = 40) -> str:
    vals = [v for v in list(values)[-width:] if isinstance(v, (int, float)) and math.isfinite(v)]
    if not vals:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    return "".join(_BARS[1 + int((v - lo) / span * (len(_BARS) - 2))] for v in vals)


def format_bytes(n: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024 or unit == "TiB":
            return f"{n:.0f} {unit}" if unit == "B" else f"{n:.2f} {unit}"
        n /= 1024
    return f"{n:.2f} TiB"


def format_duration(s: float) -> str:
    if s is None or not math.isfinite(s):
        return "--:--"
    s = int(max(0, s))
    h, rem = divmod(s, 3600)
    m, sec = divmod(rem, 60)
    return f"{h:d}:{m:02d}:{sec:02d}" if h else f"{m:02d}:{sec:02d}"


def progress_bar(done: float, total: float, width: int = 30) -> str:
    frac = 0.0 if not total else min(1.0, max(0.0, done / total))
    full = int(frac * width)
    return "█" * full + "░" * (width - full) + f" {frac * 100:5.1f}%"


class OomRiskLevel(enum.Enum):
    LOW = "low"
    MEDIUM = "medium"
    HIGH = "high"
    CRITICAL = "critical"

    @classmethod
    def from_ratio(cls, ratio: float) -> "OomRiskLevel":
        return cls.LOW if ratio < 0.5 else cls.MEDIUM if ratio < 0.75 else cls.HIGH if ratio < 0.9 else cls.CRITICAL

    @property
    def color(self) -> str:
        return {"low": "green", "medium": "yellow", "high": "red", "critical": "bright_red"}[self.value]


@dataclass
class DashboardConfig:
    title: str = "rustral-b200"
    history_len: int = 120          # points kept per metric
    refresh_ms: int = 250
    dump_path: str | None = None    # when set, every frame also writes the state there as JSON
    alt_screen: bool = True         # draw on the terminal's alternate screen and restore it on exit


@dataclass
class LeakWarning:
    tag: str
    nbytes: int
    detected_at: float
    allocation_count: int = 1


@dataclass
class EpochSnapshot:
    epoch: int
    loss: float
    accuracy: float | None = None
    examples_per_sec: float = 0.0

    def push_to_dashboard(self, dash: "TrainingDashboard") -> None:
        dash.push_epoch(self)


class TrainingDashboard:
    """State of a run as the dashboard shows it.  Every method may be called from any thread."""

    def __init__(self, title: str | DashboardConfig = "rustral-b200", config: DashboardConfig | None = None):
        if isinstance(title, DashboardConfig):
            config, title = title, title.title
        self.config = config or DashboardConfig(title=title)
        self.title = self.config.title
        self._lock = threading.RLock()
        self.started = time.time()
        self.losses: list = []
        self.accuracies: list = []
        self.lrs: list = []
        self.memory_history: list = []
        self.epoch = self.total_epochs = self.batch = self.total_batches = self.step = 0
        self.samples_seen = 0
        self.throughput = 0.0
        self._rate_t, self._rate_n = None, 0
        self.memory_used = self.memory_peak = self.memory_capacity = 0
        self.memory_by_tag: list = []
        self.allocs = self.deallocs = 0
        self.unstable_allocations = 0
        self.leaks: list = []
        self.warnings: list = []
        self.events: list = []
        self._profiler = None
        self._leak_age_s = 30.0

    # ---- progress ---------------------------------------------------------------------------------------------
    def set_total_epochs(self, n: int) -> None:
        with self._lock:
            self.total_epochs = int(n)

    def set_total_batches(self, n: int) -> None:
        with self._lock:
            self.total_batches = int(n)

    def set_epoch(self, e: int) -> None:
        with self._lock:
            self.epoch = int(e)

    def set_batch(self, b: int) -> None:
        with self._lock:
            self.batch = int(b)

    def set_step(self, s: int) -> None:
        with self._lock:
            self.step = int(s)

    def reset_epoch(self) -> None:
        with self._lock:
            self.batch = 0

    def record_batch_samples(self, n: int) -> None:
        """Counts samples; the throughput shown is the rate over the last second or more."""
        now = time.time()
        with self._lock:
            self.samples_seen += int(n)
            if self._rate_t is None:
                self._rate_t, self._rate_n = now, 0
            self._rate_n += int(n)
            if now - self._rate_t >= 1.0:
                self.throughput = self._rate_n / (now - self._rate_t)
                self._rate_t, self._rate_n = now, 0
                self._rate_settled = True
            elif not getattr(self, "_rate_settled", False) and now > self._rate_t:
                self.throughput = self._rate_n / (now - self._rate_t)     # provisional until the first full second

    def _push(self, hist: list, v: float) -> None:
        hist.append(float(v))
        del hist[:-self.config.history_len]

    # ---- metrics ----------------------------------------------------------------------------------------------
    def record_loss(self, loss: float) -> None:
        with self._lock:
            if not math.isfinite(loss):
                self.add_warning(f"non-finite loss at step {self.step}: {loss}")
            self._push(self.losses, loss)

    def record_accuracy(self, acc: float) -> None:
        with self._lock:
            self._push(self.accuracies, acc)

    def record_lr(self, lr: float) -> None:
        with self._lock:
            self._push(self.lrs, lr)

    def push_epoch(self, s: EpochSnapshot) -> None:
        with self._lock:
            self.epoch = s.epoch
            self.record_loss(s.loss)
            if s.accuracy is not None:
                self.record_accuracy(s.accuracy)
            if s.examples_per_sec:
                self.throughput = s.examples_per_sec

    def push_scalar(self, name: str, value: float) -> None:
        low = name.lower()
        if "loss" in low:
            self.record_loss(value)
        elif "acc" in low:
            self.record_accuracy(value)
        elif low in ("lr", "learning_rate") or low.endswith("/lr"):
            self.record_lr(value)

    def current_loss(self):
        with self._lock:
            return self.losses[-1] if self.losses else None

    def current_accuracy(self):
        with self._lock:
            return self.accuracies[-1] if self.accuracies else None

    def current_lr(self):
        with self._lock:
            return self.lrs[-1] if self.lrs else None

    # ---- memory -----------------------------------------------------------------------------------------------
    def set_memory(self, used: int, capacity: int) -> None:
        with self._lock:
            self.memory_used, self.memory_capacity = int(used), int(capacity)
            self.memory_peak = max(self.memory_peak, self.memory_used)
            self._push(self.memory_history, used)

    def set_memory_bytes(self, used: int) -> None:
        self.set_memory(used, self.memory_capacity)

    def set_peak_memory(self, nbytes: int) -> None:
        with self._lock:
            self.memory_peak = int(nbytes)

    def set_available_memory(self, nbytes: int) -> None:
        with self._lock:
            self.memory_capacity = int(nbytes)

    def set_memory_by_tag(self, by_tag) -> None:
        with self._lock:
            self.memory_by_tag = sorted(((str(t), int(n)) for t, n in by_tag), key=lambda kv: -kv[1])

    def set_allocation_counts(self, allocs: int, deallocs: int) -> None:
        with self._lock:
            self.allocs, self.deallocs = int(allocs), int(deallocs)

    def report_leak(self, tag: str, nbytes: int, allocation_count: int = 1) -> None:
        with self._lock:
            for l in self.leaks:
                if l.tag == tag:
                    l.nbytes, l.allocation_count = int(nbytes), int(allocation_count)
                    return
            self.leaks.append(LeakWarning(tag, int(nbytes), time.time(), int(allocation_count)))

    def report_unstable_allocations(self, count: int) -> None:
        with self._lock:
            self.unstable_allocations = int(count)

    def clear_leaks(self) -> None:
        with self._lock:
            self.leaks = []

    def has_leaks(self) -> bool:
        with self._lock:
            return bool(self.leaks)

    def oom_risk_level(self) -> OomRiskLevel | None:
        with self._lock:
            return OomRiskLevel.from_ratio(self.memory_used / self.memory_capacity) if self.memory_capacity else None

    def oom_risk(self) -> str:
        lvl = self.oom_risk_level()
        return "unknown" if lvl is None else lvl.value

    def attach_memory_profiler(self, profiler, leak_age_s: float = 30.0) -> None:
        """Feeds the memory pane and the leak warnings from a `core.MemoryProfiler`: allocations still live after
        `leak_age_s` seconds are reported as leaks (grouped by tag), on every `poll_memory_profiler` call (the render
        loop makes one per frame)."""
        with self._lock:
            self._profiler, self._leak_age_s = profiler, float(leak_age_s)

    def poll_memory_profiler(self) -> None:
        prof = self._profiler
        if prof is None:
            return
        by_tag, grouped = {}, {}
        for _, (tag, n, _) in list(prof.active.items()):
            by_tag[tag] = by_tag.get(tag, 0) + n
        for _, tag, n in prof.find_leaks(self._leak_age_s):
            tot, cnt = grouped.get(tag, (0, 0))
            grouped[tag] = (tot + n, cnt + 1)
        allocs = sum(1 for e in prof.events if getattr(e, "kind", "alloc") == "alloc")
        with self._lock:
            self.set_memory(prof.current, prof.capacity_bytes if prof.capacity_bytes < (1 << 60) else self.memory_capacity)
            self.memory_peak = max(self.memory_peak, prof.peak)
            self.set_memory_by_tag(by_tag.items())
            self.set_allocation_counts(allocs, len(prof.events) - allocs)
            live = set(grouped)
            self.leaks = [l for l in self.leaks if l.tag in live]
            for tag, (tot, cnt) in grouped.items():
                self.report_leak(tag, tot, cnt)

    # ---- warnings and events ----------------------------------------------------------------------------------
    def add_warning(self, msg: str) -> None:
        with self._lock:
            self.warnings.append(str(msg))
            del self.warnings[:-8]

    warn = add_warning

    def log_event(self, msg: str) -> None:
        with self._lock:
            self.events.append((time.time(), str(msg)))
            del self.events[:-20]

    # ---- derived ----------------------------------------------------------------------------------------------
    def elapsed(self) -> float:
        return time.time() - self.started

    def eta_seconds(self) -> float | None:
        with self._lock:
            total = self.total_epochs * self.total_batches if self.total_batches else self.total_epochs
            done = self.epoch * self.total_batches + self.batch if self.total_batches else self.epoch
            if not total or done <= 0:
                return None
            return self.elapsed() * (total - done) / done

    def throughput_str(self) -> str:
        t = self.throughput
        return f"{t / 1e6:.2f} M/s" if t >= 1e6 else f"{t / 1e3:.1f} k/s" if t >= 1e3 else f"{t:.1f}/s"

    def eta_str(self) -> str:
        return format_duration(self.eta_seconds())

    def dump_metrics(self) -> str:
        with self._lock:
            lvl = self.oom_risk_level()
            return json.dumps({
                "title": self.title, "epoch": self.epoch, "total_epochs": self.total_epochs, "batch": self.batch,
                "total_batches": self.total_batches, "step": self.step, "elapsed_s": round(self.elapsed(), 3),
                "eta_s": self.eta_seconds(), "throughput": self.throughput, "samples_seen": self.samples_seen,
                "loss": self.current_loss(), "accuracy": self.current_accuracy(), "lr": self.current_lr(),
                "loss_history": list(self.losses), "memory": {"used": self.memory_used, "peak": self.memory_peak,
                                                              "capacity": self.memory_capacity,
                                                              "oom_risk": None if lvl is None else lvl.value,
                                                              "by_tag": self.memory_by_tag, "allocs": self.allocs,
                                                              "deallocs": self.deallocs},
                "leaks": [{"tag": l.tag, "bytes": l.nbytes, "allocations": l.allocation_count} for l in self.leaks],
                "unstable_allocations": self.unstable_allocations, "warnings": list(self.warnings),
                "events": [m for _, m in self.events]})


# ------------------------------------------------------------------------------------------------------ drawing
def _box(title: str, lines: list, width: int) -> list:
    inner = width - 2
    head = f"─ {title} "
    out = ["┌" + head + "─" * max(0, inner - len(head)) + "┐"]
    for ln in lines:
        vis = _visible_len(ln)
        if vis > inner:
            ln, vis = _clip(ln, inner), inner
        out.append("│" + ln + " " * (inner - vis) + "│")
    out.append("└" + "─" * inner + "┘")
    return out


def _visible_len(s: str) -> int:
    n, i = 0, 0
    while i < len(s):
        if s[i] == "\x1b":
            j = s.find("m", i)
            i = len(s) if j < 0 else j + 1
        else:
            n += 1
            i += 1
    return n


def _clip(s: str, width: int) -> str:
    out, n, i = [], 0, 0
    while i < len(s) and n < width:
        if s[i] == "\x1b":
            j = s.find("m", i)
            j = len(s) - 1 if j < 0 else j
            out.append(s[i:j + 1])
            i = j + 1
        else:
            out.append(s[i])
            n += 1
            i += 1
    return "".join(out) + (_COLORS["reset"] if "\x1b" in s else "")


class DashboardRenderer:
    """Draws a `TrainingDashboard`.  `render_text` is the compact form (one block of lines); `render_panes` the four
    boxed panels.  `render_frame` draws once and polls the keyboard; `run` repeats that until `q` or `stop()`."""

    def __init__(self, dash: TrainingDashboard, file=None, ansi: bool = True, width: int | None = None, keys=None):
        self.dash, self.file, self.ansi = dash, file or sys.stderr, ansi
        self.width = width
        self.running = True
        self.paused = False
        self._keys = keys                    # callable returning pending characters (tests); default: the terminal
        self._term_state = None
        self._alt = False

    # ---- text -------------------------------------------------------------------------------------------------
    def _c(self, name: str, text: str) -> str:
        return f"{_COLORS[name]}{text}{_COLORS['reset']}" if self.ansi else text

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
            lines += [f"! leak {l.tag}: {format_bytes(l.nbytes)} in {l.allocation_count} allocation(s)" for l in d.leaks]
            lines += [f"! {w}" for w in d.warnings[-5:]]
        return "\n".join(lines)

    def _progress_pane(self, w: int) -> list:
        d = self.dash
        bar_w = max(10, w - 34)
        lines = []
        if d.total_epochs:
            lines.append(f" epoch {d.epoch:>5}/{d.total_epochs:<5} {progress_bar(d.epoch, d.total_epochs, bar_w)}")
        else:
            lines.append(f" epoch {d.epoch}")
        if d.total_batches:
            lines.append(f" batch {d.batch:>5}/{d.total_batches:<5} {progress_bar(d.batch, d.total_batches, bar_w)}")
        lines.append(f" step {d.step}   elapsed {format_duration(d.elapsed())}   ETA {d.eta_str()}   throughput {d.throughput_str()}")
        return _box("progress", lines, w)

    def _metrics_pane(self, w: int) -> list:
        d = self.dash
        sw = max(8, min(d.config.history_len, w - 30))
        lines = []
        for name, hist, fmt in (("loss", d.losses, "{:.4f}"), ("accuracy", d.accuracies, "{:.4f}"), ("lr", d.lrs, "{:.3e}")):
            if hist:
                lines.append(f" {name:<9}{fmt.format(hist[-1]):>12}  {self._c('cyan', sparkline(hist, sw))}")
        if d.losses and len(d.losses) > 1:
            finite = [v for v in d.losses if math.isfinite(v)]
            if finite:
                lines.append(f" loss min {min(finite):.4f}  max {max(finite):.4f}  over {len(d.losses)} points")
        return _box("metrics", lines or [" (no metrics yet)"], w)

    def _memory_pane(self, w: int) -> list:
        d = self.dash
        lines = []
        lvl = d.oom_risk_level()
        if d.memory_capacity:
            bar = progress_bar(d.memory_used, d.memory_capacity, max(10, w - 48))
            lines.append(f" used {format_bytes(d.memory_used):>11} / {format_bytes(d.memory_capacity):<11} {self._c(lvl.color, bar)}")
            lines.append(f" peak {format_bytes(d.memory_peak):>11}   OOM risk: {self._c(lvl.color, lvl.value.upper())}")
        else:
            lines.append(f" used {format_bytes(d.memory_used)}   peak {format_bytes(d.memory_peak)}")
        if d.memory_history:
            lines.append(f" history {self._c('cyan', sparkline(d.memory_history, max(8, w - 14)))}")
        if d.allocs or d.deallocs:
            lines.append(f" allocations {d.allocs}  frees {d.deallocs}  live {d.allocs - d.deallocs}"
                         + (f"  unstable {d.unstable_allocations}" if d.unstable_allocations else ""))
        for tag, n in d.memory_by_tag[:5]:
            lines.append(f"   {tag:<24.24} {format_bytes(n):>12}")
        return _box("memory", lines, w)

    def _warnings_pane(self, w: int) -> list:
        d = self.dash
        lines = []
        for l in d.leaks:
            lines.append(self._c("red", f" LEAK {l.tag}: {format_bytes(l.nbytes)} held by {l.allocation_count} allocation(s) "
                                        f"for {format_duration(time.time() - l.detected_at)}"))
        lvl = d.oom_risk_level()
        if lvl in (OomRiskLevel.HIGH, OomRiskLevel.CRITICAL):
            lines.append(self._c(lvl.color, f" memory at {100 * d.memory_used / d.memory_capacity:.0f} % of capacity"))
        lines += [self._c("yellow", f" {wmsg}") for wmsg in d.warnings[-5:]]
        lines += [f" {format_duration(t - d.started)} {m}" for t, m in d.events[-4:]]
        return _box("warnings and events", lines or [" none"], w)

    def render_panes(self, width: int | None = None) -> str:
        w = width or self.width or _terminal_width()
        d = self.dash
        with d._lock:
            head = self._c("bold", f" {d.title} ") + ("  [paused]" if self.paused else "") + "   q quit · p pause · c clear leaks"
            rows = [head] + self._progress_pane(w) + self._metrics_pane(w) + self._memory_pane(w) + self._warnings_pane(w)
        return "\n".join(rows)

    def draw(self) -> None:
        text = self.render_panes() if self.ansi else self.render_text()
        if self.ansi:
            self.file.write("\x1b[2J\x1b[H")
        self.file.write(text + "\n")
        self.file.flush()

    # ---- keyboard ---------------------------------------------------------------------------------------------
    def _pending_keys(self) -> str:
        if self._keys is not None:
            return self._keys()
        try:
            if not sys.stdin.isatty():
                return ""
            import select
            out = ""
            while select.select([sys.stdin], [], [], 0)[0]:
                ch = os.read(sys.stdin.fileno(), 1).decode(errors="ignore")
                if not ch:
                    break
                out += ch
            return out
        except (OSError, ValueError):
            return ""

    def handle_key(self, ch: str) -> bool:
        """Returns True when the key asks to quit."""
        if ch in ("q", "Q", "\x03"):
            self.running = False
            return True
        if ch in ("p", "P", " "):
            self.paused = not self.paused
        elif ch in ("c", "C"):
            self.dash.clear_leaks()
        return False

    def enter(self) -> None:
        """Terminal set-up for interactive use: alternate screen, keys delivered unbuffered and unechoed."""
        if self.ansi and self.dash.config.alt_screen:
            self.file.write("\x1b[?1049h\x1b[?25l")
            self._alt = True
        try:
            if self._keys is None and sys.stdin.isatty():
                import termios
                import tty
                self._term_state = termios.tcgetattr(sys.stdin.fileno())
                tty.setcbreak(sys.stdin.fileno())
        except (ImportError, OSError, ValueError):
            self._term_state = None

    def leave(self) -> None:
        if self._term_state is not None:
            import termios
            termios.tcsetattr(sys.stdin.fileno(), termios.TCSADRAIN, self._term_state)
            self._term_state = None
        if self._alt:
            self.file.write("\x1b[?25h\x1b[?1049l")
            self.file.flush()
            self._alt = False

    def render_frame(self) -> bool:
        """Handles pending keys, refreshes the memory pane from an attached profiler, draws (unless paused) and, with a
        `dump_path`, writes the JSON state.  Returns True when `q` was pressed."""
        for ch in self._pending_keys():
            if self.handle_key(ch):
                return True
        self.dash.poll_memory_profiler()
        if not self.paused:
            self.draw()
        path = self.dash.config.dump_path
        if path:
            tmp = path + ".tmp"
            with open(tmp, "w") as f:
                f.write(self.dash.dump_metrics())
            os.replace(tmp, path)
        return False

    def run(self, stop_event: threading.Event | None = None) -> None:
        """Draws until `q` is pressed, `stop()` is called or `stop_event` is set."""
        self.enter()
        try:
            while self.running and not (stop_event is not None and stop_event.is_set()):
                if self.render_frame():
                    break
                time.sleep(self.dash.config.refresh_ms / 1e3)
        finally:
            self.leave()

    def is_running(self) -> bool:
        return self.running

    def stop(self) -> None:
        self.running = False


def _terminal_width() -> int:
    try:
        return max(60, min(140, os.get_terminal_size().columns))
    except OSError:
        return 100


class TuiMetricsBackend(MetricsBackend):
    def __init__(self, dash: TrainingDashboard | None = None, config: DashboardConfig | None = None):
        self.dash = dash if dash is not None else TrainingDashboard(config=config or DashboardConfig())

    def dashboard(self) -> TrainingDashboard:
        return self.dash

    def log_scalar(self, m) -> None:
        step = getattr(m, "step", None)
        if step is not None:
            self.dash.set_step(step)
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


def run_dashboard(dash: TrainingDashboard | DashboardConfig, refresh_s: float | None = None, file=None,
                  stop_event: threading.Event | None = None):
    """Renders `dash` from a daemon thread (device memory is sampled before every frame when CUDA is present).  Returns
    the thread; `thread.stop_event.set()` ends it, `thread.renderer` is its `DashboardRenderer`.  Given a
    `DashboardConfig` instead of a dashboard, creates the dashboard and returns it (`dashboard.render_thread`)."""
    made = None
    if isinstance(dash, DashboardConfig):
        made = dash = TrainingDashboard(config=dash)
    if refresh_s is not None:
        dash.config.refresh_ms = int(refresh_s * 1e3)
    out = file or sys.stderr
    interactive = hasattr(out, "isatty") and out.isatty()
    r = DashboardRenderer(dash, out, ansi=True)
    if not interactive:
        dash.config.alt_screen = False
    stop = stop_event or threading.Event()

    def loop():
        r.enter()
        try:
            while not stop.wait(dash.config.refresh_ms / 1e3) and r.running:
                try:
                    import torch
                    if torch.cuda.is_available() and dash._profiler is None:
                        free, total = torch.cuda.mem_get_info()
                        dash.set_memory(total - free, total)
                except Exception:   # noqa: BLE001 - the dashboard must never take training down
                    pass
                if r.render_frame():
                    break
        finally:
            r.leave()

    t = threading.Thread(target=loop, daemon=True)
    t.stop_event = stop
    t.renderer = r
    t.start()
    if made is not None:
        made.render_thread = t
        return made
    return t
