"""Dashboard hook for the trainers (crates/runtime/src/tui_hook.rs:23: init_global_dashboard + per-epoch push).

`attach_dashboard(trainer)` starts the text dashboard on a background thread and makes the trainer push an
`EpochSnapshot` after every epoch; `TuiHook` is the object form for code that manages the thread itself."""
from __future__ import annotations

import threading

import torch

from ..utils.tui import EpochSnapshot, TrainingDashboard, init_global_dashboard, run_dashboard


class TuiHook:
    def __init__(self, dashboard: TrainingDashboard | None = None, title: str = "rustral-b200", refresh_s: float = 0.5,
                 file=None, start_thread: bool = True):
        self.stop_event = threading.Event()
        if dashboard is None and start_thread:
            self.dashboard = init_global_dashboard(title, refresh_s, file)
            self.thread = None
        else:
            self.dashboard = dashboard if dashboard is not None else TrainingDashboard(title=title)
            self.thread = run_dashboard(self.dashboard, refresh_s, file, self.stop_event) if start_thread else None

    def on_epoch(self, stats) -> None:
        """`stats` is what a trainer reports per epoch: the tape trainers' `EpochStats` (epoch, examples, mean_loss,
        elapsed, accuracy) or any object with `train_loss` / `loss` and `samples_per_s` / `examples_per_sec`."""
        loss = next((getattr(stats, k) for k in ("mean_loss", "train_loss", "loss") if getattr(stats, k, None) is not None), 0.0)
        rate = next((getattr(stats, k) for k in ("samples_per_s", "examples_per_sec") if getattr(stats, k, None)), None)
        if rate is None:
            n, dt = getattr(stats, "examples", None), getattr(stats, "elapsed", None)
            rate = n / dt if n and dt else 0.0
        snap = EpochSnapshot(epoch=int(getattr(stats, "epoch", 0)), loss=float(loss),
                             accuracy=getattr(stats, "accuracy", None), examples_per_sec=float(rate))
        snap.push_to_dashboard(self.dashboard)
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info()
            self.dashboard.set_memory(total - free, total)

    def close(self) -> None:
        self.stop_event.set()


def attach_dashboard(trainer, **kw) -> TuiHook:
    hook = TuiHook(**kw)
    trainer.on_epoch = hook.on_epoch
    return hook
