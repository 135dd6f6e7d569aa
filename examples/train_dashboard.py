"""The terminal training dashboard driven by a real (small) training loop: progress with ETA and throughput, loss /
accuracy / learning-rate sparklines, the memory pane fed by a `MemoryProfiler` (with a deliberately long-lived
allocation so that a leak warning appears), and the warnings pane.  Keys: q quit, p pause, c clear leak warnings
(crates/tui/examples/train_dashboard.rs).

    python examples/train_dashboard.py                 # interactive, alternate screen
    python examples/train_dashboard.py --plain         # a few text frames on stdout, for logs and pipes
    python examples/train_dashboard.py --dump state.json
"""
import io
import sys
import time

import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx, MemoryProfiler
from rustral_b200.nn import CrossEntropyLoss, LinearBuilder, Sequential
from rustral_b200.optim import Adam, WarmupCosine
from rustral_b200.utils.tui import DashboardConfig, DashboardRenderer, TrainingDashboard, run_dashboard


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--epochs", type=int, default=4)
    ap.add_argument("--batches", type=int, default=25)
    ap.add_argument("--plain", action="store_true")
    ap.add_argument("--dump", default=None)
    ap.add_argument("--delay", type=float, default=0.0, help="seconds to sleep per batch, to watch the dashboard move")
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    dash = TrainingDashboard(DashboardConfig(title="dashboard demo", refresh_ms=100, dump_path=a.dump))
    dash.set_total_epochs(a.epochs)
    dash.set_total_batches(a.batches)
    mem = MemoryProfiler(capacity_bytes=64 << 20)
    dash.attach_memory_profiler(mem, leak_age_s=0.2)
    leaked = mem.alloc("forgotten_buffer", 3 << 20)                 # never freed: shows up as a leak after 0.2 s
    interactive = not a.plain and sys.stderr.isatty()
    thread = run_dashboard(dash, file=sys.stderr) if interactive else None

    g = torch.Generator().manual_seed(a.seed)
    centres = torch.randn(4, 16, generator=g) * 1.5
    model = Sequential(LinearBuilder(16, 64).with_bias().seed(a.seed).activation("gelu").build(backend),
                       LinearBuilder(64, 4).with_bias().seed(a.seed + 1).build(backend))
    opt = Adam(lr=1e-2)
    sched = WarmupCosine(1e-2, 1e-4, 10, a.epochs * a.batches).attach(opt)
    ce = CrossEntropyLoss()
    frames = []
    plain = DashboardRenderer(dash, io.StringIO(), ansi=False, width=100)
    for epoch in range(a.epochs):
        dash.set_epoch(epoch)
        dash.reset_epoch()
        for b in range(a.batches):
            y = torch.randint(0, 4, (64,), generator=g)
            x = (centres[y] + torch.randn(64, 16, generator=g)).to(dev, dt)
            with mem.track_tensor("batch", x):
                model.zero_grad()
                logits = model(x, ForwardCtx.train(backend)).float()
                loss = ce(logits, y.to(dev))
                loss.backward()
                opt.step(model.parameters())
                sched.step()
            dash.set_batch(b + 1)
            dash.set_step(epoch * a.batches + b + 1)
            dash.record_batch_samples(64)
            dash.record_loss(float(loss.detach()))
            dash.record_accuracy(float((logits.argmax(-1).cpu() == y).float().mean()))
            dash.record_lr(opt.lr)
            if a.delay:
                time.sleep(a.delay)
            if thread is not None and not thread.renderer.is_running():
                break
        dash.log_event(f"epoch {epoch} done, loss {dash.current_loss():.3f}")
        if not interactive:
            time.sleep(0.25 if epoch == 0 else 0.0)                # lets the forgotten buffer age past the leak threshold
            plain.render_frame()
            frames.append(plain.render_text())
        if thread is not None and not thread.renderer.is_running():
            break
    if thread is not None:
        thread.stop_event.set()
        thread.join(2.0)
    elif a.plain:
        print(frames[-1])
    mem.free(leaked)
    return {"frames": frames, "has_leaks": dash.has_leaks(), "loss": dash.current_loss(), "accuracy": dash.current_accuracy(),
            "state": dash.dump_metrics()}


if __name__ == "__main__":
    main()
