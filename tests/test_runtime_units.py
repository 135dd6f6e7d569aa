"""Runtime pieces one by one: the thread-parallel `ParallelTrainer` / `Learner` pair, the bounded `InferencePool`, strict
model loading, the synthetic end-to-end run and the dashboard hook of the tape trainer
(crates/runtime/src/{trainer,inference,model_io,serious_training,tui_hook}.rs `mod tests`)."""
import threading
import time

import pytest
import torch

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.core.errors import SerializationError, ShapeMismatch
from rustral_b200.nn import LinearBuilder, Sequential
from rustral_b200.optim import Adam
from rustral_b200.runtime.inference import InferencePool, PoolClosed
from rustral_b200.runtime.model_io import load_model, load_model_from_path, save_model, save_model_to_path
from rustral_b200.runtime.serious_training import SeriousTrainingConfig, train_synthetic_classification
from rustral_b200.runtime.trainer import Learner, ParallelTrainer, TrainerConfig

BE = CpuBackend()


# ---- ParallelTrainer ------------------------------------------------------------------------------------------------
class _LineFit(Learner):
    """y = w x + b by per-example gradients merged into their mean."""

    def __init__(self, lr):
        self.w, self.b, self.lr = 0.0, 0.0, lr
        self.threads = set()
        self.applied = 0

    def loss_and_update(self, datum):
        self.threads.add(threading.get_ident())
        x, y = datum
        err = self.w * x + self.b - y
        return err * err, (2 * err * x, 2 * err)

    def merge_updates(self, updates):
        n = len(updates)
        return sum(u[0] for u in updates) / n, sum(u[1] for u in updates) / n

    def apply_update(self, update):
        self.w -= self.lr * update[0]
        self.b -= self.lr * update[1]
        self.applied += 1


def test_parallel_trainer_fits_a_line_and_applies_one_update_per_batch():
    data = [(x / 10.0, 3.0 * x / 10.0 - 1.0) for x in range(-20, 20)]
    learner = _LineFit(0.1)
    stats = ParallelTrainer(TrainerConfig(epochs=60, batch_size=8, parallelism=4)).train(learner, data)
    assert learner.w == pytest.approx(3.0, abs=0.05) and learner.b == pytest.approx(-1.0, abs=0.05)
    assert learner.applied == 60 * 5 and len(stats) == 60 and [s.epoch for s in stats[:3]] == [0, 1, 2]
    assert stats[0].examples == 40 and stats[-1].mean_loss < 1e-3 < stats[0].mean_loss
    assert len(learner.threads) >= 1 and threading.get_ident() not in learner.threads     # the work ran on pool threads


def test_parallel_trainer_result_does_not_depend_on_the_number_of_threads():
    data = [(x / 7.0, 0.5 * x / 7.0 + 2.0) for x in range(30)]
    out = []
    for par in (1, 3):
        l = _LineFit(0.05)
        ParallelTrainer(TrainerConfig(epochs=5, batch_size=6, parallelism=par)).train(l, data)
        out.append((l.w, l.b))
    assert out[0] == out[1]                        # results are merged in input order, so the sums are identical


# ---- InferencePool --------------------------------------------------------------------------------------------------
def test_inference_pool_answers_every_caller_and_delivers_exceptions():
    def handler(x):
        if x < 0:
            raise ValueError(f"negative input {x}")
        time.sleep(0.002)
        return x * x
    pool = InferencePool(workers=3, queue_bound=4, handler=handler)
    results = {}

    def call(i):
        results[i] = pool.infer(i)
    ts = [threading.Thread(target=call, args=(i,)) for i in range(20)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert results == {i: i * i for i in range(20)}
    with pytest.raises(ValueError, match="negative input -3"):
        pool.infer(-3)
    assert pool.infer(5) == 25                                         # the worker survived the exception
    pool.shutdown()
    with pytest.raises(PoolClosed):
        pool.infer(1)
    pool.shutdown()                                                    # idempotent


def test_inference_pool_applies_back_pressure_and_times_out():
    gate = threading.Event()
    pool = InferencePool(workers=1, queue_bound=1, handler=lambda x: (gate.wait(5), x)[1])
    first = threading.Thread(target=pool.infer, args=(1,))
    first.start()
    time.sleep(0.05)                                                   # the worker now holds request 1
    second = threading.Thread(target=pool.infer, args=(2,))
    second.start()
    time.sleep(0.05)                                                   # request 2 fills the queue
    import queue
    with pytest.raises((queue.Full, TimeoutError)):
        pool.infer(3, timeout=0.05)                                    # no room: the caller is held, then gives up
    gate.set()
    first.join(); second.join()
    assert pool.infer(4) == 4
    pool.shutdown()


# ---- strict model loading -------------------------------------------------------------------------------------------
def _mlp(seed, hidden=8):
    return Sequential(LinearBuilder(4, hidden).with_bias().seed(seed).build(BE), LinearBuilder(hidden, 2).with_bias().seed(seed + 1).build(BE))


def test_load_model_is_strict_and_changes_nothing_when_it_refuses(tmp_path):
    a, b = _mlp(1), _mlp(2)
    blob = save_model(a)
    before = [p.tensor.clone() for p in b.parameters()]
    with pytest.raises(ShapeMismatch):
        load_model(_mlp(3, hidden=9), blob)
    with pytest.raises(SerializationError, match="missing keys"):
        load_model(Sequential(*a.layers, LinearBuilder(2, 2).build(BE)), blob)
    with pytest.raises(SerializationError, match="unexpected keys"):
        load_model(Sequential(a.layers[0]), blob)
    with pytest.raises(SerializationError):
        load_model(b, blob[:40])
    assert all(torch.equal(x, p.tensor) for x, p in zip(before, b.parameters()))
    path = tmp_path / "m.safetensors"
    save_model_to_path(a, str(path))
    assert not (tmp_path / "m.safetensors.partial").exists()
    load_model_from_path(b, str(path))
    x = torch.randn(3, 4)
    assert torch.equal(a(x), b(x))


# ---- synthetic end-to-end run ---------------------------------------------------------------------------------------
def test_synthetic_classification_learns_and_round_trips_its_checkpoint(tmp_path):
    out = train_synthetic_classification(BE, SeriousTrainingConfig(epochs=120, checkpoint_dir=str(tmp_path)))
    assert out.loss_end < 0.25 * out.loss_start and out.checkpoint_roundtrip_ok
    assert (tmp_path / "mid.safetensors").stat().st_size > 100
    again = train_synthetic_classification(BE, SeriousTrainingConfig(epochs=120))
    assert again.loss_end == out.loss_end                              # LCG data + seeded init: bit-reproducible


# ---- dashboard hook -------------------------------------------------------------------------------------------------
def test_dashboard_hook_receives_the_trainers_loss_accuracy_and_rate():
    from rustral_b200.core.module import Module, Trainable
    from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer
    from rustral_b200.runtime.tui_hook import TuiHook

    class M(Module, Trainable, SupervisedTapeModel):
        def __init__(self):
            self.lin = LinearBuilder(2, 2).with_bias().seed(1).build(BE)

        def forward_tape(self, x, tape, ctx):
            return tape.apply("lin", lambda: self.lin(x, ctx))
    hook = TuiHook(start_thread=False)
    data = [([1.0, 0.0], 0), ([0.0, 1.0], 1)] * 8
    builder = Trainer.classification(Adam(0.1)).epochs(5).batch_size(4)
    builder.on_epoch = hook.on_epoch
    report = builder.fit(BE, M(), data)
    d = hook.dashboard
    assert len(d.losses) == 5 and d.losses == pytest.approx([e.mean_loss for e in report.epochs])
    assert d.losses[-1] < d.losses[0] and d.losses[0] > 0.1            # real losses, not a default of zero
    assert d.accuracies[-1] == 1.0 and d.epoch == 4 and d.throughput > 0


def test_trainer_builder_sends_epoch_summaries_to_a_metrics_logger(tmp_path):
    import json
    from rustral_b200.core.module import Module, Trainable
    from rustral_b200.metrics import MetricsLogger, TensorBoardWriter
    from rustral_b200.runtime.tape_trainer import SupervisedTapeModel, Trainer

    class M(Module, Trainable, SupervisedTapeModel):
        def __init__(self):
            self.lin = LinearBuilder(2, 2).with_bias().seed(1).build(BE)

        def forward_tape(self, x, tape, ctx):
            return tape.apply("lin", lambda: self.lin(x, ctx))
    seen = []
    log = MetricsLogger([TensorBoardWriter(str(tmp_path), "fit")])
    data = [([1.0, 0.0], 0), ([0.0, 1.0], 1)] * 8
    report = Trainer.classification(Adam(0.1)).epochs(3).batch_size(4).metrics(log).epoch_callback(seen.append).fit(BE, M(), data)
    rows = [json.loads(l) for l in open(tmp_path / "fit.jsonl")]
    losses = [r["value"] for r in rows if r["name"] == "train/loss"]
    assert losses == pytest.approx([e.mean_loss for e in report.epochs]) and [r["step"] for r in rows if r["name"] == "train/loss"] == [0, 1, 2]
    assert [r["value"] for r in rows if r["name"] == "train/accuracy"][-1] == report.accuracy
    assert [r["value"] for r in rows if r["name"] == "train/lr"] == [0.1, 0.1, 0.1]
    assert [s.epoch for s in seen] == [0, 1, 2] and seen[-1].mean_loss == report.epochs[-1].mean_loss
