"""TapeTrainer: the supervised training loop of the reference (crates/runtime/src/tape_trainer.rs:44-485).

Same contract (`SupervisedTapeModel.forward_tape / loss_tape`, seeded per-epoch shuffle `seed ^ epoch * 0x9E37`,
EpochStats / ThroughputStats / TrainingReport, RUSTRAL_PROFILE hooks), but a batch is ONE batched forward and one
backward instead of one forward graph per example (tape_trainer.rs:368), and accuracy is read back once per batch.
"""
from __future__ import annotations

import random
import time
from dataclasses import dataclass, field

import torch

from ..autograd import Tape
from ..core import ForwardCtx
from ..core.operation_profiler import finish_profile_from_env, operation_profiler_from_env
from ..core.tensor_pool import pool_from_env


class SupervisedTapeModel:
    """forward_tape(x, tape, ctx) -> TensorId of the logits; loss_tape(logits, y, tape, ctx) -> TensorId of the loss.
    `collate(xs) / collate_targets(ys)` turn a list of examples into batch tensors (default: stack)."""

    def forward_tape(self, x, tape: Tape, ctx: ForwardCtx):
        raise NotImplementedError

    def loss_tape(self, logits, y, tape: Tape, ctx: ForwardCtx):
        return tape.cross_entropy_loss(logits, y)

    def collate(self, xs):
        return torch.stack([torch.as_tensor(x) for x in xs])

    def collate_targets(self, ys):
        return torch.as_tensor(ys)


@dataclass
class EpochStats:
    epoch: int
    examples: int
    mean_loss: float
    elapsed: float
    accuracy: float | None = None


@dataclass
class ThroughputStats:
    examples_per_sec: float
    batches_per_sec: float


@dataclass
class TrainingReport:
    epochs: list = field(default_factory=list)
    accuracy: float | None = None
    throughput: ThroughputStats | None = None


@dataclass
class TapeTrainerConfig:
    epochs: int = 1
    lr: float = 1e-3
    batch_size: int = 1
    shuffle: bool = True
    seed: int = 0


class TapeTrainer:
    def __init__(self, config: TapeTrainerConfig, optimizer, backend=None, metrics=None):
        self.config, self.optimizer, self.backend = config, optimizer, backend
        self.tensor_pool = pool_from_env()
        self.metrics = metrics
        self.on_epoch = None           # callback(EpochStats), e.g. the dashboard hook

    def train_model(self, model, data, closure=None) -> TrainingReport:
        return self._fit(model, data, classification=False)

    def fit(self, model, data) -> TrainingReport:
        return self._fit(model, data, classification=False)

    def fit_classification(self, model, data) -> TrainingReport:
        return self._fit(model, data, classification=True)

    def _fit(self, model, data, classification: bool) -> TrainingReport:
        cfg = self.config
        data = list(data)
        profiler = operation_profiler_from_env()
        report = TrainingReport()
        params = model.parameters()
        t_start, n_batches, n_examples = time.perf_counter(), 0, 0
        for epoch in range(cfg.epochs):
            idx = list(range(len(data)))
            if cfg.shuffle:
                random.Random(cfg.seed ^ (epoch * 0x9E37)).shuffle(idx)
            t0 = time.perf_counter()
            loss_sum, correct, seen = 0.0, 0, 0
            for b0 in range(0, len(idx), cfg.batch_size):
                batch = [data[i] for i in idx[b0:b0 + cfg.batch_size]]
                ctx = ForwardCtx.train(self.backend, profiler=profiler, seed=cfg.seed + epoch)
                tape = Tape(ctx)
                x = model.collate([ex[0] for ex in batch])
                y = model.collate_targets([ex[1] for ex in batch])
                logits = model.forward_tape(x, tape, ctx)
                loss = model.loss_tape(logits, y, tape, ctx)
                for p in params:
                    p.zero_grad()
                tape.values[loss].backward()
                # a parameter brought onto the tape with watch_parameter() is a separate leaf that shares the
                # parameter's storage: its gradient lands on that leaf and is handed to the parameter here
                for p in params:
                    tid = tape.param_map.get(p.id)
                    g = tape.values[tid].grad if tid is not None else None
                    if g is not None:
                        p.tensor.grad = g if p.tensor.grad is None else p.tensor.grad + g
                self.optimizer.step(params)
                if self.tensor_pool is not None:
                    self.tensor_pool.begin_step()
                loss_sum += float(tape.values[loss].detach()) * len(batch)
                seen += len(batch)
                if classification:
                    pred = tape.values[logits].detach().float().argmax(-1).cpu()
                    correct += int((pred == torch.as_tensor(y).cpu()).sum())
                n_batches += 1
            n_examples += seen
            st = EpochStats(epoch, seen, loss_sum / max(1, seen), time.perf_counter() - t0,
                            correct / max(1, seen) if classification else None)
            report.epochs.append(st)
            if self.metrics is not None:
                self.metrics.log_training_summary(epoch, st.mean_loss, st.accuracy, getattr(self.optimizer, "lr", None))
            if self.on_epoch is not None:
                self.on_epoch(st)
        dt = max(1e-9, time.perf_counter() - t_start)
        report.throughput = ThroughputStats(n_examples / dt, n_batches / dt)
        if classification and report.epochs:
            report.accuracy = report.epochs[-1].accuracy
        finish_profile_from_env(profiler)
        return report


class Classification:
    """Task marker of the `Trainer` builder (crates/runtime/src/high_level_trainer.rs:22): accuracy is tracked and the
    model's `loss_tape` defaults to cross-entropy.  `Trainer.for_task(Classification, opt)` is `Trainer.classification(opt)`."""


class Regression:
    """Task marker: no accuracy; the model supplies its own `loss_tape` (typically mean squared error)."""


class Trainer:
    """Builder: Trainer.classification(opt).epochs(3).batch_size(32).shuffle(True).seed(0).fit(backend, model, data)
    (crates/runtime/src/high_level_trainer.rs:22-94)."""

    def __init__(self, optimizer, classification: bool):
        self._opt, self._cls = optimizer, classification
        self._cfg = TapeTrainerConfig()
        self._metrics = None
        self.on_epoch = None           # callback(EpochStats); `attach_dashboard(builder)` sets it

    @classmethod
    def classification(cls, optimizer):
        return cls(optimizer, True)

    @classmethod
    def regression(cls, optimizer):
        return cls(optimizer, False)

    @classmethod
    def for_task(cls, task, optimizer):
        if task not in (Classification, Regression):
            raise ValueError("task must be Classification or Regression")
        return cls(optimizer, task is Classification)

    def epochs(self, n: int):
        self._cfg.epochs = n
        return self

    def batch_size(self, n: int):
        self._cfg.batch_size = n
        return self

    def shuffle(self, flag: bool):
        self._cfg.shuffle = flag
        return self

    def seed(self, s: int):
        self._cfg.seed = s
        return self

    def metrics(self, logger):
        """A `MetricsLogger` that receives the per-epoch training summary."""
        self._metrics = logger
        return self

    def epoch_callback(self, fn):
        self.on_epoch = fn
        return self

    def fit(self, backend, model, data) -> TrainingReport:
        tr = TapeTrainer(self._cfg, self._opt, backend, self._metrics)
        tr.on_epoch = self.on_epoch
        return tr.fit_classification(model, data) if self._cls else tr.fit(model, data)
