"""ParallelTrainer / Learner: thread data parallelism over a batch on the host
(crates/runtime/src/trainer.rs:8-112).  Kept for CPU-side models; GPU training goes through LMTrainer / TapeTrainer."""
from __future__ import annotations

import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

from .tape_trainer import EpochStats


@dataclass
class TrainerConfig:
    epochs: int = 1
    batch_size: int = 32
    parallelism: int = 4


class Learner:
    """loss_and_update(datum) -> (loss, update); merge_updates(list) -> update; apply_update(update)."""

    def loss_and_update(self, datum):
        raise NotImplementedError

    def merge_updates(self, updates):
        raise NotImplementedError

    def apply_update(self, update) -> None:
        raise NotImplementedError


class ParallelTrainer:
    def __init__(self, config: TrainerConfig):
        self.config = config

    def train(self, learner: Learner, data) -> list:
        data = list(data)
        stats = []
        with ThreadPoolExecutor(max_workers=max(1, self.config.parallelism)) as ex:
            for epoch in range(self.config.epochs):
                t0, total, n = time.perf_counter(), 0.0, 0
                for b0 in range(0, len(data), self.config.batch_size):
                    batch = data[b0:b0 + self.config.batch_size]
                    results = list(ex.map(learner.loss_and_update, batch))
                    total += sum(r[0] for r in results)
                    n += len(results)
                    learner.apply_update(learner.merge_updates([r[1] for r in results]))
                stats.append(EpochStats(epoch, n, total / max(1, n), time.perf_counter() - t0))
        return stats
