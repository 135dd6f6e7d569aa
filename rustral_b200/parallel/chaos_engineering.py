"""Seeded fault injection for resilience tests (crates/distributed/src/chaos_engineering.rs:46-582).

Faults are FLAGS decided on the host from a seeded generator: callers ask `can_communicate`, `get_delay_ms`,
`packet_lost`, or wrap a step in `run_with_faults`, which raises CommunicationError / sleeps / corrupts a checkpoint
file accordingly.  No fault is ever injected on a device: GPU out-of-memory and hardware-error faults are reported
to the caller as exceptions raised before any launch.
"""
from __future__ import annotations

import enum
import os
import random
import time
from dataclasses import dataclass, field

from .process_group import CommunicationError


class CheckpointCorruption(enum.Enum):
    BIT_FLIP = "bit_flip"
    TRUNCATED = "truncated"
    WRONG_CHECKSUM = "wrong_checksum"
    MISSING_KEYS = "missing_keys"


class FaultKind(enum.Enum):
    NETWORK_PARTITION = "network_partition"
    GPU_OUT_OF_MEMORY = "gpu_out_of_memory"
    GPU_HARDWARE_ERROR = "gpu_hardware_error"
    SLOW_WORKER = "slow_worker"
    PROCESS_CRASH = "process_crash"
    CORRUPTED_CHECKPOINT = "corrupted_checkpoint"
    MEMORY_LEAK = "memory_leak"
    PACKET_LOSS = "packet_loss"


@dataclass
class FaultType:
    kind: FaultKind
    delay_ms: float = 0.0
    loss_rate: float = 0.0
    corruption: CheckpointCorruption | None = None
    ranks: tuple = ()          # affected ranks; empty = chosen at trigger time


@dataclass
class FaultInjection:
    fault: FaultType
    trigger_probability: float = 0.01
    trigger_delay_ticks: int = 0
    duration_ticks: int = 1
    max_triggers: int = 1 << 30
    triggers: int = 0

    def should_trigger(self, rng: random.Random, tick: int) -> bool:
        if tick < self.trigger_delay_ticks or self.triggers >= self.max_triggers:
            return False
        return rng.random() < self.trigger_probability


@dataclass
class FaultResult:
    fault: FaultType
    tick: int
    ranks: tuple
    recovered: bool = False


@dataclass
class TestReport:
    ticks: int
    faults_triggered: int
    faults_recovered: int
    by_kind: dict = field(default_factory=dict)

    __test__ = False     # not a pytest class


class ChaosMonkey:
    def __init__(self, seed: int = 0, world_size: int = 1):
        self.rng = random.Random(seed)
        self.world_size = world_size
        self.injections: list = []
        self.active: list = []        # (FaultResult, expires_at_tick)
        self.history: list = []
        self.tick_count = 0

    def add_injection(self, inj: FaultInjection) -> None:
        self.injections.append(inj)

    def add_common_faults(self, world_size: int | None = None) -> None:
        """1% OOM, 5% slow worker (500 ms), 0.1% partition, 2% packet loss at 10%, rare crash
        (crates/distributed/src/chaos_engineering.rs:199-244)."""
        if world_size:
            self.world_size = world_size
        add = self.add_injection
        add(FaultInjection(FaultType(FaultKind.GPU_OUT_OF_MEMORY), 0.01))
        add(FaultInjection(FaultType(FaultKind.SLOW_WORKER, delay_ms=500.0), 0.05, duration_ticks=3))
        add(FaultInjection(FaultType(FaultKind.NETWORK_PARTITION), 0.001, duration_ticks=5))
        add(FaultInjection(FaultType(FaultKind.PACKET_LOSS, loss_rate=0.1), 0.02, duration_ticks=4))
        add(FaultInjection(FaultType(FaultKind.PROCESS_CRASH), 0.001))

    def tick(self) -> list:
        """Expires finished faults (marking them recovered) and triggers new ones; returns the new FaultResults."""
        self.tick_count += 1
        still = []
        for res, until in self.active:
            if self.tick_count >= until:
                res.recovered = True
            else:
                still.append((res, until))
        self.active = still
        new = []
        for inj in self.injections:
            if inj.should_trigger(self.rng, self.tick_count):
                inj.triggers += 1
                ranks = inj.fault.ranks or (self.rng.randrange(self.world_size),)
                if inj.fault.kind is FaultKind.NETWORK_PARTITION and not inj.fault.ranks:
                    half = max(1, self.world_size // 2)
                    ranks = tuple(sorted(self.rng.sample(range(self.world_size), half)))
                res = FaultResult(inj.fault, self.tick_count, tuple(ranks))
                self.active.append((res, self.tick_count + inj.duration_ticks))
                self.history.append(res)
                new.append(res)
        return new

    def _active_of(self, kind: FaultKind):
        return [r for r, _ in self.active if r.fault.kind is kind]

    def is_rank_affected(self, rank: int) -> bool:
        return any(rank in r.ranks for r, _ in self.active)

    def can_communicate(self, a: int, b: int) -> bool:
        for r in self._active_of(FaultKind.NETWORK_PARTITION):
            if (a in r.ranks) != (b in r.ranks):
                return False
        for r in self._active_of(FaultKind.PROCESS_CRASH):
            if a in r.ranks or b in r.ranks:
                return False
        return True

    def get_delay_ms(self, rank: int) -> float:
        return sum(r.fault.delay_ms for r in self._active_of(FaultKind.SLOW_WORKER) if rank in r.ranks)

    def packet_lost(self, a: int, b: int) -> bool:
        for r in self._active_of(FaultKind.PACKET_LOSS):
            if (a in r.ranks or b in r.ranks) and self.rng.random() < r.fault.loss_rate:
                return True
        return False

    def run_with_faults(self, fn, rank: int = 0, sleep=time.sleep):
        """tick(), then run `fn` under the faults active for `rank`: slow workers sleep first, crashes / partitions /
        device faults raise CommunicationError before `fn` is entered."""
        self.tick()
        for r, _ in self.active:
            if rank in r.ranks and r.fault.kind in (FaultKind.PROCESS_CRASH, FaultKind.GPU_HARDWARE_ERROR,
                                                     FaultKind.GPU_OUT_OF_MEMORY, FaultKind.NETWORK_PARTITION):
                raise CommunicationError(f"injected fault: {r.fault.kind.value} on rank {rank}")
        d = self.get_delay_ms(rank)
        if d > 0:
            sleep(d / 1e3)
        return fn()

    def generate_report(self) -> TestReport:
        by = {}
        for r in self.history:
            by[r.fault.kind.value] = by.get(r.fault.kind.value, 0) + 1
        return TestReport(self.tick_count, len(self.history), sum(1 for r in self.history if r.recovered), by)


def corrupt_checkpoint_file(path: str, how: CheckpointCorruption, seed: int = 0) -> None:
    """Damages a checkpoint file on disk the way the named corruption would."""
    rng = random.Random(seed)
    with open(path, "rb") as f:
        blob = bytearray(f.read())
    if how is CheckpointCorruption.TRUNCATED:
        blob = blob[:max(1, len(blob) // 2)]
    elif how is CheckpointCorruption.BIT_FLIP:
        i = rng.randrange(8, min(len(blob), 64))      # inside the header: guaranteed to be noticed
        blob[i] ^= 1 << rng.randrange(8)
    elif how is CheckpointCorruption.WRONG_CHECKSUM:
        blob[0:8] = (int.from_bytes(blob[0:8], "little") + 7).to_bytes(8, "little")
    else:
        import json
        import struct
        (hlen,) = struct.unpack("<Q", bytes(blob[:8]))
        header = json.loads(bytes(blob[8:8 + hlen]).decode())
        keys = [k for k in header if k != "__metadata__"]
        if keys:
            header.pop(keys[0])
        hj = json.dumps(header).encode()
        hj += b" " * ((8 - len(hj) % 8) % 8)
        blob = bytearray(struct.pack("<Q", len(hj)) + hj + bytes(blob[8 + hlen:]))
    with open(path, "wb") as f:
        f.write(bytes(blob))


class ChaosScenarios:
    @staticmethod
    def slow_worker(world_size: int, rank: int = 0, delay_ms: float = 500.0, seed: int = 0) -> ChaosMonkey:
        m = ChaosMonkey(seed, world_size)
        m.add_injection(FaultInjection(FaultType(FaultKind.SLOW_WORKER, delay_ms=delay_ms, ranks=(rank,)), 1.0, duration_ticks=1 << 30,
                                       max_triggers=1))
        return m

    @staticmethod
    def network_partition(world_size: int, seed: int = 0, at_tick: int = 3, duration: int = 5) -> ChaosMonkey:
        m = ChaosMonkey(seed, world_size)
        m.add_injection(FaultInjection(FaultType(FaultKind.NETWORK_PARTITION), 1.0, at_tick, duration, 1))
        return m

    @staticmethod
    def cascading_failure(world_size: int, seed: int = 0) -> ChaosMonkey:
        m = ChaosMonkey(seed, world_size)
        for i in range(min(3, world_size)):
            m.add_injection(FaultInjection(FaultType(FaultKind.PROCESS_CRASH, ranks=(i,)), 1.0, 2 + 2 * i, 3, 1))
        return m

    @staticmethod
    def random_stress(world_size: int, seed: int = 0) -> ChaosMonkey:
        m = ChaosMonkey(seed, world_size)
        m.add_common_faults(world_size)
        for inj in m.injections:
            inj.trigger_probability = min(1.0, inj.trigger_probability * 10)
        return m
