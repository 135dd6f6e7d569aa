"""Failure detection and elastic recovery (crates/distributed/src/fault_tolerance.rs:30-456).

All of it runs on the host: heartbeats travel through a key-value store (torch's TCPStore between processes, a
dict inside one process), device-side waits are bounded and surface as CommunicationError, and a failed step is
retried from the last checkpoint.  Nothing here faults or hangs a GPU.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

from .process_group import CommunicationError, DistributedError, ProcessGroup, RankMismatch


class NodeState(enum.Enum):
    HEALTHY = "healthy"
    SUSPECTED = "suspected"
    FAILED = "failed"
    JOINING = "joining"
    LEAVING = "leaving"


@dataclass
class NodeInfo:
    rank: int
    state: NodeState = NodeState.HEALTHY
    last_heartbeat: float = 0.0
    last_checkpoint: int = -1


class DictStore:
    """In-process stand-in for a TCPStore (set / get of small byte strings)."""

    def __init__(self):
        self._d: dict = {}

    def set(self, k: str, v) -> None:
        self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        return self._d[k]

    def check(self, keys) -> bool:
        return all(k in self._d for k in keys)


class HealthMonitor:
    """HEALTHY -> SUSPECTED after `timeout_ms` without a heartbeat, SUSPECTED -> FAILED after twice that."""

    def __init__(self, my_rank: int, timeout_ms: float = 5000.0, store=None, clock=time.monotonic):
        self.my_rank, self.timeout_ms = my_rank, timeout_ms
        self.store = store
        self.clock = clock
        self.nodes: dict = {}

    def register_node(self, rank: int) -> None:
        self.nodes[rank] = NodeInfo(rank, NodeState.HEALTHY, self.clock())

    def heartbeat(self, rank: int | None = None) -> None:
        """Records a heartbeat; with a store, publishes this rank's beat for the others to read."""
        rank = self.my_rank if rank is None else rank
        now = self.clock()
        if rank in self.nodes:
            n = self.nodes[rank]
            n.last_heartbeat = now
            if n.state in (NodeState.SUSPECTED, NodeState.JOINING):
                n.state = NodeState.HEALTHY
        if self.store is not None and rank == self.my_rank:
            self.store.set(f"hb/{rank}", repr(now))

    def poll_store(self) -> None:
        """Pulls the other ranks' published heartbeats."""
        if self.store is None:
            return
        for r, n in self.nodes.items():
            if r == self.my_rank:
                continue
            try:
                if self.store.check([f"hb/{r}"]):
                    t = float(self.store.get(f"hb/{r}").decode())
                    if t > n.last_heartbeat:
                        n.last_heartbeat = t
                        if n.state is NodeState.SUSPECTED:
                            n.state = NodeState.HEALTHY
            except (KeyError, ValueError):
                pass

    def check_health(self) -> list:
        """Advances the state machines; returns the ranks that became FAILED in this call."""
        self.poll_store()
        now = self.clock()
        newly = []
        for n in self.nodes.values():
            if n.state in (NodeState.FAILED, NodeState.LEAVING):
                continue
            age_ms = (now - n.last_heartbeat) * 1e3
            if age_ms > 2 * self.timeout_ms:
                n.state = NodeState.FAILED
                newly.append(n.rank)
            elif age_ms > self.timeout_ms:
                n.state = NodeState.SUSPECTED
        return newly

    def healthy_nodes(self) -> list:
        return sorted(r for r, n in self.nodes.items() if n.state is NodeState.HEALTHY)

    def checkpoint_completed(self, rank: int, epoch: int) -> None:
        if rank in self.nodes:
            self.nodes[rank].last_checkpoint = epoch


@dataclass
class MembershipChange:
    kind: str                     # "nodes_failed" | "nodes_joining" | "reconfiguration_complete"
    ranks: list = field(default_factory=list)
    new_world_size: int = 0
    new_rank: int = 0


class ElasticProcessGroup:
    def __init__(self, base: ProcessGroup, health: HealthMonitor):
        self.base, self.health = base, health
        self.failed: set = set()
        for r in range(base.world_size):
            if r not in health.nodes:
                health.register_node(r)

    def check_membership(self):
        newly = self.health.check_health()
        if newly:
            self.failed.update(newly)
            return MembershipChange("nodes_failed", sorted(newly))
        return None

    def effective_world_size(self) -> int:
        return self.base.world_size - len(self.failed)

    def is_active(self, rank: int) -> bool:
        return rank not in self.failed

    def reconfigure(self) -> MembershipChange:
        """New dense ranks for the survivors (the caller rebuilds communicators with them)."""
        alive = [r for r in range(self.base.world_size) if r not in self.failed]
        return MembershipChange("reconfiguration_complete", alive, len(alive),
                                alive.index(self.base.rank) if self.base.rank in alive else -1)


class CheckpointStore:
    """What ElasticTrainer needs from a checkpoint backend."""

    def save(self, step: int, state) -> None:
        raise NotImplementedError

    def load(self, step: int):
        raise NotImplementedError

    def latest(self):
        raise NotImplementedError


class MemoryCheckpointStore(CheckpointStore):
    def __init__(self):
        self._d: dict = {}

    def save(self, step, state):
        import copy
        self._d[step] = copy.deepcopy(state)

    def load(self, step):
        return self._d[step]

    def latest(self):
        return max(self._d) if self._d else None


@dataclass
class RestartConfig:
    max_restarts: int = 3
    restart_delay_s: float = 10.0
    checkpoint_on_failure: bool = True


@dataclass
class FaultStats:
    failures: int = 0
    recoveries: int = 0
    retries: int = 0
    lost_steps: int = 0


class ElasticTrainer:
    """Runs `train_fn(step, state) -> state`, checkpointing every `checkpoint_every` steps; a CommunicationError or
    RankMismatch rolls back to the latest checkpoint and retries, up to `max_retries` times in a row."""

    def __init__(self, store: CheckpointStore, health_check_interval_s: float = 30.0, max_retries: int = 3,
                 checkpoint_every: int = 1, elastic_group: ElasticProcessGroup | None = None, sleep=time.sleep,
                 restart: RestartConfig | None = None):
        self.store, self.max_retries, self.checkpoint_every = store, max_retries, checkpoint_every
        self.health_check_interval_s = health_check_interval_s
        self.group = elastic_group
        self.stats = FaultStats()
        self.sleep = sleep
        self.restart = restart or RestartConfig(restart_delay_s=0.0)

    def recover_from_checkpoint(self):
        step = self.store.latest()
        if step is None:
            return 0, None
        self.stats.recoveries += 1
        return step, self.store.load(step)

    def train_loop(self, train_fn, num_steps: int, initial_state=None):
        state, step, retries = initial_state, 0, 0
        if self.store.latest() is None:
            self.store.save(0, state)
        while step < num_steps:
            try:
                if self.group is not None:
                    change = self.group.check_membership()
                    if change is not None:
                        raise CommunicationError(f"ranks failed: {change.ranks}")
                state = train_fn(step, state)
                step += 1
                retries = 0
                if step % self.checkpoint_every == 0:
                    self.store.save(step, state)
            except (CommunicationError, RankMismatch) as e:
                self.stats.failures += 1
                retries += 1
                self.stats.retries += 1
                if retries > self.max_retries:
                    raise DistributedError(f"giving up after {self.max_retries} retries: {e}") from e
                if self.restart.restart_delay_s > 0:
                    self.sleep(self.restart.restart_delay_s)
                ck_step, ck_state = self.recover_from_checkpoint()
                self.stats.lost_steps += step - ck_step
                step, state = ck_step, ck_state
                if self.group is not None:
                    self.group.failed.clear()
                    for n in self.group.health.nodes.values():     # the job was restarted: everyone reports in again
                        n.state = NodeState.HEALTHY
                        n.last_heartbeat = self.group.health.clock()
        return state


class TimedBarrier:
    """Host-side barrier bookkeeping with a deadline: arrive(rank); is_complete(); timed_out()."""

    def __init__(self, world_size: int, timeout_s: float, clock=time.monotonic):
        self.world_size, self.timeout_s, self.clock = world_size, timeout_s, clock
        self.reset()

    def reset(self):
        self.arrived: set = set()
        self.t0 = self.clock()

    def arrive(self, rank: int):
        self.arrived.add(rank)

    def is_complete(self) -> bool:
        return len(self.arrived) >= self.world_size

    def timed_out(self) -> bool:
        return not self.is_complete() and (self.clock() - self.t0) > self.timeout_s

    def missing(self) -> list:
        return sorted(set(range(self.world_size)) - self.arrived)


@dataclass
class CheckpointVersion:
    epoch: int
    step: int


class StateSync:
    """Tracks which nodes have loaded the agreed checkpoint version after a reconfiguration."""

    def __init__(self, target_world_size: int, min_nodes: int = 1):
        self.target_world_size, self.min_nodes = target_world_size, min_nodes
        self.synced: dict = {}

    def report(self, rank: int, version: CheckpointVersion):
        self.synced[rank] = version

    def can_proceed(self) -> bool:
        if len(self.synced) < self.min_nodes:
            return False
        vs = {(v.epoch, v.step) for v in self.synced.values()}
        return len(vs) == 1

    def is_complete(self) -> bool:
        return len(self.synced) >= self.target_world_size and self.can_proceed()


class StepWatchdog:
    """Host-side wall-clock limit per training step.

    `with watchdog.step():` arms a timer; if the block has not finished after `limit_s` the watchdog records the
    overrun and calls `on_timeout` from its own thread (e.g. to mark the rank as suspected in the health monitor or to
    abort the process group).  Leaving the block after an overrun raises `CommunicationError`, which is what
    `ElasticTrainer` treats as recoverable.  Device-side waits are bounded on their own and report through the
    status word; this is the host's counterpart for a step that stalls anywhere else (a collective, a data loader)."""

    def __init__(self, limit_s: float, on_timeout=None):
        self.limit_s, self.on_timeout = limit_s, on_timeout
        self.overruns = 0
        self._timer = None
        self._fired = False

    def _fire(self):
        self._fired = True
        self.overruns += 1
        if self.on_timeout is not None:
            self.on_timeout()

    def step(self):
        return self

    def __enter__(self):
        import threading
        self._fired = False
        self._timer = threading.Timer(self.limit_s, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def __exit__(self, exc_type, exc, tb):
        self._timer.cancel()
        if self._fired and exc_type is None:
            raise CommunicationError(f"step exceeded its wall-clock limit of {self.limit_s} s")
        return False
