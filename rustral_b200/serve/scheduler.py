"""Iteration-level (continuous-batching) scheduler (crates/nn/src/continuous_batching.rs:41-452).

Each call to `schedule()` retires finished requests, resumes paused ones, admits waiting requests while KV blocks
last, preempts low-priority work under memory pressure and returns the batch for the next model step: full
prompts for requests in prefill, the last token for requests in decode.  The scheduling policy is honoured
(the reference stores it and never reads it), and the end-of-sequence id is configurable (the reference hard-codes 2).
"""
from __future__ import annotations

import enum
import time
from collections import deque
from dataclasses import dataclass, field

from .kv_cache import PagedCache


class RequestPriority(enum.IntEnum):
    LOW = 0
    NORMAL = 1
    HIGH = 2
    CRITICAL = 3


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    GENERATING = "generating"
    PAUSED = "paused"
    COMPLETED = "completed"


class SchedulingPolicy(enum.Enum):
    FCFS = "fcfs"
    SRTF = "srtf"            # shortest remaining tokens first
    PRIORITY = "priority"


@dataclass
class Request:
    id: int
    prompt: list
    max_tokens: int
    priority: RequestPriority = RequestPriority.NORMAL
    eos_id: int | None = None
    state: RequestState = RequestState.WAITING
    generated: list = field(default_factory=list)
    arrival_time: float = field(default_factory=time.perf_counter)
    first_token_time: float | None = None
    finish_time: float | None = None
    token_times: list = field(default_factory=list)

    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    def remaining(self) -> int:
        return self.max_tokens - len(self.generated)

    def add_token(self, tok: int, now: float | None = None) -> None:
        now = time.perf_counter() if now is None else now
        if self.first_token_time is None:
            self.first_token_time = now
        self.token_times.append(now)
        self.generated.append(int(tok))

    def should_complete(self) -> bool:
        if len(self.generated) >= self.max_tokens:
            return True
        return self.eos_id is not None and len(self.generated) > 0 and self.generated[-1] == self.eos_id

    def last_token(self) -> int:
        return self.generated[-1] if self.generated else self.prompt[-1]


@dataclass
class Batch:
    request_ids: list
    input_ids: list          # per request: full prompt (prefill) or [last token] (decode)
    seq_lens: list           # tokens in the cache after this step
    block_tables: list
    is_prefill: list

    def __len__(self):
        return len(self.request_ids)


@dataclass
class SchedulerStats:
    completed: int = 0
    preempted: int = 0
    admitted: int = 0
    total_generated: int = 0
    total_latency: float = 0.0

    @property
    def avg_latency(self) -> float:
        return self.total_latency / self.completed if self.completed else 0.0


class Scheduler:
    def __init__(self, cache: PagedCache, max_batch_size: int = 64, policy: SchedulingPolicy = SchedulingPolicy.FCFS,
                 preemption_threshold: float = 0.5, max_prefill_tokens: int = 8192):
        self.cache = cache
        self.max_batch_size = max_batch_size
        self.policy = policy
        self.preemption_threshold = preemption_threshold
        self.max_prefill_tokens = max_prefill_tokens
        self.pending: deque = deque()
        self.running: dict = {}
        self.paused: deque = deque()
        self.completed: list = []
        self.stats = SchedulerStats()
        self._next_id = 0

    # ---- submission -----------------------------------------------------------------------------------------
    def add_request(self, prompt, max_tokens: int, priority: RequestPriority = RequestPriority.NORMAL, eos_id=None,
                    arrival_time: float | None = None) -> int:
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, list(prompt), max_tokens, priority, eos_id)
        if arrival_time is not None:
            req.arrival_time = arrival_time
        self.pending.append(req)
        return rid

    def has_work(self) -> bool:
        return bool(self.pending or self.running or self.paused)

    # ---- one iteration ------------------------------------------------------------------------------------------
    def _order(self, reqs):
        if self.policy is SchedulingPolicy.SRTF:
            return sorted(reqs, key=lambda r: (r.remaining() + (0 if r.generated else len(r.prompt)), r.id))
        if self.policy is SchedulingPolicy.PRIORITY:
            return sorted(reqs, key=lambda r: (-int(r.priority), r.id))
        return list(reqs)

    def _retire(self) -> None:
        for rid in [rid for rid, r in self.running.items() if r.should_complete()]:
            r = self.running.pop(rid)
            r.state = RequestState.COMPLETED
            r.finish_time = time.perf_counter()
            self.cache.free(rid)
            self.completed.append(r)
            self.stats.completed += 1
            self.stats.total_generated += len(r.generated)
            self.stats.total_latency += r.finish_time - r.arrival_time

    def _try_resume(self) -> None:
        for _ in range(len(self.paused)):
            if len(self.running) >= self.max_batch_size:
                break
            r = self.paused[0]
            if not self.cache.allocate(r.id, r.total_len() + 1):
                break
            self.paused.popleft()
            r.state = RequestState.PREFILL          # its cache was released: the whole prefix is recomputed
            self.running[r.id] = r

    def _admit(self) -> None:
        budget = self.max_prefill_tokens
        for r in self._order(self.pending):
            if len(self.running) >= self.max_batch_size:
                break
            if len(r.prompt) > budget and budget < self.max_prefill_tokens:
                break
            if not self.cache.allocate(r.id, len(r.prompt) + 1):
                break                                   # head-of-line: keep arrival order when memory is short
            self.pending.remove(r)
            r.state = RequestState.PREFILL
            self.running[r.id] = r
            self.stats.admitted += 1
            budget -= len(r.prompt)

    def _maybe_preempt(self) -> None:
        """Under memory pressure (few free blocks and a non-empty queue) pause the lowest-priority running
        request; its blocks are released and it is recomputed from its tokens when resumed."""
        if not self.pending or len(self.running) <= 1:
            return
        if self.cache.free_blocks > 0 and len(self.running) / self.max_batch_size <= self.preemption_threshold:
            return
        waiting_best = max(int(r.priority) for r in self.pending)
        victims = [r for r in self.running.values() if int(r.priority) < waiting_best and r.priority == RequestPriority.LOW]
        if not victims or self.cache.free_blocks > 0:
            return
        v = max(victims, key=lambda r: r.id)
        self.running.pop(v.id)
        self.cache.free(v.id)
        v.state = RequestState.PAUSED
        self.paused.append(v)
        self.stats.preempted += 1

    def schedule(self) -> Batch:
        self._retire()
        self._try_resume()
        self._admit()
        self._maybe_preempt()
        ids, inputs, lens, tables, pre = [], [], [], [], []
        for r in self._order(self.running.values()):
            if r.state is RequestState.PREFILL:
                toks = r.prompt + r.generated          # a resumed request re-runs its whole prefix
                inputs.append(list(toks))
                pre.append(True)
            else:
                inputs.append([r.last_token()])
                pre.append(False)
            ids.append(r.id)
            lens.append(r.total_len())
            tables.append(self.cache.block_table(r.id))
        return Batch(ids, inputs, lens, tables, pre)

    def update(self, outputs: dict, now: float | None = None) -> None:
        """outputs: request id -> sampled token.  Grows block tables; raises when the cache is exhausted."""
        for rid, tok in outputs.items():
            r = self.running.get(rid)
            if r is None:
                continue
            r.add_token(tok, now)
            r.state = RequestState.GENERATING
            if not r.should_complete() and not self.cache.allocate(rid, r.total_len() + 1):
                # out of blocks: pause this request instead of failing the whole batch
                self.running.pop(rid)
                self.cache.free(rid)
                r.state = RequestState.PAUSED
                self.paused.append(r)
                self.stats.preempted += 1

    def get(self, rid: int):
        if rid in self.running:
            return self.running[rid]
        for coll in (self.pending, self.paused, self.completed):
            for r in coll:
                if r.id == rid:
                    return r
        return None
