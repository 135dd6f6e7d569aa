"""Iteration-level (continuous-batching) scheduler (crates/nn/src/continuous_batching.rs:41-452).

Each call to `schedule()` retires finished requests, resumes paused ones, admits waiting requests while KV blocks
last, preempts low-priority work under memory pressure and returns the batch for the next model step: full
prompts for requests in prefill, the last token for requests in decode.  The scheduling policy is honoured
(the reference stores it and never reads it), and the end-of-sequence id is configurable (the reference hard-codes 2).

`Scheduler` keeps the decisions (queues, ordering, admission against the block allocator, preemption, retirement) in
the C++ core of the runtime library (csrc/runtime/scheduler.cpp); this module keeps the tokens and the timing of each
request.  `PyScheduler` is the same logic in Python, kept as the specification the core is tested against.
"""
from __future__ import annotations

import ctypes as C
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


class PyScheduler:
    """The scheduler in plain Python: the executable specification the native core (`Scheduler`) is tested against."""

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

    def abort(self, rid: int) -> bool:
        """Removes an unfinished request from whichever queue holds it and frees its blocks."""
        r = self.get(rid)
        if r is None or r.state is RequestState.COMPLETED:
            return False
        self.running.pop(rid, None)
        for q in (self.pending, self.paused):
            for x in list(q):
                if x.id == rid:
                    q.remove(x)
        self.cache.free(rid)
        return True

    def get(self, rid: int):
        if rid in self.running:
            return self.running[rid]
        for coll in (self.pending, self.paused, self.completed):
            for r in coll:
                if r.id == rid:
                    return r
        return None


_STATE_OF = {0: RequestState.WAITING, 1: RequestState.PREFILL, 2: RequestState.GENERATING, 3: RequestState.PAUSED,
             4: RequestState.COMPLETED}
_POLICY_CODE = {SchedulingPolicy.FCFS: 0, SchedulingPolicy.SRTF: 1, SchedulingPolicy.PRIORITY: 2}


class Scheduler:
    """Continuous-batching scheduler on the native core.  Same interface and decisions as `PyScheduler`."""

    def __init__(self, cache: PagedCache, max_batch_size: int = 64, policy: SchedulingPolicy = SchedulingPolicy.FCFS,
                 preemption_threshold: float = 0.5, max_prefill_tokens: int = 8192):
        from .. import _native as N
        self.cache = cache
        self.max_batch_size, self.policy = max_batch_size, policy
        self.preemption_threshold, self.max_prefill_tokens = preemption_threshold, max_prefill_tokens
        self._lib = N.runtime()
        self._h = self._lib.rb_sched_create(cache._h, max_batch_size, _POLICY_CODE[policy], float(preemption_threshold),
                                            max_prefill_tokens)
        if not self._h:
            raise ValueError("Scheduler: max_batch_size and max_prefill_tokens must be positive")
        self.requests: dict = {}
        self.completed: list = []
        self._latency = 0.0
        cap = max_batch_size
        self._ids, self._pre, self._lens = (C.c_int64 * cap)(), (C.c_int32 * cap)(), (C.c_int32 * cap)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rb_sched_destroy(h)

    # ---- submission -----------------------------------------------------------------------------------------
    def add_request(self, prompt, max_tokens: int, priority: RequestPriority = RequestPriority.NORMAL, eos_id=None,
                    arrival_time: float | None = None) -> int:
        prompt = list(prompt)
        rid = int(self._lib.rb_sched_add(self._h, len(prompt), int(max_tokens), int(priority), 0 if eos_id is None else 1,
                                         0 if eos_id is None else int(eos_id)))
        if rid < 0:
            raise ValueError("Scheduler.add_request: invalid request")
        req = Request(rid, prompt, max_tokens, priority, eos_id)
        if arrival_time is not None:
            req.arrival_time = arrival_time
        self.requests[rid] = req
        return rid

    def has_work(self) -> bool:
        return bool(self._lib.rb_sched_has_work(self._h))

    # ---- one iteration ------------------------------------------------------------------------------------------
    def _collect_retired(self) -> None:
        buf = (C.c_int64 * 64)()
        while True:
            n = self._lib.rb_sched_take_retired(self._h, buf, 64)
            for i in range(n):
                r = self.requests[int(buf[i])]
                r.state = RequestState.COMPLETED
                r.finish_time = time.perf_counter()
                self._latency += r.finish_time - r.arrival_time
                self.completed.append(r)
            if n < 64:
                return

    def _retire(self) -> None:
        self._lib.rb_sched_retire(self._h)
        self._collect_retired()

    def schedule(self) -> Batch:
        n = self._lib.rb_sched_schedule(self._h, self._ids, self._pre, self._lens, len(self._ids))
        if n < 0:
            raise RuntimeError(f"scheduler core failed ({n})")
        self._collect_retired()
        ids, inputs, lens, tables, pre = [], [], [], [], []
        for i in range(n):
            r = self.requests[int(self._ids[i])]
            if self._pre[i]:
                r.state = RequestState.PREFILL
                inputs.append(r.prompt + r.generated)          # a resumed request re-runs its whole prefix
            else:
                inputs.append([r.last_token()])
            pre.append(bool(self._pre[i]))
            ids.append(r.id)
            lens.append(int(self._lens[i]))
            tables.append(self.cache.block_table(r.id))
        return Batch(ids, inputs, lens, tables, pre)

    def update(self, outputs: dict, now: float | None = None) -> None:
        """outputs: request id -> sampled token.  Grows block tables; a request that finds no free block is paused."""
        n = len(outputs)
        if not n:
            return
        ids = (C.c_int64 * n)(*[int(k) for k in outputs])
        toks = (C.c_int64 * n)(*[int(v) for v in outputs.values()])
        res = (C.c_int32 * n)()
        self._lib.rb_sched_update(self._h, ids, toks, n, res)
        for i, (rid, tok) in enumerate(outputs.items()):
            if res[i] == 0:
                continue
            r = self.requests[rid]
            r.add_token(tok, now)
            r.state = RequestState.PAUSED if res[i] == 2 else RequestState.GENERATING

    # ---- inspection ---------------------------------------------------------------------------------------------
    def get(self, rid: int):
        return self.requests.get(rid)

    def abort(self, rid: int) -> bool:
        """Removes an unfinished request from whichever queue holds it, frees its blocks and drops its record."""
        if self._lib.rb_sched_abort(self._h, int(rid)) == 1:
            self.requests.pop(rid, None)
            return True
        return False

    def forget(self, rid: int) -> None:
        """Drops a completed request's record (long-running servers call this after delivering the result)."""
        r = self.requests.get(rid)
        if r is not None and r.state is RequestState.COMPLETED:
            self._lib.rb_sched_forget(self._h, rid)
            del self.requests[rid]

    def _listed(self, which: int) -> list:
        n = self._lib.rb_sched_list(self._h, which, None, 0)
        buf = (C.c_int64 * max(n, 1))()
        self._lib.rb_sched_list(self._h, which, buf, n)
        return [self.requests[int(buf[i])] for i in range(n)]

    @property
    def pending(self) -> list:
        return self._listed(0)

    @property
    def running(self) -> dict:
        return {r.id: r for r in self._listed(1)}

    @property
    def paused(self) -> list:
        return self._listed(2)

    @property
    def stats(self) -> SchedulerStats:
        out = (C.c_int64 * 4)()
        self._lib.rb_sched_stats(self._h, out)
        return SchedulerStats(int(out[0]), int(out[1]), int(out[2]), int(out[3]), self._latency)
