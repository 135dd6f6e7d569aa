"""ServingEngine: continuous batching around a real model step, with latency accounting
(crates/nn/src/continuous_batching.rs:496-546)."""
from __future__ import annotations

import statistics
import time
from dataclasses import dataclass

import torch

from .model_runner import ModelRunner
from .sampler import Sampler
from .scheduler import RequestPriority, RequestState, Scheduler, SchedulingPolicy


@dataclass
class ServingMetrics:
    completed: int
    output_tokens: int
    wall_s: float
    ttft_p50_ms: float
    ttft_p99_ms: float
    itl_p50_ms: float
    itl_p99_ms: float
    output_tokens_per_s: float

    def to_dict(self) -> dict:
        return dict(self.__dict__)


def _pct(xs, q):
    if not xs:
        return 0.0
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


class ServingEngine:
    def __init__(self, runner: ModelRunner, max_batch_size: int = 64, policy: SchedulingPolicy = SchedulingPolicy.FCFS,
                 sampler: Sampler | None = None, eos_id: int | None = None, prefill_chunk: int = 2048,
                 max_prefill_tokens: int = 8192):
        """`prefill_chunk`: prompt tokens processed per step, summed over all requests in prefill (0: whole prompts, one
        model pass per prompt).  A longer prompt is spread over several steps, each of which also serves the decode
        batch, so that a long prompt delays the running requests by one chunk's time, not by the whole prompt's."""
        self.runner = runner
        self.prefill_chunk = int(prefill_chunk)
        self._prefill_pos: dict = {}          # request id -> prompt tokens already in the cache
        self.scheduler = Scheduler(runner.cache, max_batch_size, policy, max_prefill_tokens=max_prefill_tokens)
        self.sampler = sampler or Sampler.greedy()
        self.eos_id = eos_id
        self.callbacks: dict = {}
        self.steps = 0

    def submit(self, prompt, max_tokens: int, priority: RequestPriority = RequestPriority.NORMAL, callback=None,
               arrival_time: float | None = None) -> int:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if len(prompt) + max_tokens > self.runner.cfg.seq_len:
            raise ValueError(f"prompt + max_tokens exceeds the model's context of {self.runner.cfg.seq_len}")
        # A request that could never hold its whole sequence in the KV cache would sit at the head of the queue for
        # ever (admission keeps the order when memory is short) and stall everything behind it: refuse it here.
        cache = self.runner.cache
        need = cache.blocks_needed(len(prompt) + max_tokens + 1)
        if need > cache.num_blocks:
            raise ValueError(f"request needs {need} KV blocks of {cache.block_size} tokens, the cache has {cache.num_blocks}")
        rid = self.scheduler.add_request(prompt, max_tokens, priority, self.eos_id, arrival_time)
        if callback is not None:
            self.callbacks[rid] = callback
        return rid

    def step(self) -> dict:
        """One iteration: schedule, run the model, sample, update.  Returns request id -> new token.

        With `prefill_chunk` > 0 the step is ONE model pass over up to `prefill_chunk` prompt tokens (several short
        prompts, or the next piece of a long one) plus the decode batch; a request whose prompt is not finished yet
        yields no token in this step.  A step without prompt work replays the decode graph."""
        sch = self.scheduler
        done_before = len(sch.completed)
        batch = sch.schedule()
        for r in sch.completed[done_before:]:
            cb = self.callbacks.pop(r.id, None)
            if cb is not None:
                cb(r)
        scheduled = set(batch.request_ids)
        for rid in [rid for rid in self._prefill_pos if rid not in scheduled]:
            del self._prefill_pos[rid]             # paused, aborted or finished: a resumed request starts over
        if len(batch) == 0:
            return {}
        outputs = {}
        vocab = self.runner.cfg.vocab_size
        dec_ids, dec_tok, dec_len, chunks = [], [], [], []
        budget = self.prefill_chunk
        for rid, inp, n, pre in zip(batch.request_ids, batch.input_ids, batch.seq_lens, batch.is_prefill):
            if not pre:
                dec_ids.append(rid)
                dec_tok.append(inp[0])
                dec_len.append(n)
            elif self.prefill_chunk <= 0:
                logits = self.runner.prefill(rid, inp)
                outputs[rid] = int(self.sampler.sample(logits[:vocab].unsqueeze(0))[0])
            elif budget > 0:
                pos = self._prefill_pos.get(rid, 0)
                take = min(len(inp) - pos, budget)
                budget -= take
                chunks.append((rid, inp[pos:pos + take], pos, pos + take == len(inp)))
        if chunks:
            chunk_logits, dec_logits = self.runner.step_mixed(chunks, dec_ids, dec_tok, dec_len)
            for (rid, toks, pos, last), lg in zip(chunks, chunk_logits):
                if last:
                    self._prefill_pos.pop(rid, None)
                    outputs[rid] = int(self.sampler.sample(lg[:vocab].unsqueeze(0))[0])
                else:
                    self._prefill_pos[rid] = pos + len(toks)
            if dec_ids:
                outputs.update(dict(zip(dec_ids, self.sampler.sample(dec_logits[:, :vocab]).tolist())))
        elif dec_ids:
            logits = self.runner.decode(dec_ids, dec_tok, dec_len)
            toks = self.sampler.sample(logits[:, :vocab]).tolist()
            outputs.update(dict(zip(dec_ids, toks)))
        if self.runner.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        sch.update(outputs, time.perf_counter())
        self.steps += 1
        return outputs

    def run_to_completion(self, max_steps: int = 1 << 30) -> list:
        n = 0
        while self.scheduler.has_work() and n < max_steps:
            self.step()
            n += 1
        self.scheduler._retire()
        return self.scheduler.completed

    def generate(self, prompt, max_tokens: int, keep_record: bool = False) -> list:
        """Runs one request to completion and returns its tokens.  The request's record is dropped afterwards (a
        long-running server would otherwise accumulate every request it ever served) unless `keep_record`."""
        rid = self.submit(prompt, max_tokens)
        self.run_to_completion()
        tokens = list(self.scheduler.get(rid).generated)
        if not keep_record:
            self.release(rid)
        return tokens

    def abort(self, rid: int) -> bool:
        """Cancels one unfinished request: its KV blocks are freed and its prefill progress and callback are dropped.
        False when the request is unknown or already finished."""
        ok = self.scheduler.abort(rid)
        if ok:
            self.callbacks.pop(rid, None)
            self._prefill_pos.pop(rid, None)
        return ok

    def abort_all(self) -> list:
        """Removes every unfinished request (after a failed model step: retrying it would fail the same way), frees
        their KV blocks and returns their ids."""
        sch = self.scheduler
        ids = [r.id for r in list(sch.pending)] + list(sch.running.keys()) + [r.id for r in list(sch.paused)]
        for rid in ids:
            sch.abort(rid)
            self.callbacks.pop(rid, None)
            self._prefill_pos.pop(rid, None)
        return ids

    def release(self, rid: int) -> None:
        """Forgets a COMPLETED request: its entry in the scheduler (and the native core) and in `scheduler.completed`."""
        sch = self.scheduler
        r = sch.get(rid)
        if r is None or r.state is not RequestState.COMPLETED:
            return
        sch.completed[:] = [c for c in sch.completed if c.id != rid]
        if hasattr(sch, "forget"):
            sch.forget(rid)

    def metrics(self, wall_s: float) -> ServingMetrics:
        done = self.scheduler.completed
        ttft = [(r.first_token_time - r.arrival_time) * 1e3 for r in done if r.first_token_time is not None]
        itl = []
        for r in done:
            itl += [(b - a) * 1e3 for a, b in zip(r.token_times, r.token_times[1:])]
        out_tokens = sum(len(r.generated) for r in done)
        return ServingMetrics(len(done), out_tokens, wall_s, _pct(ttft, 0.5), _pct(ttft, 0.99), _pct(itl, 0.5), _pct(itl, 0.99),
                              out_tokens / wall_s if wall_s > 0 else 0.0)


def run_poisson_workload(engine: ServingEngine, num_requests: int, rate_per_s: float, prompt_range=(128, 2048),
                         output_range=(128, 512), seed: int = 0, time_limit_s: float = 3600.0, clock=None) -> ServingMetrics:
    """Open-loop load test: requests arrive by a Poisson process at `rate_per_s`, prompt and output lengths uniform in
    the given ranges, prompt tokens uniform random; the engine steps in real time and a request is submitted once
    its arrival time has passed (its latency clock starts at the ARRIVAL time, so queueing counts).  `clock(now)`
    may replace each loop iteration's time by an agreed one (tensor-parallel ranks: rank 0's), so that all ranks
    admit the same requests in the same iteration."""
    g = torch.Generator().manual_seed(seed)
    vocab = engine.runner.cfg.vocab_size
    gaps = torch.empty(num_requests).exponential_(rate_per_s, generator=g)
    arrivals = torch.cumsum(gaps, 0).tolist()
    plen = torch.randint(prompt_range[0], prompt_range[1] + 1, (num_requests,), generator=g).tolist()
    olen = torch.randint(output_range[0], output_range[1] + 1, (num_requests,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in plen]
    t0 = time.perf_counter()
    nxt = 0
    while nxt < num_requests or engine.scheduler.has_work():
        now = time.perf_counter() - t0
        if clock is not None:
            now = clock(now)
        if now >= time_limit_s:
            break
        while nxt < num_requests and arrivals[nxt] <= now:
            engine.submit(prompts[nxt], olen[nxt], arrival_time=t0 + arrivals[nxt])
            nxt += 1
        if engine.scheduler.has_work():
            engine.step()
        elif nxt < num_requests:
            time.sleep(min(0.001, max(0.0, arrivals[nxt] - now)))
    engine.scheduler._retire()
    return engine.metrics(time.perf_counter() - t0)
