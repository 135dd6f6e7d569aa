"""Serving: KV caches, continuous-batching scheduler, sampler, model runner, engine, HTTP front end."""
from .kv_cache import CacheQuantization, CacheConfig, CacheMemoryStats, KVCache, SlidingWindowCache, PagedCache, BatchedCache
from .scheduler import RequestPriority, RequestState, Request, SchedulingPolicy, Batch, Scheduler, PyScheduler, SchedulerStats
from .sampler import Sampler
from .model_runner import ModelRunner
from .engine import ServingEngine, ServingMetrics, run_poisson_workload

__all__ = [n for n in dir() if not n.startswith("_")]
