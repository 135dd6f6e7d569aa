"""Autotuner: search over kernel tile configurations with CUDA-event timing and a persistent cache
(crates/autotuner/src/{lib,kernel_config,search,tuner,cache}.rs).

The search strategies (grid, random, evolutionary, explore/exploit) live in C++ (csrc/runtime/search.cpp); this
package defines the tunable kernels, times candidates on the device and stores winners in a JSON cache keyed by
(kernel id, device, dtype, shape bucket).  Unlike the reference's tuner, it is wired to real kernels: `tune_gemm`
picks tile width, split-K factor and rasterisation group for the tcgen05 GEMM, and `GemmTuningTable.apply` feeds
the cached choice back into `ops.gemm`.
"""
from __future__ import annotations

import ctypes as C
import enum
import json
import os
import sys
import time
from dataclasses import dataclass, field

import torch

from .. import _native as N


class Strategy(enum.IntEnum):
    GRID = 0
    RANDOM = 1
    EVOLUTIONARY = 2
    BAYESIAN = 3


def dim_bucket(n: int) -> str:
    """Tiny < 256, Small <= 512, Medium < 2048, Large < 8192, XLarge (crates/autotuner/src/kernel_config.rs)."""
    return "tiny" if n < 256 else "small" if n <= 512 else "medium" if n < 2048 else "large" if n < 8192 else "xlarge"


@dataclass(frozen=True)
class MatmulShapeBucket:
    m: str
    n: str
    k: str

    @classmethod
    def of(cls, M: int, N_: int, K: int):
        return cls(dim_bucket(M), dim_bucket(N_), dim_bucket(K))

    def cache_key(self) -> str:
        return f"matmul_{self.m}_{self.n}_{self.k}"


@dataclass
class ConfigSpace:
    dims: dict          # name -> list of int choices

    def size(self) -> int:
        n = 1
        for v in self.dims.values():
            n *= len(v)
        return n

    @classmethod
    def matmul_full(cls):
        return cls({"block_n": [64, 128, 192, 256], "splits": [1, 2, 3, 4, 6, 8], "group_m": [4, 8, 16]})

    @classmethod
    def matmul_reduced(cls):
        return cls({"block_n": [128, 192, 256], "splits": [1, 2, 4], "group_m": [8]})


@dataclass
class PerfMetrics:
    time_us: float
    tflops: float = 0.0
    gbytes_per_s: float = 0.0

    @classmethod
    def from_duration(cls, time_us: float, flops: float = 0.0, bytes_: float = 0.0):
        s = time_us * 1e-6
        return cls(time_us, flops / s / 1e12 if s > 0 else 0.0, bytes_ / s / 1e9 if s > 0 else 0.0)


class SearchHandle:
    """Thin wrapper over the C++ searcher."""

    def __init__(self, space: ConfigSpace, strategy: Strategy, seed: int = 0, max_evals: int = 0):
        self.names = list(space.dims)
        sizes = [len(space.dims[n]) for n in self.names]
        flat = [c for n in self.names for c in space.dims[n]]
        self._lib = N.runtime()
        self._sizes = (C.c_int * len(sizes))(*sizes)
        self._flat = (C.c_int * len(flat))(*flat)
        self._h = self._lib.rb_search_create(int(strategy), len(sizes), self._sizes, self._flat, seed, max_evals)
        if not self._h:
            raise ValueError("invalid search space")
        self._buf = (C.c_int * len(sizes))()

    def next_config(self):
        if not self._lib.rb_search_next(self._h, self._buf):
            return None
        return dict(zip(self.names, list(self._buf)))

    def report(self, config: dict, time_us: float) -> None:
        arr = (C.c_int * len(self.names))(*[config[n] for n in self.names])
        self._lib.rb_search_report(self._h, arr, float(time_us))

    def best(self):
        t = C.c_double()
        if not self._lib.rb_search_best(self._h, self._buf, C.byref(t)):
            return None, float("inf")
        return dict(zip(self.names, list(self._buf))), t.value

    def num_evals(self) -> int:
        return self._lib.rb_search_num_evals(self._h)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rb_search_destroy(h)


@dataclass
class TunerConfig:
    strategy: Strategy = Strategy.BAYESIAN
    warmup: int = 3
    timing: int = 10
    max_tuning_time_s: float = 60.0
    max_evals: int = 48
    use_cache: bool = True
    cache_results: bool = True
    min_improvement_pct: float = 1.0
    verbose: bool = False
    ci_mode: bool = False
    enabled: bool = True
    device_id: str = ""
    dtype: str = "bf16"
    seed: int = 0

    @classmethod
    def fast(cls):
        return cls(Strategy.RANDOM, warmup=2, timing=5, max_tuning_time_s=10.0, max_evals=12)

    @classmethod
    def ci_safe(cls):
        return cls(Strategy.RANDOM, warmup=1, timing=2, max_tuning_time_s=5.0, max_evals=5, ci_mode=True)

    @classmethod
    def disabled(cls):
        return cls(enabled=False)


@dataclass
class CacheEntry:
    config: dict
    time_us: float
    device_id: str
    dtype: str
    shape_bucket: str
    timestamp: float
    version: str = "1"
    num_samples: int = 0


class ConfigCache:
    """JSON at <cache>/rustral/autotuner/kernel_configs.json; entries older than 30 days or from another device are
    ignored on load."""

    MAX_AGE_S = 30 * 24 * 3600

    def __init__(self, path: str | None = None, device_id: str = ""):
        base = os.environ.get("RUSTRAL_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "rustral")
        self.path = path or os.path.join(base, "autotuner", "kernel_configs.json")
        self.device_id = device_id
        self.entries: dict = {}
        self.hits = self.misses = 0
        self.load()

    @staticmethod
    def key(kernel_id: str, device_id: str, dtype: str, bucket: str) -> str:
        return f"{kernel_id}|{device_id}|{dtype}|{bucket}"

    def load(self) -> None:
        try:
            with open(self.path) as f:
                raw = json.load(f)
        except (OSError, json.JSONDecodeError):
            return
        now = time.time()
        for k, e in raw.items():
            try:
                ce = CacheEntry(**e)
            except TypeError:
                continue
            if now - ce.timestamp <= self.MAX_AGE_S and (not self.device_id or ce.device_id == self.device_id):
                self.entries[k] = ce

    def save(self) -> None:
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + ".partial"
        with open(tmp, "w") as f:
            json.dump({k: e.__dict__ for k, e in self.entries.items()}, f, indent=1)
        os.replace(tmp, self.path)

    def get_config(self, kernel_id, device_id, dtype, bucket):
        e = self.entries.get(self.key(kernel_id, device_id, dtype, bucket))
        if e is None:
            self.misses += 1
        else:
            self.hits += 1
        return e

    def store_config(self, kernel_id, device_id, dtype, bucket, config: dict, time_us: float, num_samples: int) -> None:
        self.entries[self.key(kernel_id, device_id, dtype, bucket)] = CacheEntry(dict(config), time_us, device_id, dtype, bucket,
                                                                                 time.time(), "1", num_samples)

    def hit_rate(self) -> float:
        tot = self.hits + self.misses
        return self.hits / tot if tot else 0.0

    def stats(self) -> "CacheStats":
        by_device: dict = {}
        for e in self.entries.values():
            by_device[e.device_id] = by_device.get(e.device_id, 0) + 1
        return CacheStats(len(self.entries), by_device, self.path)


@dataclass
class CacheStats:
    """What the configuration cache holds (crates/autotuner/src/cache.rs:208-272)."""
    total_entries: int
    by_device: dict
    cache_path: str

    def print(self, file=None) -> None:
        out = file or sys.stdout
        print("Config cache statistics:", file=out)
        print(f"  total entries: {self.total_entries}", file=out)
        print(f"  cache path: {self.cache_path}", file=out)
        for dev, n in sorted(self.by_device.items()):
            print(f"    {dev}: {n}", file=out)


@dataclass
class TunerStats:
    """Running totals of an `AutoTuner` (crates/autotuner/src/tuner.rs:616-650).  Also answers the dictionary keys
    `tuned` and `cache_hits`."""
    total_tunings: int = 0
    total_configs_tried: int = 0
    total_tuning_time: float = 0.0
    cache_hits: int = 0
    cache_misses: int = 0

    def hit_rate(self) -> float:
        tot = self.cache_hits + self.cache_misses
        return self.cache_hits / tot if tot else 0.0

    def __getitem__(self, key):
        return {"tuned": self.total_tunings, "cache_hits": self.cache_hits, "cache_misses": self.cache_misses,
                "configs_tried": self.total_configs_tried}[key]

    def print(self, file=None) -> None:
        out = file or sys.stdout
        print("AutoTuner statistics:", file=out)
        print(f"  tuning sessions: {self.total_tunings}", file=out)
        print(f"  configurations tried: {self.total_configs_tried}", file=out)
        print(f"  tuning time: {self.total_tuning_time:.2f} s", file=out)
        if self.total_tunings:
            print(f"  average per session: {self.total_tuning_time / self.total_tunings:.2f} s", file=out)
        if self.cache_hits + self.cache_misses:
            print(f"  cache hit rate: {100.0 * self.hit_rate():.1f} %", file=out)


TuningCache = ConfigCache
TunerStrategy = Strategy          # the reference's name of the enumeration (crates/autotuner/src/tuner.rs:175)


class TunableKernel:
    """kernel_id / config_space / with_config(config) -> callable / input_signature (shape bucket string)."""

    kernel_id = "kernel"

    def config_space(self) -> ConfigSpace:
        raise NotImplementedError

    def with_config(self, config: dict):
        raise NotImplementedError

    def default_config(self) -> dict:
        return {k: v[0] for k, v in self.config_space().dims.items()}

    def input_signature(self) -> str:
        return "-"

    def flops(self) -> float:
        return 0.0


def benchmark_kernel(fn, warmup: int, iters: int, host_timed: bool = False) -> float:
    """Median microseconds per call: CUDA events on the current stream when a GPU is present, host clock otherwise
    (or when `host_timed`: a kernel object that does its work on the CPU sets `host_timed = True`)."""
    for _ in range(warmup):
        fn()
    if torch.cuda.is_available() and not host_timed:
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
    else:
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e6)
    ts.sort()
    return ts[len(ts) // 2]


@dataclass
class TuningResult:
    config: dict
    time_us: float
    default_time_us: float
    evaluated: int
    from_cache: bool = False

    @property
    def improvement_pct(self) -> float:
        return 100.0 * (self.default_time_us - self.time_us) / self.default_time_us if self.default_time_us > 0 else 0.0


class AutoTuner:
    def __init__(self, config: TunerConfig | None = None, cache: ConfigCache | None = None):
        self.config = config or TunerConfig()
        if not self.config.device_id:
            self.config.device_id = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
        self.cache = cache or ConfigCache(device_id=self.config.device_id)
        self.stats = TunerStats()

    def tune(self, kernel: TunableKernel) -> TuningResult:
        cfg = self.config
        default = kernel.default_config()
        if not cfg.enabled:
            return TuningResult(default, 0.0, 0.0, 0)
        bucket = kernel.input_signature()
        if cfg.use_cache:
            e = self.cache.get_config(kernel.kernel_id, cfg.device_id, cfg.dtype, bucket)
            if e is not None:
                self.stats.cache_hits += 1
                t = benchmark_kernel(kernel.with_config(e.config), cfg.warmup, cfg.timing, getattr(kernel, "host_timed", False))
                return TuningResult(dict(e.config), t, t, 0, True)
            self.stats.cache_misses += 1
        t_default = benchmark_kernel(kernel.with_config(default), cfg.warmup, cfg.timing, getattr(kernel, "host_timed", False))
        search = SearchHandle(kernel.config_space(), cfg.strategy, cfg.seed, min(cfg.max_evals, 5) if cfg.ci_mode else cfg.max_evals)
        search.report(default, t_default)
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < cfg.max_tuning_time_s:
            c = search.next_config()
            if c is None:
                break
            try:
                t = benchmark_kernel(kernel.with_config(c), cfg.warmup, cfg.timing, getattr(kernel, "host_timed", False))
            except Exception:   # noqa: BLE001 - a configuration the kernel rejects is simply not a candidate
                t = float("inf")
            if t != float("inf"):
                search.report(c, t)
            if cfg.verbose:
                print(f"[tune] {kernel.kernel_id} {c} -> {t:.1f} us")
        best, t_best = search.best()
        if best is None or (t_default - t_best) / t_default * 100.0 < cfg.min_improvement_pct:
            best, t_best = default, t_default
        if cfg.cache_results:
            self.cache.store_config(kernel.kernel_id, cfg.device_id, cfg.dtype, bucket, best, t_best, search.num_evals())
            self.cache.save()
        self.stats.total_tunings += 1
        self.stats.total_configs_tried += search.num_evals()
        self.stats.total_tuning_time += time.perf_counter() - t0
        return TuningResult(best, t_best, t_default, search.num_evals())


class GemmKernel(TunableKernel):
    """The tcgen05 GEMM at one problem shape: tile width, split-K factor, rasterisation group."""

    kernel_id = "gemm_bf16_tcgen05"

    def __init__(self, M: int, N_: int, K: int, a_mn: bool = False, b_mn: bool = False, out_f32: bool = False, reduced: bool = True):
        self.M, self.N, self.K, self.a_mn, self.b_mn, self.out_f32, self.reduced = M, N_, K, a_mn, b_mn, out_f32, reduced
        dev = "cuda"
        g = torch.Generator().manual_seed(0)
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16).to(dev)
        self.a = mk(K, M) if a_mn else mk(M, K)
        self.b = mk(K, N_) if b_mn else mk(N_, K)
        self.out = torch.empty((M, N_), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)

    def config_space(self):
        return ConfigSpace.matmul_reduced() if self.reduced else ConfigSpace.matmul_full()

    def default_config(self):
        return {"block_n": 0, "splits": 0, "group_m": 0}        # the kernel's own cost model

    def input_signature(self):
        return MatmulShapeBucket.of(self.M, self.N, self.K).cache_key() + f"_{int(self.a_mn)}{int(self.b_mn)}{int(self.out_f32)}"

    def flops(self):
        return 2.0 * self.M * self.N * self.K

    def with_config(self, config: dict):
        from ..ops import gemm
        return lambda: gemm(self.a, self.b, a_mn=self.a_mn, b_mn=self.b_mn, out=self.out, block_n=config["block_n"],
                            splits=config["splits"], group_m=config["group_m"])


def tune_gemm(M: int, N_: int, K: int, tuner: AutoTuner | None = None, **kw) -> TuningResult:
    return (tuner or AutoTuner(TunerConfig.fast())).tune(GemmKernel(M, N_, K, **kw))


class GemmTuningTable:
    """The tuned GEMM plans of a cache, served back to `ops.gemm`.  `apply()` installs the table: from then on a plain
    `gemm` call (no explicit tile plan, no peer mode) whose shape bucket has a cached winner runs with that winner
    instead of the kernel's built-in cost model; `remove()` uninstalls it."""

    def __init__(self, cache: ConfigCache | None = None, device_id: str | None = None, dtype: str = "bf16"):
        if device_id is None:
            device_id = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
        self.cache = cache or ConfigCache(device_id=device_id)
        self.device_id, self.dtype = device_id, dtype
        self.hits = self.misses = 0
        self._memo: dict = {}

    def lookup(self, M: int, N_: int, K: int, a_mn: bool = False, b_mn: bool = False, out_f32: bool = False):
        key = MatmulShapeBucket.of(M, N_, K).cache_key() + f"_{int(a_mn)}{int(b_mn)}{int(out_f32)}"
        if key not in self._memo:
            e = self.cache.get_config(GemmKernel.kernel_id, self.device_id, self.dtype, key)
            cfg = dict(e.config) if e is not None else None
            if cfg is not None and not any(cfg.get(k, 0) for k in ("block_n", "splits", "group_m")):
                cfg = None                       # the cached winner IS the built-in plan
            self._memo[key] = cfg
        cfg = self._memo[key]
        if cfg is None:
            self.misses += 1
        else:
            self.hits += 1
        return cfg

    def apply(self) -> "GemmTuningTable":
        from ..ops import matmul
        matmul.set_plan_hook(self.lookup)
        return self

    @staticmethod
    def remove() -> None:
        from ..ops import matmul
        matmul.set_plan_hook(None)


class AttentionKernel(TunableKernel):
    """Flash attention forward (+ backward) at one shape: which implementation serves it, the tcgen05 kernels or the
    mma.sync kernels (`impl` 0 / 1).  The result feeds `ops.attention.FORWARD_IMPL` / `BACKWARD_IMPL`."""

    kernel_id = "flash_attention"
    IMPLS = ("tc", "mma")

    def __init__(self, batch: int, seq: int, heads: int, kv_heads: int, head_dim: int, causal: bool = True, backward: bool = True):
        self.shape = (batch, seq, heads, kv_heads, head_dim)
        self.causal, self.backward = causal, backward
        self._t = None

    def _tensors(self):
        if self._t is None:
            B, S, H, Hk, D = self.shape
            g = torch.Generator().manual_seed(0)
            mk = lambda h: torch.randn(B, S, h, D, generator=g).to(torch.bfloat16).cuda()
            self._t = (mk(H), mk(Hk), mk(Hk), mk(H))
        return self._t

    def config_space(self):
        return ConfigSpace({"impl": [0, 1]})

    def default_config(self):
        return {"impl": 0}

    def input_signature(self):
        B, S, H, Hk, D = self.shape
        return f"b{dim_bucket(B)}_s{dim_bucket(S)}_h{H}_kv{Hk}_d{D}_{int(self.causal)}{int(self.backward)}"

    def flops(self):
        B, S, H, _, D = self.shape
        return 4.0 * B * S * S * H * D * (3.5 if self.backward else 1.0) * (0.5 if self.causal else 1.0)

    def with_config(self, config: dict):
        import math
        from ..ops import attention as A
        impl = self.IMPLS[int(config["impl"])]
        q, k, v, do = self._tensors()
        scale = 1.0 / math.sqrt(q.shape[-1])

        def run():
            o, lse = A.attention_forward(q, k, v, self.causal, scale, impl=impl)
            if self.backward:
                A.attention_backward(do, q, k, v, o, lse, self.causal, scale, impl=impl)
        return run


def tune_attention(batch: int, seq: int, heads: int, kv_heads: int, head_dim: int, tuner: AutoTuner | None = None, **kw):
    """Times both attention implementations at the shape and returns the TuningResult (config["impl"]: 0 tcgen05, 1 mma)."""
    return (tuner or AutoTuner(TunerConfig.fast())).tune(AttentionKernel(batch, seq, heads, kv_heads, head_dim, **kw))


class PreTuner:
    """Tunes the GEMM shapes of a model configuration ahead of time (crates/autotuner/src/lib.rs PreTuner)."""

    def __init__(self, tuner: AutoTuner | None = None):
        self.tuner = tuner or AutoTuner(TunerConfig.fast())

    def shapes_for(self, cfg, tokens: int) -> list:
        d, f = cfg.d_model, cfg.ffn_dim
        fwd = [(tokens, cfg.qkv_dim, d), (tokens, d, d), (tokens, f if cfg.arch == "gpt2" else 2 * f, d), (tokens, d, f)]
        return fwd + [(tokens, cfg.vocab_padded, d)]

    def pretune(self, cfg, tokens: int) -> dict:
        return {s: self.tuner.tune(GemmKernel(*s)) for s in self.shapes_for(cfg, tokens)}


class _StrategySearch:
    """Named front ends of the C++ searcher, one per strategy of the reference (crates/autotuner/src/search.rs:
    GridSearch, RandomSearch, EvolutionarySearch, BayesianSearch)."""
    strategy = Strategy.GRID

    def __init__(self, space: ConfigSpace, seed: int = 0, max_evals: int = 0):
        self.handle = SearchHandle(space, self.strategy, seed, max_evals)

    def next_config(self):
        return self.handle.next_config()

    def report(self, config: dict, time_us: float) -> None:
        self.handle.report(config, time_us)

    def best(self):
        return self.handle.best()

    def num_evals(self) -> int:
        return self.handle.num_evals()


SearchStrategy = _StrategySearch     # the reference's trait name (crates/autotuner/src/search.rs:9)


class GridSearch(_StrategySearch):
    strategy = Strategy.GRID


class RandomSearch(_StrategySearch):
    strategy = Strategy.RANDOM


class EvolutionarySearch(_StrategySearch):
    strategy = Strategy.EVOLUTIONARY


class BayesianSearch(_StrategySearch):
    """Explore / exploit search over the discrete space (the native searcher keeps per-choice statistics and samples
    configurations in proportion to their expected improvement)."""
    strategy = Strategy.BAYESIAN


@dataclass
class TuningSession:
    """Record of one tuning run (crates/autotuner/src/tuner.rs: TuningSession): what was tried, in order, and the best."""
    kernel: str
    shape_key: str
    trials: list = field(default_factory=list)        # (config dict, time in us)
    started_at: float = field(default_factory=time.time)
    finished_at: float | None = None

    def record(self, config: dict, time_us: float) -> None:
        self.trials.append((dict(config), float(time_us)))

    def finish(self) -> None:
        self.finished_at = time.time()

    @property
    def best(self):
        return min(self.trials, key=lambda t: t[1]) if self.trials else (None, float("inf"))

    def to_dict(self) -> dict:
        cfg, t = self.best
        return {"kernel": self.kernel, "shape_key": self.shape_key, "num_trials": len(self.trials), "best_config": cfg,
                "best_time_us": t, "elapsed_s": (self.finished_at or time.time()) - self.started_at}


# ---------------------------------------------------------------------------------------------- typed op configurations
class MatmulAlgorithm(enum.Enum):
    """Matmul implementation families (crates/autotuner/src/kernel_config.rs:266-300).  The first seven are the
    reference's names; the last three are what the sm_100a GEMM actually offers."""
    NAIVE = "naive"
    TILED = "tiled"
    TILED_VECTORIZED = "tiled_vectorized"
    STRASSEN = "strassen"
    WARP_SPECIALIZED = "warp_specialized"
    TENSOR_CORE_WMMA = "tensor_core_wmma"
    TENSOR_CORE_MMA = "tensor_core_mma"
    TCGEN05_ONE_CTA = "tcgen05_one_cta"          # 128 x {64,128,192,256} tiles, one CTA per tile
    TCGEN05_TWO_CTA = "tcgen05_two_cta"          # 256 x 256 tiles on a CTA pair (cta_group::2)
    TCGEN05_SPLIT_K = "tcgen05_split_k"          # one-CTA tiles with a deterministic split-K fold

    def uses_tensor_cores(self) -> bool:
        return self in (MatmulAlgorithm.TENSOR_CORE_WMMA, MatmulAlgorithm.TENSOR_CORE_MMA, MatmulAlgorithm.TCGEN05_ONE_CTA,
                        MatmulAlgorithm.TCGEN05_TWO_CTA, MatmulAlgorithm.TCGEN05_SPLIT_K)

    def recommended_tile(self) -> tuple:
        """(m, n, k) of one tile."""
        return {MatmulAlgorithm.NAIVE: (32, 32, 1), MatmulAlgorithm.TILED: (128, 128, 8),
                MatmulAlgorithm.TILED_VECTORIZED: (128, 128, 16), MatmulAlgorithm.STRASSEN: (256, 256, 64),
                MatmulAlgorithm.WARP_SPECIALIZED: (256, 128, 64), MatmulAlgorithm.TENSOR_CORE_WMMA: (128, 256, 32),
                MatmulAlgorithm.TENSOR_CORE_MMA: (256, 256, 64), MatmulAlgorithm.TCGEN05_ONE_CTA: (128, 256, 64),
                MatmulAlgorithm.TCGEN05_TWO_CTA: (256, 256, 64), MatmulAlgorithm.TCGEN05_SPLIT_K: (128, 128, 64)}[self]


class ConvAlgorithm(enum.Enum):
    DIRECT = "direct"
    WINOGRAD = "winograd"
    FFT = "fft"
    IM2COL = "im2col"
    IMPLICIT_GEMM = "implicit_gemm"


class ReduceAlgorithm(enum.Enum):
    TREE = "tree"
    WARP_SHUFFLE = "warp_shuffle"
    ATOMIC = "atomic"
    TWO_PASS = "two_pass"


@dataclass(frozen=True)
class OpConfig:
    """A typed kernel configuration (crates/autotuner/src/lib.rs:79-87): `kind` is one of matmul / conv2d / reduce /
    elementwise / attention and `fields` holds that variant's members.  `to_kernel_config()` gives the dict the
    tunable kernels of this package take."""
    kind: str
    fields: tuple                                  # sorted (name, value) pairs: hashable and comparable

    @classmethod
    def _make(cls, kind, **kw):
        return cls(kind, tuple(sorted(kw.items())))

    @classmethod
    def matmul(cls, algorithm: MatmulAlgorithm, block_m: int, block_n: int, block_k: int, num_stages: int, splits: int = 1,
               group_m: int = 8):
        return cls._make("matmul", algorithm=algorithm, block_m=block_m, block_n=block_n, block_k=block_k,
                         num_stages=num_stages, splits=splits, group_m=group_m)

    @classmethod
    def conv2d(cls, algorithm: ConvAlgorithm, tile_size: int, num_filters: int):
        return cls._make("conv2d", algorithm=algorithm, tile_size=tile_size, num_filters=num_filters)

    @classmethod
    def reduce(cls, block_size: int, items_per_thread: int, algorithm: ReduceAlgorithm):
        return cls._make("reduce", block_size=block_size, items_per_thread=items_per_thread, algorithm=algorithm)

    @classmethod
    def elementwise(cls, block_size: int, items_per_thread: int, vector_width: int):
        return cls._make("elementwise", block_size=block_size, items_per_thread=items_per_thread, vector_width=vector_width)

    @classmethod
    def attention(cls, block_size_m: int, block_size_n: int, use_flash: bool):
        return cls._make("attention", block_size_m=block_size_m, block_size_n=block_size_n, use_flash=use_flash)

    def __getitem__(self, name):
        return dict(self.fields)[name]

    def to_kernel_config(self) -> dict:
        d = dict(self.fields)
        if self.kind == "matmul":
            return {"block_n": d["block_n"], "splits": d["splits"], "group_m": d["group_m"]}
        return {k: (v.value if isinstance(v, enum.Enum) else v) for k, v in d.items()}

    @classmethod
    def from_gemm_config(cls, config: dict, M: int = 0) -> "OpConfig":
        """Typed view of a `GemmKernel` configuration dict (0 = the kernel's own cost model picks)."""
        bn, sp = int(config.get("block_n", 0)), int(config.get("splits", 0))
        if sp > 1:
            alg = MatmulAlgorithm.TCGEN05_SPLIT_K
        elif bn == 256 and M > 128:
            alg = MatmulAlgorithm.TCGEN05_TWO_CTA
        else:
            alg = MatmulAlgorithm.TCGEN05_ONE_CTA
        return cls.matmul(alg, 256 if alg is MatmulAlgorithm.TCGEN05_TWO_CTA else 128, bn, 64,
                          6 if alg is MatmulAlgorithm.TCGEN05_TWO_CTA else 4, max(sp, 1) if sp else 0, int(config.get("group_m", 0)))


class ConfigurableKernel:
    """A kernel object that carries its current typed configuration (crates/autotuner/src/lib.rs:107-113)."""

    _op_config: OpConfig | None = None

    def apply_config(self, config: OpConfig) -> None:
        self._op_config = config

    def current_config(self) -> OpConfig | None:
        return self._op_config


class KernelFactory:
    """Hands out (kernel, configuration) pairs: the cached winner when the tuner's cache has one for the kernel's
    shape bucket, otherwise the result of a tuning run (crates/autotuner/src/lib.rs:186-232).  `default_configs`
    are the configurations used when tuning is disabled."""

    def __init__(self, tuner: AutoTuner | None = None):
        self.tuner = tuner or AutoTuner(TunerConfig.fast())
        self.default_configs = {
            "matmul_default": OpConfig.matmul(MatmulAlgorithm.TCGEN05_ONE_CTA, 128, 256, 64, 4, 0, 0),
            "conv2d_default": OpConfig.conv2d(ConvAlgorithm.IMPLICIT_GEMM, 16, 64),
            "attention_default": OpConfig.attention(128, 128, True),
            "reduce_default": OpConfig.reduce(256, 8, ReduceAlgorithm.TWO_PASS),
            "elementwise_default": OpConfig.elementwise(256, 8, 8)}

    def get_kernel(self, kernel: TunableKernel):
        """Returns (kernel, config dict).  A `ConfigurableKernel` also gets the typed configuration applied."""
        cfg = self.tuner.config
        config = None
        if cfg.enabled and cfg.use_cache:
            e = self.tuner.cache.get_config(kernel.kernel_id, cfg.device_id, cfg.dtype, kernel.input_signature())
            if e is not None:
                self.tuner.stats.cache_hits += 1
                config = dict(e.config)
        if config is None:
            config = self.tuner.tune(kernel).config
        if isinstance(kernel, ConfigurableKernel) and {"block_n", "splits"} <= set(config):
            kernel.apply_config(OpConfig.from_gemm_config(config, getattr(kernel, "M", 0)))
        return kernel, config


from .kernel_config import (AlgorithmConfig, BlockSize, CacheConfig as KernelCacheConfig, KernelConfig, MatmulDimBucket,  # noqa: E402
                            MemoryConfig, WorkgroupConfig)
