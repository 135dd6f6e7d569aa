"""OperationProfiler: per-op timing with CUDA events (crates/core/src/operation_profiler.rs:45-623).

The reference times every op with the host clock, including its "gpu" column.  Here an op recorded on a CUDA
stream is bracketed by two CUDA events on that stream; elapsed times are resolved lazily (at report time or when
the pending list grows), so profiling adds no synchronisation to the hot loop.  Host ops use perf_counter.
"""
from __future__ import annotations

import enum
import json
import os
import time
from dataclasses import dataclass, field

import torch


class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"


def shape_bucket(shape) -> str:
    """Coarse shape key: every dimension rounded up to a power of two (crates/core/src/operation_profiler.rs:108)."""
    if shape is None:
        return "-"
    out = []
    for d in shape:
        d = int(d)
        b = 1
        while b < d:
            b <<= 1
        out.append(str(b))
    return "x".join(out) if out else "scalar"


@dataclass
class OperationStats:
    count: int = 0
    total_ms: float = 0.0
    min_ms: float = float("inf")
    max_ms: float = 0.0
    last_ms: float = 0.0
    cpu_ms: float = 0.0
    gpu_ms: float = 0.0
    device_type: str = "cpu"
    shape_buckets: dict = field(default_factory=dict)

    def record(self, ms: float, device: DeviceType, bucket: str) -> None:
        self.count += 1
        self.total_ms += ms
        self.min_ms = min(self.min_ms, ms)
        self.max_ms = max(self.max_ms, ms)
        self.last_ms = ms
        if device is DeviceType.CUDA:
            self.gpu_ms += ms
        else:
            self.cpu_ms += ms
        self.device_type = device.value
        self.shape_buckets[bucket] = self.shape_buckets.get(bucket, 0) + 1

    @property
    def mean_ms(self) -> float:
        return self.total_ms / self.count if self.count else 0.0

    def to_dict(self) -> dict:
        return {"count": self.count, "total_ms": self.total_ms, "mean_ms": self.mean_ms,
                "min_ms": 0.0 if self.count == 0 else self.min_ms, "max_ms": self.max_ms, "last_ms": self.last_ms,
                "cpu_ms": self.cpu_ms, "gpu_ms": self.gpu_ms, "device_type": self.device_type,
                "shape_buckets": dict(self.shape_buckets)}


class MatmulDim(enum.Enum):
    """Size class of one GEMM dimension: Tiny < 256, Small <= 512, Medium < 2048, Large < 8192, XLarge
    (crates/core/src/operation_profiler.rs:123-146)."""
    TINY = "tiny"
    SMALL = "small"
    MEDIUM = "medium"
    LARGE = "large"
    XLARGE = "xlarge"

    @classmethod
    def from_size(cls, size: int) -> "MatmulDim":
        return cls.TINY if size < 256 else cls.SMALL if size <= 512 else cls.MEDIUM if size < 2048 else \
            cls.LARGE if size < 8192 else cls.XLARGE


@dataclass(frozen=True)
class ShapeBucket:
    """Coarse class of a tensor shape for aggregating timings (crates/core/src/operation_profiler.rs:108-184): Small / Medium
    / Large / XLarge by the largest dimension (< 512, < 2048, < 8192), or a matmul bucket of three `MatmulDim`s.
    `shape_bucket()` above is the finer power-of-two key the profiler records by default."""
    kind: str                       # "small" | "medium" | "large" | "xlarge" | "matmul"
    m: MatmulDim | None = None
    n: MatmulDim | None = None
    k: MatmulDim | None = None

    @classmethod
    def from_dims(cls, dims) -> "ShapeBucket":
        mx = max((int(d) for d in dims), default=0)
        return cls("small" if mx < 512 else "medium" if mx < 2048 else "large" if mx < 8192 else "xlarge")

    @classmethod
    def from_matmul_dims(cls, m: int, n: int, k: int) -> "ShapeBucket":
        return cls("matmul", MatmulDim.from_size(m), MatmulDim.from_size(n), MatmulDim.from_size(k))

    def __str__(self) -> str:
        return self.kind if self.kind != "matmul" else f"matmul[{self.m.value},{self.n.value},{self.k.value}]"


@dataclass
class ProfilingHooks:
    """Which measurements a profiler takes (crates/core/src/operation_profiler.rs:45-75).  `OperationProfiler.with_hooks`
    applies them: without `per_op_timing` guards record nothing, without `cpu_gpu_breakdown` everything is timed on the
    host clock, without `shape_bucket_recording` all calls of an operation share one bucket."""
    cpu_gpu_breakdown: bool = True
    per_op_timing: bool = True
    memory_tracking: bool = False
    shape_bucket_recording: bool = True

    @classmethod
    def all(cls) -> "ProfilingHooks":
        return cls(True, True, True, True)

    @classmethod
    def none(cls) -> "ProfilingHooks":
        return cls(False, False, False, False)


@dataclass
class SnapshotOp:
    """One row of a profiler snapshot (crates/core/src/operation_profiler.rs:341-347)."""
    name: str
    count: int
    avg_ms: float
    max_ms: float
    device_type: str


@dataclass
class ProfilerSnapshot:
    ops: dict
    total_ms: float

    def rows(self) -> list:
        """The operations as `SnapshotOp` rows, most expensive first."""
        out = [SnapshotOp(n, int(d.get("count", 0)), float(d.get("mean_ms", d.get("total_ms", 0.0) / max(1, d.get("count", 1)))),
                          float(d.get("max_ms", 0.0)), str(d.get("device_type", "cpu"))) for n, d in self.ops.items()]
        return sorted(out, key=lambda r: -r.avg_ms * r.count)

    def to_json(self) -> str:
        return json.dumps({"total_ms": self.total_ms, "ops": self.ops}, indent=2, sort_keys=True)


class OperationGuard:
    """RAII-style guard: records on exit."""

    def __init__(self, profiler: "OperationProfiler", name: str, shape=None, device: DeviceType | None = None):
        self.p, self.name, self.bucket = profiler, name, shape_bucket(shape)
        self.device = device
        self._t0 = 0.0
        self._ev = None

    def __enter__(self):
        dev = self.device
        if dev is None:
            dev = DeviceType.CUDA if (self.p.use_cuda_events and torch.cuda.is_available()) else DeviceType.CPU
        self.device = dev
        if dev is DeviceType.CUDA:
            if self.p.nvtx:
                torch.cuda.nvtx.range_push(self.name)      # shows up as a named range in Nsight timelines
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.device is DeviceType.CUDA:
            self._ev[1].record()
            if self.p.nvtx:
                torch.cuda.nvtx.range_pop()
            self.p._pending.append((self.name, self.bucket, self._ev))
            if len(self.p._pending) >= self.p.max_pending:
                self.p.resolve()
        else:
            self.p.record(self.name, (time.perf_counter() - self._t0) * 1e3, DeviceType.CPU, self.bucket)
        return False


class OperationProfiler:
    def __init__(self, enabled: bool = True, use_cuda_events: bool = True, max_pending: int = 4096,
                 nvtx: bool | None = None):
        self.enabled = enabled
        self.use_cuda_events = use_cuda_events
        # NVTX ranges around CUDA-timed operations (RUSTRAL_PROFILE_NVTX=1 turns them on by default)
        self.nvtx = (os.environ.get("RUSTRAL_PROFILE_NVTX", "0") == "1") if nvtx is None else nvtx
        self.max_pending = max_pending
        self.stats: dict = {}
        self._pending: list = []
        self.hooks = ProfilingHooks()

    def with_hooks(self, hooks: ProfilingHooks) -> "OperationProfiler":
        self.hooks = hooks
        self.enabled = self.enabled and hooks.per_op_timing
        self.use_cuda_events = self.use_cuda_events and hooks.cpu_gpu_breakdown
        return self

    @classmethod
    def ci_safe(cls) -> "OperationProfiler":
        """Low-overhead preset: host timing only."""
        return cls(enabled=True, use_cuda_events=False)

    def guard(self, name: str, shape=None, device: DeviceType | None = None):
        if not self.enabled:
            return _NULL
        return OperationGuard(self, name, shape, device)

    def record(self, name: str, ms: float, device: DeviceType = DeviceType.CPU, bucket: str = "-") -> None:
        if not self.hooks.shape_bucket_recording:
            bucket = "-"
        self.stats.setdefault(name, OperationStats()).record(ms, device, bucket)

    def resolve(self) -> None:
        """Turns pending CUDA event pairs into times (synchronises on the last event)."""
        if not self._pending:
            return
        self._pending[-1][2][1].synchronize()
        for name, bucket, (e0, e1) in self._pending:
            self.record(name, e0.elapsed_time(e1), DeviceType.CUDA, bucket)
        self._pending.clear()

    def most_expensive_ops(self, n: int = 10) -> list:
        self.resolve()
        return sorted(self.stats.items(), key=lambda kv: -kv[1].total_ms)[:n]

    def total_ms(self) -> float:
        self.resolve()
        return sum(s.total_ms for s in self.stats.values())

    def print_report(self, limit: int = 20, file=None) -> None:
        import sys
        file = file or sys.stdout
        tot = self.total_ms() or 1.0
        print(f"{'op':32s} {'count':>8s} {'total ms':>12s} {'mean ms':>10s} {'share':>7s} dev", file=file)
        for name, s in self.most_expensive_ops(limit):
            print(f"{name[:32]:32s} {s.count:8d} {s.total_ms:12.3f} {s.mean_ms:10.4f} {100 * s.total_ms / tot:6.1f}% "
                  f"{s.device_type}", file=file)

    def export_json(self, path: str | None = None) -> str:
        self.resolve()
        text = json.dumps({k: v.to_dict() for k, v in self.stats.items()}, indent=2, sort_keys=True)
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text

    def snapshot(self, limit: int = 64) -> ProfilerSnapshot:
        ops = {k: v.to_dict() for k, v in self.most_expensive_ops(limit)}
        return ProfilerSnapshot(ops, self.total_ms())

    def check_regression(self, baseline: dict, threshold: float = 0.2) -> list:
        """Ops whose mean time grew by more than `threshold` (fraction) over `baseline` (name -> mean ms or stats dict)."""
        self.resolve()
        out = []
        for name, base in baseline.items():
            base_ms = base["mean_ms"] if isinstance(base, dict) else float(base)
            cur = self.stats.get(name)
            if cur is None or base_ms <= 0:
                continue
            if cur.mean_ms > base_ms * (1.0 + threshold):
                out.append((name, base_ms, cur.mean_ms))
        return out

    def export_regression_report(self, baseline: dict, threshold: float = 0.2) -> str:
        regs = self.check_regression(baseline, threshold)
        return json.dumps({"threshold": threshold,
                           "regressions": [{"op": n, "baseline_ms": b, "current_ms": c, "ratio": c / b} for n, b, c in regs]},
                          indent=2)

    def reset(self) -> None:
        self.stats.clear()
        self._pending.clear()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL = _Null()


def operation_profiler_from_env():
    """RUSTRAL_PROFILE=1 enables profiling; CI or RUSTRAL_PROFILE_CI=1 selects the ci_safe preset
    (crates/runtime/src/tape_trainer.rs:16-23)."""
    import os
    if os.environ.get("RUSTRAL_PROFILE", "0") not in ("1", "true", "yes"):
        return None
    if os.environ.get("CI") or os.environ.get("RUSTRAL_PROFILE_CI") == "1":
        return OperationProfiler.ci_safe()
    return OperationProfiler()


def finish_profile_from_env(profiler) -> None:
    """Prints the report and honours RUSTRAL_PROFILE_EXPORT_JSON / RUSTRAL_PROFILE_SNAPSHOT_LIMIT."""
    import os
    if profiler is None:
        return
    profiler.print_report()
    path = os.environ.get("RUSTRAL_PROFILE_EXPORT_JSON")
    if path:
        limit = int(os.environ.get("RUSTRAL_PROFILE_SNAPSHOT_LIMIT", "64"))
        with open(path, "w") as f:
            f.write(profiler.snapshot(limit).to_json())
