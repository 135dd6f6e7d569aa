"""Benchmark harness with the reference's schema-v2 JSON output (crates/bench/src/lib.rs; benchmarks/SCHEMA.md)."""
from __future__ import annotations

import json
import math
import os
import platform
import socket
import statistics
import subprocess
import time
from dataclasses import dataclass, field

import torch

SCHEMA_VERSION = "2.0.0"

_T95 = {1: 12.706, 2: 4.303, 3: 3.182, 4: 2.776, 5: 2.571, 6: 2.447, 7: 2.365, 8: 2.306, 9: 2.262, 10: 2.228, 15: 2.131,
        20: 2.086, 30: 2.042, 60: 2.000, 120: 1.980}


@dataclass
class Sample:
    name: str
    backend: str
    device: str
    dtype: str
    model_params: int | None
    params: dict
    runs_ms: list = field(default_factory=list)


def time_runs(fn, warmup: int = 3, repeats: int = 10, cuda: bool | None = None) -> list:
    """Milliseconds per call.  On a GPU each repeat is bracketed by CUDA events on the current stream."""
    cuda = torch.cuda.is_available() if cuda is None else cuda
    for _ in range(warmup):
        fn()
    out = []
    if cuda:
        torch.cuda.synchronize()
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            out.append(e0.elapsed_time(e1))
    else:
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn()
            out.append((time.perf_counter() - t0) * 1e3)
    return out


def _t_crit(df: int) -> float:
    if df <= 0:
        return float("nan")
    keys = sorted(_T95)
    for k in keys:
        if df <= k:
            return _T95[k]
    return 1.96


def ci95_mean_ms(runs) -> tuple:
    """(mean, half-width of the 95% confidence interval) with Student's t."""
    n = len(runs)
    if n == 0:
        return float("nan"), float("nan")
    mean = sum(runs) / n
    if n < 2:
        return mean, float("nan")
    sd = statistics.stdev(runs)
    return mean, _t_crit(n - 1) * sd / math.sqrt(n)


def tukey_iqr_outlier_indices(runs) -> list:
    if len(runs) < 4:
        return []
    s = sorted(runs)
    q1, q3 = statistics.quantiles(s, n=4)[0], statistics.quantiles(s, n=4)[2]
    lo, hi = q1 - 1.5 * (q3 - q1), q3 + 1.5 * (q3 - q1)
    return [i for i, v in enumerate(runs) if v < lo or v > hi]


def _git_sha() -> str:
    if os.environ.get("GIT_SHA"):
        return os.environ["GIT_SHA"]
    try:
        return subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5,
                              cwd=os.path.dirname(os.path.abspath(__file__))).stdout.strip() or "unknown"
    except OSError:
        return "unknown"


def machine_info() -> dict:
    info = {"os": platform.system().lower(), "arch": platform.machine(), "hostname": socket.gethostname(),
            "python": platform.python_version(), "torch": torch.__version__, "commit": _git_sha(),
            "features": os.environ.get("RUSTRAL_BENCH_FEATURES", "sm_100a")}
    if torch.cuda.is_available():
        info["gpu"] = torch.cuda.get_device_name(0)
    return info


def samples_to_json(samples, suite: str = "rustral_b200") -> str:
    out = []
    for s in samples:
        mean, ci = ci95_mean_ms(s.runs_ms)
        out.append({"name": s.name, "backend": s.backend, "device": s.device, "dtype": s.dtype, "model_params": s.model_params,
                    "params": s.params, "runs_ms": s.runs_ms, "mean_ms": mean, "ci95_ms": None if ci != ci else ci,
                    "min_ms": min(s.runs_ms) if s.runs_ms else None, "outliers": tukey_iqr_outlier_indices(s.runs_ms)})
    return json.dumps({"schema_version": SCHEMA_VERSION, "suite": suite, "machine": machine_info(), "samples": out}, indent=1)


def validate_schema(doc: dict) -> list:
    """Returns a list of problems (empty when the document follows schema v2)."""
    errs = []
    if doc.get("schema_version") != SCHEMA_VERSION:
        errs.append("schema_version must be 2.0.0")
    for k in ("suite", "machine", "samples"):
        if k not in doc:
            errs.append(f"missing {k}")
    for i, s in enumerate(doc.get("samples", [])):
        for k in ("name", "backend", "device", "dtype", "params", "runs_ms"):
            if k not in s:
                errs.append(f"samples[{i}] missing {k}")
        if not isinstance(s.get("runs_ms", None), list) or not s.get("runs_ms"):
            errs.append(f"samples[{i}].runs_ms must be a non-empty list")
    return errs
