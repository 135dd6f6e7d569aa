"""Fusion patterns and the fused-vs-unfused test harness (crates/core/src/fusion.rs:22-363, fusion_tests.rs:91-330).

On this backend the fused form always exists (bias and activation ride in the GEMM epilogue), so FusionOptimizer
never needs its fallback on CUDA; the pattern matcher is kept for graph-level tooling and for API parity.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass

import torch

from .numerics import DType, NumericsValidator


class FusionPattern(enum.Enum):
    MATMUL_BIAS = "matmul_bias"
    MATMUL_BIAS_RELU = "matmul_bias_relu"
    MATMUL_BIAS_GELU = "matmul_bias_gelu"
    MATMUL_BIAS_SILU = "matmul_bias_silu"

    @property
    def activation(self) -> str:
        return {"matmul_bias": "none", "matmul_bias_relu": "relu", "matmul_bias_gelu": "gelu",
                "matmul_bias_silu": "silu"}[self.value]


class PatternMatcher:
    """Finds fusable op sequences in a list of op names, e.g. ["matmul", "add_row_vector", "gelu"]."""
    SEQUENCES = [
        (("matmul", "add_row_vector", "relu"), FusionPattern.MATMUL_BIAS_RELU),
        (("matmul", "add_row_vector", "gelu"), FusionPattern.MATMUL_BIAS_GELU),
        (("matmul", "add_row_vector", "silu"), FusionPattern.MATMUL_BIAS_SILU),
        (("linear", "relu"), FusionPattern.MATMUL_BIAS_RELU),
        (("linear", "gelu"), FusionPattern.MATMUL_BIAS_GELU),
        (("matmul", "add_row_vector"), FusionPattern.MATMUL_BIAS),
    ]

    def find(self, op_names) -> list:
        ops = list(op_names)
        out, i = [], 0
        while i < len(ops):
            for seq, pat in self.SEQUENCES:
                if tuple(ops[i:i + len(seq)]) == seq:
                    out.append((i, len(seq), pat))
                    i += len(seq) - 1
                    break
            i += 1
        return out


class FusionOptimizer:
    """apply_* entry points: one fused kernel; falls back to matmul + add + activation if the backend has no
    fusion table (never the case for the two backends of this package)."""

    def __init__(self, backend):
        self.backend = backend

    def apply(self, pattern: FusionPattern, x, w, b):
        f = self.backend.fusion_ops()
        if f is not None:
            return self.backend.ops()._gemm(x, w, b, pattern.activation)
        o = self.backend.ops()
        y = o.add_row_vector(o.matmul(x, o.transpose(w)), b)
        act = pattern.activation
        return y if act == "none" else getattr(o, act)(y)

    def apply_matmul_bias(self, x, w, b): return self.apply(FusionPattern.MATMUL_BIAS, x, w, b)
    def apply_matmul_bias_relu(self, x, w, b): return self.apply(FusionPattern.MATMUL_BIAS_RELU, x, w, b)
    def apply_matmul_bias_gelu(self, x, w, b): return self.apply(FusionPattern.MATMUL_BIAS_GELU, x, w, b)


@dataclass
class FusionTestResult:
    passed: bool
    max_abs_err: float
    unfused_ms: float
    fused_ms: float

    @property
    def speedup(self) -> float:
        return self.unfused_ms / self.fused_ms if self.fused_ms > 0 else float("inf")


def generate_random_data(shape, seed: int = 0, scale: float = 1.0) -> torch.Tensor:
    return torch.randn(tuple(shape), generator=torch.Generator().manual_seed(seed)) * scale


class FusionTestHarness:
    """Runs an unfused and a fused closure on the same inputs, compares numerics and times both."""

    def __init__(self, validator: NumericsValidator | None = None, repeats: int = 5):
        self.validator = validator or NumericsValidator()
        self.repeats = repeats

    def _time(self, fn):
        cuda = torch.cuda.is_available()
        out = fn()
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(self.repeats):
            out = fn()
        if cuda:
            torch.cuda.synchronize()
        return out, (time.perf_counter() - t0) * 1e3 / self.repeats

    def run_test(self, unfused_fn, fused_fn, dtype: DType = DType.F32) -> FusionTestResult:
        ref, t_ref = self._time(unfused_fn)
        got, t_got = self._time(fused_fn)
        rep = self.validator.validate_arrays(got.detach().float().cpu(), ref.detach().float().cpu(), dtype)
        return FusionTestResult(rep.ok, rep.max_abs_err, t_ref, t_got)
