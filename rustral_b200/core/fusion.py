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


class OpType(enum.Enum):
    """Kinds of operation the pattern matcher tells apart (crates/core/src/fusion.rs:82-89)."""
    MATMUL = "matmul"
    ADD_BIAS = "add_row_vector"
    RELU = "relu"
    GELU = "gelu"
    SILU = "silu"
    UNKNOWN = "unknown"

    @classmethod
    def of(cls, name: str) -> "OpType":
        for m in cls:
            if m.value == name:
                return m
        return cls.ADD_BIAS if name in ("add_bias", "bias_add") else cls.UNKNOWN


@dataclass
class Op:
    """One recorded operation: its kind and the shapes it read and wrote (crates/core/src/fusion.rs:91-105)."""
    op_type: OpType
    input_shapes: list
    output_shape: list


class PatternMatcher:
    """Finds fusable op sequences in a list of op names, e.g. ["matmul", "add_row_vector", "gelu"]."""

    def find_in_ops(self, ops) -> list:
        """`find` over `Op` records; a pattern only matches when the shapes chain (each output feeds the next input)."""
        ops = list(ops)
        hits = []
        for start, length, pat in self.find([o.op_type.value for o in ops]):
            chain = ops[start:start + length]
            if all(list(b.input_shapes[0]) == list(a.output_shape) for a, b in zip(chain, chain[1:]) if b.input_shapes):
                hits.append((start, length, pat))
        return hits
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


@dataclass
class FusionTestConfig:
    """crates/core/src/fusion_tests.rs:11-31: `strict_numerics` allows no element outside the tolerance,
    `num_random_cases` is how many seeds `run_random_cases` draws.  `use_float64_reference` is accepted so that
    configurations carry over; the comparison arithmetic here is float64 in either case."""
    strict_numerics: bool = False
    use_float64_reference: bool = False
    num_random_cases: int = 10
    verbose: bool = False


@dataclass
class FusionTestSuiteResult:
    suite_name: str
    total_tests: int
    passed_tests: int
    avg_speedup: float
    results: list

    def all_passed(self) -> bool:
        return self.passed_tests == self.total_tests

    def print_summary(self, file=None) -> None:
        import sys
        out = file or sys.stdout
        print(f"=== fusion test suite: {self.suite_name} ===", file=out)
        print(f"passed: {self.passed_tests}/{self.total_tests}   average speed-up: {self.avg_speedup:.2f}x", file=out)
        for name, r in self.results:
            print(f"  {name}: {'ok' if r.passed else 'FAILED'}  max |diff| {r.max_abs_err:.3g}  x{r.speedup:.2f}", file=out)

    def __str__(self) -> str:
        return f"{self.suite_name}: {self.passed_tests}/{self.total_tests} passed, average speed-up {self.avg_speedup:.2f}x"


class FusionTestHarness:
    """Runs an unfused and a fused closure on the same inputs, compares numerics and times both."""

    def __init__(self, validator: NumericsValidator | None = None, repeats: int = 5, config: FusionTestConfig | None = None):
        self.config = config or FusionTestConfig()
        if validator is None:
            from .numerics import NumericsConfig
            validator = NumericsValidator(NumericsConfig(strict=self.config.strict_numerics))
        self.validator = validator
        self.repeats = repeats

    def run_suite(self, suite_name: str, test_cases, dtype: DType = DType.F32) -> FusionTestSuiteResult:
        """`test_cases`: (name, unfused_fn, fused_fn) triples (crates/core/src/fusion_tests.rs:172-240)."""
        results = [(name, self.run_test(u, f, dtype)) for name, u, f in test_cases]
        if self.config.verbose:
            for name, r in results:
                print(f"[fusion] {name}: passed={r.passed} max|diff|={r.max_abs_err:.3g} x{r.speedup:.2f}")
        speed = [r.speedup for _, r in results if r.speedup != float("inf")]
        return FusionTestSuiteResult(suite_name, len(results), sum(r.passed for _, r in results),
                                     sum(speed) / len(speed) if speed else 0.0, results)

    def run_random_cases(self, suite_name: str, make_case, dtype: DType = DType.F32) -> FusionTestSuiteResult:
        """`make_case(seed) -> (unfused_fn, fused_fn)`, drawn `config.num_random_cases` times."""
        return self.run_suite(suite_name, [(f"seed{s}", *make_case(s)) for s in range(self.config.num_random_cases)], dtype)

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
