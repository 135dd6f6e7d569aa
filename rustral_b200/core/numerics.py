"""Numeric tolerances and validation (crates/core/src/numerics.rs:11-340, tolerance.rs:10-170)."""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class DType(enum.Enum):
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"
    F64 = "f64"


@dataclass(frozen=True)
class Tolerance:
    rtol: float
    atol: float
    max_ulps: int = 0

    def is_close(self, a: float, b: float) -> bool:
        return abs(a - b) <= self.atol + self.rtol * abs(b)


class NumericsConfig:
    """Per-dtype defaults: f32 1e-5/1e-8; f16 and bf16 1e-3/1e-6 with 4 ulps; f64 1e-12/1e-15."""
    DEFAULTS = {DType.F32: Tolerance(1e-5, 1e-8), DType.F16: Tolerance(1e-3, 1e-6, 4),
                DType.BF16: Tolerance(1e-2, 1e-3, 4), DType.F64: Tolerance(1e-12, 1e-15)}

    def __init__(self, overrides: dict | None = None, strict: bool = False, max_violation_fraction: float = 0.01):
        self.table = dict(self.DEFAULTS)
        self.table.update(overrides or {})
        self.strict = strict
        self.max_violation_fraction = max_violation_fraction

    def for_dtype(self, dt: DType) -> Tolerance:
        return self.table[dt]


@dataclass
class ValidationReport:
    ok: bool
    max_abs_err: float
    max_rel_err: float
    violations: int
    total: int
    has_nan: bool


@dataclass
class ValidationResult:
    """The comparison outcome under the reference's field names (crates/core/src/numerics.rs:228-275)."""
    passed: bool
    max_abs_diff: float
    max_rel_diff: float
    num_violations: int
    total_elements: int

    def violation_rate(self) -> float:
        """Share of elements outside the tolerance, in per cent."""
        return 100.0 * self.num_violations / self.total_elements if self.total_elements else 0.0


class NumericsError(AssertionError):
    """Raised by `NumericsValidator.check`: a tolerance was exceeded, a length differed or a NaN appeared
    (crates/core/src/numerics.rs:181-212).  `kind` is "tolerance_exceeded", "length_mismatch" or "nan"."""

    def __init__(self, kind: str, message: str, result: "ValidationResult | None" = None):
        super().__init__(message)
        self.kind, self.result = kind, result


class NumericsValidator:
    def __init__(self, config: NumericsConfig | None = None):
        self.config = config or NumericsConfig()

    def validate(self, actual, expected, dtype: DType = DType.F32) -> ValidationResult:
        r = self.validate_arrays(actual, expected, dtype)
        return ValidationResult(r.ok, r.max_abs_err, r.max_rel_err, r.violations, r.total)

    def check(self, actual, expected, dtype: DType = DType.F32, what: str = "") -> ValidationResult:
        """`validate`, raising `NumericsError` instead of returning a failed result."""
        a, e = torch.as_tensor(actual), torch.as_tensor(expected)
        if a.numel() != e.numel():
            raise NumericsError("length_mismatch", f"{what}: {a.numel()} elements against {e.numel()}")
        rep = self.validate_arrays(a, e, dtype)
        res = ValidationResult(rep.ok, rep.max_abs_err, rep.max_rel_err, rep.violations, rep.total)
        if rep.has_nan:
            raise NumericsError("nan", f"{what}: NaN in the values under test", res)
        if not rep.ok:
            tol = self.config.for_dtype(dtype)
            raise NumericsError("tolerance_exceeded", f"{what}: {rep.violations} of {rep.total} elements beyond rtol {tol.rtol:g} / atol "
                                f"{tol.atol:g} for {dtype.value} (max |diff| {rep.max_abs_err:.3g})", res)
        return res

    def validate_arrays(self, actual, expected, dtype: DType = DType.F32) -> ValidationReport:
        a = torch.as_tensor(actual).double().flatten()
        e = torch.as_tensor(expected).double().flatten()
        if a.numel() != e.numel():
            return ValidationReport(False, float("inf"), float("inf"), a.numel(), a.numel(), False)
        tol = self.config.for_dtype(dtype)
        has_nan = bool(torch.isnan(a).any())
        diff = (a - e).abs()
        bad = diff > (tol.atol + tol.rtol * e.abs())
        nbad = int(bad.sum())
        total = a.numel()
        allowed = 0 if self.config.strict else int(total * self.config.max_violation_fraction)
        rel = diff / e.abs().clamp_min(1e-30)
        return ValidationReport((nbad <= allowed) and not has_nan, float(diff.max()) if total else 0.0,
                                float(rel.max()) if total else 0.0, nbad, total, has_nan)


class OpFamily(enum.Enum):
    ELEMENTWISE = "elementwise"
    MATMUL = "matmul"
    REDUCTION = "reduction"
    SOFTMAX = "softmax"
    LAYERNORM = "layernorm"
    ATTENTION = "attention"
    LOSS = "loss"


class ToleranceConfig:
    """Per-op-family tolerances per backend (crates/core/src/tolerance.rs:40; tests/common/numeric.rs:20-40).
    The bf16 column is what the B200 kernels are held to against the fp32 oracle."""
    F32 = {OpFamily.ELEMENTWISE: Tolerance(1e-5, 1e-6), OpFamily.MATMUL: Tolerance(1e-4, 1e-5),
           OpFamily.REDUCTION: Tolerance(1e-4, 1e-5), OpFamily.SOFTMAX: Tolerance(1e-5, 1e-6),
           OpFamily.LAYERNORM: Tolerance(1e-4, 1e-5), OpFamily.ATTENTION: Tolerance(1e-4, 1e-5),
           OpFamily.LOSS: Tolerance(1e-5, 1e-6)}
    BF16 = {OpFamily.ELEMENTWISE: Tolerance(1e-2, 1e-2), OpFamily.MATMUL: Tolerance(2e-2, 2e-2),
            OpFamily.REDUCTION: Tolerance(1e-2, 1e-2), OpFamily.SOFTMAX: Tolerance(1e-2, 1e-3),
            OpFamily.LAYERNORM: Tolerance(2e-2, 2e-2), OpFamily.ATTENTION: Tolerance(3e-2, 3e-2),
            OpFamily.LOSS: Tolerance(1e-3, 1e-3)}

    @classmethod
    def for_family(cls, family: OpFamily, dtype: DType = DType.F32) -> Tolerance:
        return (cls.BF16 if dtype in (DType.BF16, DType.F16) else cls.F32)[family]


def assert_close(actual, expected, tol: Tolerance | None = None, what: str = "") -> None:
    tol = tol or Tolerance(1e-5, 1e-8)
    a = torch.as_tensor(actual).double()
    e = torch.as_tensor(expected).double()
    if a.shape != e.shape:
        raise AssertionError(f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}")
    bad = (a - e).abs() > (tol.atol + tol.rtol * e.abs())
    if bool(bad.any()):
        i = int(bad.flatten().nonzero()[0])
        raise AssertionError(f"{what}: {int(bad.sum())} of {a.numel()} elements differ; first at flat index {i}: "
                             f"{float(a.flatten()[i])} vs {float(e.flatten()[i])}")


assert_slices_close = assert_close
