"""Core contracts: backends, ForwardCtx, Module traits, parameters, shapes, errors, profilers, pools, numerics."""
from .errors import CoreError, ShapeMismatch, InvalidShape, InvalidArgument, BackendError, SerializationError
from .shape import Shape, ShapePolicy, ShapeExt, TensorShape
from .parameter import Parameter, ParameterId, ParameterRef, ParameterGroup
from .context import ForwardCtx, Mode, RunId
from .module import (Module, NamedParameters, Trainable, StatefulModule, Saveable, collect_named_parameters,
                     collect_named_parameter_ids)
from .backend import (Backend, CpuBackend, B200Backend, BackendCapabilities, OperationType, ConvLayout, TrainingDtype,
                      default_backend, set_default_backend)
from .tensor_ops import TensorOps, TensorInPlaceOps, TensorView, FusionOps, AttentionOps, QuantizationOps
from .operation_profiler import (OperationProfiler, OperationStats, OperationGuard, ProfilerSnapshot, DeviceType,
                                 shape_bucket, operation_profiler_from_env, finish_profile_from_env, MatmulDim, ShapeBucket,
                                 ProfilingHooks, SnapshotOp)
from .memory_profiler import (MemoryProfiler, AllocationTracker, OOMRisk, OomRisk, MemorySnapshot, MemorySummary,
                              global_profiler, track_tensor)
from .tensor_pool import TensorPool, PoolStrategy, PooledTensor, PoolStats, pool_from_env
from .numerics import (DType, Tolerance, NumericsConfig, NumericsValidator, OpFamily, ToleranceConfig, assert_close,
                       assert_slices_close, ValidationResult, NumericsError)
from .fusion import (FusionPattern, PatternMatcher, FusionOptimizer, FusionTestHarness, FusionTestConfig,
                     FusionTestSuiteResult, OpType, Op, generate_random_data)

PARALLEL_REDUCTIONS_ENV = "RUSTRAL_PARALLEL_REDUCTIONS"
PAR_REDUCE_ENV = "RUSTRAL_PAR_REDUCE"


def parallel_reductions_enabled() -> bool:
    """True when RUSTRAL_PARALLEL_REDUCTIONS or its short form RUSTRAL_PAR_REDUCE is "1" (crates/core/src/lib.rs:8-23).
    It concerns the CPU reference path only: by default its whole-tensor and column sums accumulate in float64, so the
    fp32 result does not depend on how many threads split the work; with the switch on they are plain fp32 sums, faster
    and subject to the association order of the thread count in use.  GPU reductions have a fixed order either way."""
    import os
    return os.environ.get(PARALLEL_REDUCTIONS_ENV) == "1" or os.environ.get(PAR_REDUCE_ENV) == "1"


__all__ = [n for n in dir() if not n.startswith("_")]
