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

__all__ = [n for n in dir() if not n.startswith("_")]
