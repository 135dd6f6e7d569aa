"""Core contracts: backends, ForwardCtx, Module traits, parameters, shapes, errors, profilers, pools, numerics."""
from .errors import CoreError, ShapeMismatch, InvalidShape, InvalidArgument, BackendError, SerializationError
from .shape import Shape, ShapePolicy
from .parameter import Parameter, ParameterId, ParameterRef, ParameterGroup
from .context import ForwardCtx, Mode, RunId
from .module import (Module, NamedParameters, Trainable, StatefulModule, Saveable, collect_named_parameters,
                     collect_named_parameter_ids)
from .backend import (Backend, CpuBackend, B200Backend, BackendCapabilities, OperationType, ConvLayout, TrainingDtype,
                      default_backend, set_default_backend)
from .tensor_ops import TensorOps, TensorInPlaceOps, FusionOps, AttentionOps, QuantizationOps

__all__ = [n for n in dir() if not n.startswith("_")]
