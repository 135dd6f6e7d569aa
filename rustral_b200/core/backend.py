"""Backends: the CPU reference backend and the B200 backend (crates/core/src/backend.rs:5-205).

A backend is a device plus a default dtype, a capability record and the op tables.  There are exactly two:
``CpuBackend`` (fp32, the numerical oracle) and ``B200Backend`` (bf16 parameters and
activations with fp32 accumulation, served only by the sm_100a kernels).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

import torch

from .parameter import Parameter


class OperationType(enum.Enum):
    MATMUL = "matmul"
    CONVOLUTION = "convolution"
    ATTENTION = "attention"
    NORMALIZATION = "normalization"
    ELEMENTWISE = "elementwise"
    REDUCTION = "reduction"
    SOFTMAX = "softmax"
    LOSS = "loss"


class ConvLayout(enum.Enum):
    NCHW = "nchw"
    NHWC = "nhwc"


class TrainingDtype(enum.Enum):
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"

    def torch(self):
        return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[self.value]


@dataclass
class BackendCapabilities:
    """What a backend can do and how to size work for it (14 fields, crates/core/src/backend.rs:5-34)."""
    supports_fp16: bool = False
    supports_bf16: bool = False
    supports_int8: bool = True
    supports_fused_ops: bool = True
    supports_flash_attention: bool = False
    supports_in_place: bool = True
    supports_cuda_graphs: bool = False
    supports_tensor_cores: bool = False
    max_batch_size: int = 32
    optimal_chunk_size: int = 4096
    memory_bytes: int = 0
    num_compute_units: int = 1
    preferred_conv_layout: ConvLayout = ConvLayout.NCHW
    recommended_training_dtype: TrainingDtype = TrainingDtype.F32

    def clamp_batch_size(self, requested: int) -> int:
        return max(1, min(int(requested), self.max_batch_size))

    def recommends_mixed_precision(self) -> bool:
        return self.supports_tensor_cores and (self.supports_bf16 or self.supports_fp16)

    def recommended_dtype_for_operation(self, op: OperationType) -> TrainingDtype:
        # reductions, normalisation statistics, softmax and losses stay in fp32 even under mixed precision
        if op in (OperationType.REDUCTION, OperationType.NORMALIZATION, OperationType.SOFTMAX, OperationType.LOSS):
            return TrainingDtype.F32
        return self.recommended_training_dtype


class Backend:
    """Device + dtype + op tables."""

    name = "abstract"

    def __init__(self, device: torch.device, dtype: torch.dtype):
        self._device = torch.device(device)
        self.dtype = dtype
        from .tensor_ops import TensorOps, FusionOps, AttentionOps, QuantizationOps
        self._ops = TensorOps(self)
        self._fusion = FusionOps(self)
        self._attention = AttentionOps(self)
        self._quant = QuantizationOps(self)

    def device(self) -> torch.device:
        return self._device

    def ops(self):
        return self._ops

    def fusion_ops(self):
        return self._fusion

    def attention_ops(self):
        return self._attention

    def quantization_ops(self):
        return self._quant

    def capabilities(self) -> BackendCapabilities:
        raise NotImplementedError

    # ---- parameter construction ---------------------------------------------------------------------
    def _gen(self, seed: int) -> torch.Generator:
        return torch.Generator(device="cpu").manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)

    def normal_parameter(self, name: str, shape, seed: int, scale: float) -> Parameter:
        """N(0, scale) samples drawn on the host from `seed`, so a model initialises identically on both
        backends.  scale <= 0 gives zeros.  (The reference's function of this name samples a uniform
        distribution, crates/ndarray-backend/src/lib.rs:132-146; the normal law is what its callers document.)"""
        if scale <= 0:
            t = torch.zeros(tuple(shape), dtype=torch.float32)
        else:
            t = torch.randn(tuple(shape), generator=self._gen(seed), dtype=torch.float32) * scale
        return Parameter(name, t.to(device=self._device, dtype=self.dtype))

    def uniform_parameter(self, name: str, shape, seed: int, scale: float) -> Parameter:
        """Uniform(-scale, scale) samples."""
        t = (torch.rand(tuple(shape), generator=self._gen(seed), dtype=torch.float32) * 2 - 1) * scale
        return Parameter(name, t.to(device=self._device, dtype=self.dtype))

    def constant_parameter(self, name: str, shape, value: float) -> Parameter:
        return Parameter(name, torch.full(tuple(shape), float(value), dtype=self.dtype, device=self._device))

    def parameter_from_vec(self, name: str, values, shape) -> Parameter:
        t = torch.as_tensor(values, dtype=torch.float32).reshape(tuple(shape))
        return Parameter(name, t.to(device=self._device, dtype=self.dtype))

    def tensor(self, values, shape=None, dtype=None) -> torch.Tensor:
        t = torch.as_tensor(values, dtype=torch.float32)
        if shape is not None:
            t = t.reshape(tuple(shape))
        return t.to(device=self._device, dtype=dtype or self.dtype)

    def __repr__(self):
        return f"{type(self).__name__}(device={self._device}, dtype={self.dtype})"


class CpuBackend(Backend):
    """fp32 reference backend: the oracle every kernel is checked against."""

    name = "cpu"

    def __init__(self, dtype: torch.dtype = torch.float32):
        super().__init__(torch.device("cpu"), dtype)

    def capabilities(self) -> BackendCapabilities:
        import os
        return BackendCapabilities(supports_fp16=False, supports_bf16=True, max_batch_size=32, optimal_chunk_size=4096,
                                   num_compute_units=os.cpu_count() or 1,
                                   recommended_training_dtype=TrainingDtype.F32)


class B200Backend(Backend):
    """sm_100a backend: bf16 storage, fp32 accumulation, tcgen05 GEMMs, flash attention, CUDA graphs."""

    name = "b200"

    def __init__(self, device=None, dtype: torch.dtype = torch.bfloat16):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        super().__init__(torch.device(device), dtype)
        from .. import _native
        _native.kernels()   # fail here, loudly, when the kernel library is missing

    def capabilities(self) -> BackendCapabilities:
        props = torch.cuda.get_device_properties(self._device)
        return BackendCapabilities(supports_fp16=False, supports_bf16=True, supports_flash_attention=True,
                                   supports_cuda_graphs=True, supports_tensor_cores=True, max_batch_size=4096,
                                   optimal_chunk_size=1 << 20, memory_bytes=props.total_memory,
                                   num_compute_units=props.multi_processor_count,
                                   preferred_conv_layout=ConvLayout.NHWC,
                                   recommended_training_dtype=TrainingDtype.BF16)


_default = None


def default_backend() -> Backend:
    """B200 when a CUDA device is visible, else the CPU reference backend."""
    global _default
    if _default is None:
        _default = B200Backend() if torch.cuda.is_available() else CpuBackend()
    return _default


def set_default_backend(b: Backend) -> None:
    global _default
    _default = b
