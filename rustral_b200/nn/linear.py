"""Dense layers: y = x W^T + b with W stored [out, in] (crates/nn/src/linear.rs:9-320)."""
from __future__ import annotations

from dataclasses import dataclass

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, ShapeMismatch, InvalidArgument


@dataclass
class LinearConfig:
    in_dim: int
    out_dim: int
    bias: bool = False


class Linear(Module, Trainable, Saveable):
    """Parameter names: ``weight`` [out, in], ``bias`` [out]."""

    activation = "none"

    def __init__(self, config: LinearConfig, weight: Parameter, bias: Parameter | None = None):
        if weight.shape != (config.out_dim, config.in_dim):
            raise ShapeMismatch((config.out_dim, config.in_dim), weight.shape, "Linear.weight")
        if config.bias and bias is None:
            raise InvalidArgument("LinearConfig.bias is set but no bias parameter was given")
        self.config = config
        self.weight = weight
        self.bias = bias

    @classmethod
    def new(cls, backend, in_dim: int, out_dim: int, bias: bool = True, seed: int = 42, scale: float = 0.1):
        return LinearBuilder(in_dim, out_dim).with_bias(bias).seed(seed).scale(scale).build(backend)

    def forward(self, x, ctx: ForwardCtx, residual=None):
        if x.shape[-1] != self.config.in_dim:
            raise ShapeMismatch((self.config.in_dim,), x.shape[-1:], "Linear input")
        with ctx.profile("linear" if self.activation == "none" else f"linear_{self.activation}", x.shape):
            return ops.linear(x, self.weight.tensor, None if self.bias is None else self.bias.tensor,
                              self.activation, residual)

    def __call__(self, x, ctx=None, residual=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), residual)

    def _children(self):
        yield "weight", self.weight
        if self.bias is not None:
            yield "bias", self.bias


class LinearBuilder:
    """``LinearBuilder(in, out).with_bias().seed(42).scale(0.1).build(backend)``; the bias draws from seed + 1."""

    def __init__(self, in_dim: int, out_dim: int):
        if in_dim <= 0 or out_dim <= 0:
            raise InvalidArgument("Linear dimensions must be positive")
        self._in, self._out = in_dim, out_dim
        self._bias = False
        self._seed = 42
        self._scale = 0.1
        self._zero_bias = False
        self._cls = Linear

    def with_bias(self, bias: bool = True):
        self._bias = bias
        return self

    def seed(self, seed: int):
        self._seed = seed
        return self

    def scale(self, scale: float):
        self._scale = scale
        return self

    def zero_bias(self, flag: bool = True):
        """Initialise the bias to zeros instead of sampling it (what GPT-style models use)."""
        self._zero_bias = flag
        return self

    def activation(self, name: str):
        self._cls = {"none": Linear, "relu": LinearReLU, "gelu": LinearGELU, "silu": LinearSiLU}[name]
        return self

    def build(self, backend):
        w = backend.normal_parameter("weight", (self._out, self._in), self._seed, self._scale)
        b = None
        if self._bias:
            b = backend.normal_parameter("bias", (self._out,), self._seed + 1, 0.0 if self._zero_bias else self._scale)
        return self._cls(LinearConfig(self._in, self._out, self._bias), w, b)


class LinearReLU(Linear):
    """Linear + bias + ReLU in one GEMM epilogue (crates/nn/src/linear.rs:211)."""
    activation = "relu"

    def __init__(self, config, weight, bias=None):
        if bias is None:
            raise InvalidArgument("LinearReLU requires a bias")
        super().__init__(config, weight, bias)


class LinearGELU(LinearReLU):
    """Linear + bias + tanh-GELU in one GEMM epilogue (crates/nn/src/linear.rs:289)."""
    activation = "gelu"


class LinearSiLU(LinearReLU):
    activation = "silu"


class FusionHelper:
    """try-fused-then-fallback entry points kept for API parity (crates/nn/src/fusion_helper.rs:9-60); the fused
    GEMM epilogue always exists here, so there is no fallback branch."""

    @staticmethod
    def try_linear_bias(x, w, b, ctx=None):
        return ops.linear(x, w, b, "none")

    @staticmethod
    def try_linear_relu(x, w, b, ctx=None):
        return ops.linear(x, w, b, "relu")

    @staticmethod
    def try_linear_gelu(x, w, b, ctx=None):
        return ops.linear(x, w, b, "gelu")
