"""Weight quantization: INT8 (per-tensor / per-channel / asymmetric), INT4 group-wise, FP8 formats, fake-quant for QAT
(crates/nn/src/quantization.rs:27-560).  Weights are stored quantized (the reference dequantizes to f32 and calls a
plain matmul).  Forward pass on CUDA tensors:

* FP8 (e4m3 / e5m2 weights, one scale per output channel): the tokens are quantised to e4m3 with one scale per row by
  `rb_quantize_fp8_rows`, the product runs on `tcgen05.mma kind::f8f6f4` and the scales and the bias are applied in the
  GEMM epilogue (`ops.quant.gemm_fp8`).
* INT8: `rb_dequant_int8_bf16` expands `q - zero_point` to bf16 (exact), the bf16 tensor-core GEMM multiplies the scale
  back in its epilogue (per tensor: alpha; per channel: column scales).
* INT4 groups: `rb_dequant_int4_bf16` expands to bf16, then the bf16 GEMM.

CPU tensors compute the same quantities in fp32."""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, InvalidArgument


class QuantizationScheme(enum.Enum):
    INT8 = "int8"
    INT8_ASYMMETRIC = "int8_asymmetric"
    INT8_PER_CHANNEL = "int8_per_channel"
    INT4 = "int4"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"

    @property
    def bits(self) -> int:
        return 4 if self is QuantizationScheme.INT4 else 8

    @property
    def compression_ratio(self) -> float:
        return 32.0 / self.bits


@dataclass
class QuantConfig:
    scheme: QuantizationScheme = QuantizationScheme.INT8
    group_size: int = 128
    symmetric: bool = True
    per_channel: bool = False
    outlier_threshold: float = 0.0


@dataclass
class QuantParams:
    scale: torch.Tensor
    zero_point: torch.Tensor

    @classmethod
    def from_tensor(cls, t: torch.Tensor, symmetric: bool = True, dim: int | None = None) -> "QuantParams":
        f = t.detach().float()
        if symmetric:
            amax = f.abs().amax() if dim is None else f.abs().amax(dim, keepdim=True)
            scale = (amax / 127.0).clamp_min(1e-12)
            return cls(scale, torch.zeros_like(scale))
        lo = f.amin() if dim is None else f.amin(dim, keepdim=True)
        hi = f.amax() if dim is None else f.amax(dim, keepdim=True)
        scale = ((hi - lo) / 255.0).clamp_min(1e-12)
        zp = torch.round(-lo / scale) - 128
        return cls(scale, zp)

    def quantize(self, t: torch.Tensor) -> torch.Tensor:
        q = torch.round(t.float() / self.scale) + self.zero_point
        return q.clamp(-128, 127).to(torch.int8)

    def dequantize(self, q: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
        return ((q.float() - self.zero_point) * self.scale).to(dtype)


class QuantizedLinear(Module):
    """8-bit weights [out, in]: int8 with a per-tensor or per-output-channel scale (and zero point), or e4m3 / e5m2 bytes
    with one scale per output channel."""

    def __init__(self, qweight, params: QuantParams, bias=None, compute_dtype=torch.float32,
                 scheme: QuantizationScheme = QuantizationScheme.INT8):
        self.qweight, self.params, self.bias, self.compute_dtype, self.scheme = qweight, params, bias, compute_dtype, scheme

    @classmethod
    def from_linear(cls, linear, scheme: QuantizationScheme = QuantizationScheme.INT8):
        w = linear.weight.tensor.detach()
        bias = None if linear.bias is None else linear.bias.tensor.detach()
        if scheme in (QuantizationScheme.FP8_E4M3, QuantizationScheme.FP8_E5M2):
            f = w.float()
            fmax, fdt = (448.0, torch.float8_e4m3fn) if scheme is QuantizationScheme.FP8_E4M3 else (57344.0, torch.float8_e5m2)
            amax = f.abs().amax(1)
            scale = torch.where(amax > 0, amax / fmax, torch.ones_like(amax))
            q = (f / scale[:, None]).clamp(-fmax, fmax).to(fdt).view(torch.uint8)
            return cls(q, QuantParams(scale.contiguous(), torch.zeros_like(scale)), bias, w.dtype, scheme)
        per_ch = scheme is QuantizationScheme.INT8_PER_CHANNEL
        p = QuantParams.from_tensor(w, symmetric=scheme is not QuantizationScheme.INT8_ASYMMETRIC, dim=1 if per_ch else None)
        return cls(p.quantize(w), p, bias, w.dtype, scheme)

    @property
    def is_fp8(self) -> bool:
        return self.scheme in (QuantizationScheme.FP8_E4M3, QuantizationScheme.FP8_E5M2)

    def stored_bytes(self) -> int:
        """Bytes of the quantised weight as stored: payload, scales, zero points (the bias is not part of it)."""
        return sum(t.numel() * t.element_size() for t in (self.qweight, self.params.scale, self.params.zero_point))

    def dequantized_weight(self):
        if self.is_fp8:
            fdt = torch.float8_e4m3fn if self.scheme is QuantizationScheme.FP8_E4M3 else torch.float8_e5m2
            return (self.qweight.view(fdt).float() * self.params.scale[:, None]).to(self.compute_dtype)
        return self.params.dequantize(self.qweight, self.compute_dtype)

    def forward(self, x, ctx: ForwardCtx | None = None):
        from ..ops import quant as Q
        x2 = x.reshape(-1, x.shape[-1])
        out_f = self.qweight.shape[0]
        if self.is_fp8:
            # tokens -> e4m3 with one scale per row; product on the 8-bit tensor-core path
            a8, a_scale = Q.quantize_fp8_rows(x2)
            bias = None if self.bias is None else (self.bias.to(torch.bfloat16) if x.is_cuda else self.bias)
            y = Q.gemm_fp8(a8, a_scale, self.qweight, self.params.scale, bias=bias,
                           out_dtype=torch.bfloat16 if x.is_cuda else x.dtype, b_e5m2=self.scheme is QuantizationScheme.FP8_E5M2)
            return y.to(x.dtype).reshape(*x.shape[:-1], out_f)
        if x.is_cuda and not self.is_fp8 and self.qweight.shape[1] % 16 == 0:
            zp = self.params.zero_point
            wq = Q.dequant_int8(self.qweight, None if not bool((zp != 0).any()) else zp)       # q - z in bf16, exact
            scale = self.params.scale.reshape(-1).float()
            xb = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
            bias = None if self.bias is None else self.bias.to(torch.bfloat16)
            if scale.numel() == 1:
                y = ops.gemm(xb.contiguous(), wq, bias=bias, alpha=float(scale))
            else:
                y = ops.gemm(xb.contiguous(), wq, bias=bias, col_scale=scale.contiguous())
            return y.to(x.dtype).reshape(*x.shape[:-1], out_f)
        return ops.linear(x, self.dequantized_weight().contiguous(), self.bias)

    def memory_bytes(self) -> int:
        return self.qweight.numel() + self.params.scale.numel() * 4


class GPTQLinear(Module):
    """int4 group-wise quantization: scale = absmax / 7 per group of `group_size` input features, zero point 8, two
    nibbles per byte.  (Round-to-nearest; no Hessian-based error compensation, as in the reference.)"""

    def __init__(self, packed, scales, shape, group_size: int, bias=None, compute_dtype=torch.float32):
        self.packed, self.scales, self.shape, self.group_size = packed, scales, tuple(shape), group_size
        self.bias, self.compute_dtype = bias, compute_dtype

    @classmethod
    def from_linear(cls, linear, group_size: int = 128):
        w = linear.weight.tensor.detach().float()
        out, inn = w.shape
        if inn % group_size or inn % 2:
            raise InvalidArgument("in_features must be a multiple of the group size and even")
        g = w.view(out, inn // group_size, group_size)
        scales = (g.abs().amax(-1, keepdim=True) / 7.0).clamp_min(1e-12)
        q = (torch.round(g / scales) + 8).clamp(0, 15).to(torch.uint8).view(out, inn)
        packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
        return cls(packed, scales.squeeze(-1), (out, inn), group_size,
                   None if linear.bias is None else linear.bias.tensor.detach(), linear.weight.tensor.dtype)

    def stored_bytes(self) -> int:
        return self.packed.numel() * self.packed.element_size() + self.scales.numel() * self.scales.element_size()

    def dequantized_weight(self):
        out, inn = self.shape
        q = torch.empty((out, inn), dtype=torch.uint8, device=self.packed.device)
        q[:, 0::2] = self.packed & 0xF
        q[:, 1::2] = self.packed >> 4
        g = (q.float() - 8.0).view(out, inn // self.group_size, self.group_size) * self.scales.unsqueeze(-1)
        return g.view(out, inn).to(self.compute_dtype)

    def forward(self, x, ctx: ForwardCtx | None = None):
        if x.is_cuda and self.shape[1] % 32 == 0 and self.group_size % 32 == 0:
            from ..ops import quant as Q
            w = Q.dequant_int4(self.packed, self.scales, self.group_size)                        # bf16, one kernel
            x2 = x.reshape(-1, x.shape[-1])
            xb = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
            bias = None if self.bias is None else self.bias.to(torch.bfloat16)
            y = ops.gemm(xb.contiguous(), w, bias=bias)
            return y.to(x.dtype).reshape(*x.shape[:-1], self.shape[0])
        return ops.linear(x, self.dequantized_weight().contiguous(), self.bias)

    def memory_bytes(self) -> int:
        return self.packed.numel() + self.scales.numel() * 4


class DynamicQuantizer:
    """Quantizes activations on the fly (per tensor, symmetric) and reports the error."""

    def quantize(self, t: torch.Tensor):
        p = QuantParams.from_tensor(t)
        return p.quantize(t), p

    def roundtrip_error(self, t: torch.Tensor) -> float:
        q, p = self.quantize(t)
        return float((p.dequantize(q) - t.float()).abs().max())


class QATTrainer:
    """Fake quantization with a straight-through estimator for quantization-aware training."""

    @staticmethod
    def fake_quantize(t: torch.Tensor, num_bits: int = 8) -> torch.Tensor:
        qmax = 2 ** (num_bits - 1) - 1
        scale = (t.detach().abs().amax() / qmax).clamp_min(1e-12)
        q = torch.clamp(torch.round(t / scale), -qmax - 1, qmax) * scale
        return t + (q - t).detach()


@dataclass
class QuantizationStats:
    """Size of a model's linear weights before and after quantisation (crates/nn/src/quantization.rs:499-506)."""
    original_size_mb: float
    quantized_size_mb: float
    compression_ratio: float
    layers_quantized: int
    scheme: QuantizationScheme


def quantize_model_with_stats(model, scheme: QuantizationScheme = QuantizationScheme.INT8, group_size: int = 128) -> QuantizationStats:
    """`quantize_model` plus the accounting: fp32 bytes of every replaced weight against the stored bytes of its
    quantised form (payload, scales and zero points)."""
    from .linear import Linear
    before = {}

    def walk(m):
        for v in vars(m).values():
            for e in (v if isinstance(v, list) else [v]):
                if isinstance(e, Linear):
                    before[id(e)] = e.weight.tensor.numel() * 4
                elif hasattr(e, "__dict__") and hasattr(e, "named_parameters"):
                    walk(e)
    walk(model)
    n = quantize_model(model, scheme, group_size)
    after = 0

    def walk_q(m):
        nonlocal after
        for v in vars(m).values():
            for e in (v if isinstance(v, list) else [v]):
                if isinstance(e, (QuantizedLinear, GPTQLinear)):
                    after += e.stored_bytes()
                elif hasattr(e, "__dict__") and hasattr(e, "named_parameters"):
                    walk_q(e)
    walk_q(model)
    orig = sum(before.values())
    return QuantizationStats(orig / 2 ** 20, after / 2 ** 20, orig / after if after else 0.0, n, scheme)


def quantize_model(model, scheme: QuantizationScheme = QuantizationScheme.INT8, group_size: int = 128):
    """Replaces every Linear attribute (recursively, lists included) by its quantized counterpart; returns the count."""
    from .linear import Linear
    n = 0
    for k, v in list(vars(model).items()):
        if isinstance(v, Linear):
            setattr(model, k, GPTQLinear.from_linear(v, group_size) if scheme is QuantizationScheme.INT4
                    else QuantizedLinear.from_linear(v, scheme))
            n += 1
        elif isinstance(v, list):
            for i, e in enumerate(v):
                if isinstance(e, Linear):
                    v[i] = GPTQLinear.from_linear(e, group_size) if scheme is QuantizationScheme.INT4 else QuantizedLinear.from_linear(e, scheme)
                    n += 1
                elif hasattr(e, "__dict__"):
                    n += quantize_model(e, scheme, group_size)
        elif hasattr(v, "__dict__") and not isinstance(v, (torch.Tensor, type)) and hasattr(v, "named_parameters"):
            n += quantize_model(v, scheme, group_size)
    return n
