"""Conv2d and pooling (crates/nn/src/conv.rs:7-340).  NCHW input; the convolution is lowered to one GEMM on the
unfolded patches (im2col), so on the B200 backend it runs on the tcgen05 kernel; any number of input channels
(the reference assumes one, conv.rs:47-57)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, ShapeMismatch


@dataclass
class Conv2dConfig:
    out_channels: int
    kernel_h: int
    kernel_w: int
    stride: int = 1
    bias: bool = True
    no_padding: bool = False
    in_channels: int = 1


class Conv2d(Module, Trainable, Saveable):
    """Parameters: weight [O, C, kh, kw], bias [O].  "Same"-style zero padding of k // 2 unless `no_padding`."""

    def __init__(self, config: Conv2dConfig, weight: Parameter, bias: Parameter | None):
        self.config, self.weight, self.bias = config, weight, bias

    @classmethod
    def new(cls, backend, config: Conv2dConfig, seed: int = 42):
        c = config
        fan_in = c.in_channels * c.kernel_h * c.kernel_w
        w = backend.normal_parameter("weight", (c.out_channels, c.in_channels, c.kernel_h, c.kernel_w), seed, fan_in ** -0.5)
        b = backend.constant_parameter("bias", (c.out_channels,), 0.0) if c.bias else None
        return cls(c, w, b)

    def forward(self, x, ctx: ForwardCtx | None = None):
        c = self.config
        if x.dim() != 4 or x.shape[1] != c.in_channels:
            raise ShapeMismatch(("N", c.in_channels, "H", "W"), x.shape, "Conv2d input")
        pad = (0, 0) if c.no_padding else (c.kernel_h // 2, c.kernel_w // 2)
        N, C, H, W = x.shape
        cols = F.unfold(x.float(), (c.kernel_h, c.kernel_w), padding=pad, stride=c.stride)       # [N, C*kh*kw, L]
        L = cols.shape[-1]
        a = cols.transpose(1, 2).reshape(N * L, -1).to(x.dtype).contiguous()
        k = a.shape[1]
        wmat = self.weight.tensor.reshape(c.out_channels, k)
        if x.is_cuda and k % 8:            # TMA needs 16-byte row pitches: pad the contraction dimension with zeros
            padk = (-k) % 8
            a = F.pad(a, (0, padk))
            wmat = F.pad(wmat, (0, padk))
        y = ops.linear(a, wmat.contiguous(), None if self.bias is None else self.bias.tensor)
        ho = (H + 2 * pad[0] - c.kernel_h) // c.stride + 1
        wo = (W + 2 * pad[1] - c.kernel_w) // c.stride + 1
        return y.reshape(N, ho, wo, c.out_channels).permute(0, 3, 1, 2).contiguous()

    def _children(self):
        yield "weight", self.weight
        if self.bias is not None:
            yield "bias", self.bias


def max_pool2d(x: torch.Tensor, kernel: int = 2, stride: int | None = None) -> torch.Tensor:
    return F.max_pool2d(x, kernel, stride or kernel)


def global_max_pool2d(x: torch.Tensor) -> torch.Tensor:
    return x.amax((2, 3))
