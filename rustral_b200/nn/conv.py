"""Conv2d and pooling (crates/nn/src/conv.rs:7-340).  NCHW input, any number of input channels (the reference assumes
one, conv.rs:47-57).  Two paths: small filter banks in inference run the direct kernel of csrc/kernels/conv.cu (one
launch: taps, bias and the NCHW store); everything else, and every call that needs gradients, is lowered to one GEMM
on the unfolded patches (im2col), which on the B200 backend is the tcgen05 kernel."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import _native as N_
from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, ShapeMismatch


N_.optional_sig("rb_conv2d_fwd", [N_.c_void_p, N_.c_void_p, N_.c_void_p, N_.c_void_p] + [N_.c_int] * 10 + [N_.c_void_p])
DIRECT_MAX_FILTER_ELEMS = 12288          # the direct kernel keeps the filter bank in 48 KB of shared memory as fp32


def _conv2d_direct(x, weight, bias, stride: int, pad) -> torch.Tensor:
    """Inference-only direct convolution (no autograd graph): bf16 NCHW in, bf16 NCHW out."""
    N, C, H, W = x.shape
    O, _, kh, kw = weight.shape
    ho, wo = (H + 2 * pad[0] - kh) // stride + 1, (W + 2 * pad[1] - kw) // stride + 1
    x = x.detach().contiguous()
    wt = weight.detach().to(torch.bfloat16).contiguous()
    b = None if bias is None else bias.detach().to(torch.bfloat16).contiguous()
    y = torch.empty((N, O, ho, wo), dtype=torch.bfloat16, device=x.device)
    N_.check(N_.kernels().rb_conv2d_fwd(x.data_ptr(), wt.data_ptr(), N_.ptr(b), y.data_ptr(), N, C, H, W, O, kh, kw, stride,
                                        pad[0], pad[1], N_.stream_ptr()), "rb_conv2d_fwd")
    return y


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
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or (ctx is not None and ctx.is_training()))
        if (x.is_cuda and x.dtype == torch.bfloat16 and not needs_grad
                and c.out_channels * C * c.kernel_h * c.kernel_w <= DIRECT_MAX_FILTER_ELEMS):
            return _conv2d_direct(x, self.weight.tensor, None if self.bias is None else self.bias.tensor, c.stride, pad)
        cols = F.unfold(x.float(), (c.kernel_h, c.kernel_w), padding=pad, stride=c.stride)       # [N, C*kh*kw, L]
        L = cols.shape[-1]
        a = cols.transpose(1, 2).reshape(N * L, -1).to(x.dtype).contiguous()
        k = a.shape[1]
        wmat = self.weight.tensor.reshape(c.out_channels, k)
        if x.is_cuda and k % 8:            # TMA needs 16-byte row pitches: pad the contraction dimension with zeros
            padk = (-k) % 8
            a = F.pad(a, (0, padk))
            wmat = F.pad(wmat, (0, padk))
        bvec = None if self.bias is None else self.bias.tensor
        if x.is_cuda and c.out_channels % 8:   # the GEMM's output rows need a 16-byte pitch too: pad the filters with zeros
            pado = (-c.out_channels) % 8
            wmat = F.pad(wmat, (0, 0, 0, pado))
            bvec = None if bvec is None else F.pad(bvec, (0, pado))
        y = ops.linear(a, wmat.contiguous(), bvec)
        if y.shape[1] != c.out_channels:
            y = y[:, :c.out_channels]
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
