"""Conv2d and pooling (crates/nn/src/conv.rs:7-340).  NCHW input, any number of input channels (the reference assumes
one, conv.rs:47-57).  Two paths: small filter banks in inference run the direct kernel of csrc/kernels/conv.cu (one
launch: taps, bias and the NCHW store); everything else, and every call that needs gradients, is lowered to one GEMM
on the unfolded patches (im2col), which on the B200 backend is the tcgen05 kernel with native unfolding, folding and
layout kernels around it, forward and backward (`_Conv2dGemmFn`); CPU tensors use `F.unfold` and the reference GEMM."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import _native as N_
from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, ShapeMismatch


N_.optional_sig("rb_conv2d_fwd", [N_.c_void_p, N_.c_void_p, N_.c_void_p, N_.c_void_p] + [N_.c_int] * 10 + [N_.c_void_p])
_P, _I = N_.c_void_p, N_.c_int
N_.optional_sig("rb_im2col", [_P, _P] + [_I] * 10 + [_P])
N_.optional_sig("rb_col2im", [_P, _P] + [_I] * 10 + [_P])
N_.optional_sig("rb_nhwc_to_nchw", [_P, N_.c_ll, _P, _I, _I, _I, _P])
N_.optional_sig("rb_nchw_to_nhwc", [_P, _P, _I, _I, _I, _I, _P])
DIRECT_MAX_FILTER_ELEMS = 12288          # the direct kernel keeps the filter bank in 48 KB of shared memory as fp32


class _Conv2dGemmFn(torch.autograd.Function):
    """Convolution of bf16 CUDA tensors as one tcgen05 GEMM over unfolded patches, forward and backward, with native
    kernels for the unfolding (`rb_im2col`), its adjoint (`rb_col2im`) and the NHWC <-> NCHW copies around the GEMMs
    (csrc/kernels/conv.cu).  Backward: dW = dY^T cols, db = column sums of dY, dcols = dY W, dx = col2im(dcols)."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, pad):
        N, C, H, W = x.shape
        O, _, kh, kw = weight.shape
        ho, wo = (H + 2 * pad[0] - kh) // stride + 1, (W + 2 * pad[1] - kw) // stride + 1
        L, K = ho * wo, C * kh * kw
        Kp, Op = (K + 7) // 8 * 8, (O + 7) // 8 * 8            # 16-byte row pitches for the GEMM's operands and output
        lib = N_.kernels()
        x = x.contiguous()
        cols = torch.empty((N * L, Kp), dtype=torch.bfloat16, device=x.device)
        N_.check(lib.rb_im2col(x.data_ptr(), cols.data_ptr(), N, C, H, W, kh, kw, stride, pad[0], pad[1], Kp, N_.stream_ptr()), "rb_im2col")
        wmat = torch.zeros((Op, Kp), dtype=torch.bfloat16, device=x.device)
        wmat[:O, :K] = weight.detach().reshape(O, K)
        bvec = None
        if bias is not None:
            bvec = torch.zeros(Op, dtype=torch.bfloat16, device=x.device)
            bvec[:O] = bias.detach()
        y2 = ops.gemm(cols, wmat, bias=bvec)                   # [N * L, Op]
        y = torch.empty((N, O, ho, wo), dtype=torch.bfloat16, device=x.device)
        N_.check(lib.rb_nhwc_to_nchw(y2.data_ptr(), y2.stride(0), y.data_ptr(), N, L, O, N_.stream_ptr()), "rb_nhwc_to_nchw")
        ctx.save_for_backward(cols, wmat)
        ctx.geom = (N, C, H, W, O, kh, kw, stride, pad, L, K, Kp, Op)
        ctx.has_bias = bias is not None
        ctx.w_dtype = weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        cols, wmat = ctx.saved_tensors
        N, C, H, W, O, kh, kw, stride, pad, L, K, Kp, Op = ctx.geom
        lib = N_.kernels()
        dy = dy.contiguous().to(torch.bfloat16)
        dy2 = torch.empty((N * L, Op), dtype=torch.bfloat16, device=dy.device)
        N_.check(lib.rb_nchw_to_nhwc(dy.data_ptr(), dy2.data_ptr(), N, L, O, Op, N_.stream_ptr()), "rb_nchw_to_nhwc")
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dwm = ops.gemm(dy2, cols, a_mn=True, b_mn=True, out_dtype=torch.float32)      # [Op, Kp] = dY^T cols
            dw = dwm[:O, :K].reshape(O, C, kh, kw).to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops.sum_dim0(dy2)[:O].to(ctx.b_dtype)
        if ctx.needs_input_grad[0]:
            dcols = ops.gemm(dy2, wmat, b_mn=True)                                        # [N * L, Kp] = dY W
            dx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=dy.device)
            N_.check(lib.rb_col2im(dcols.data_ptr(), dx.data_ptr(), N, C, H, W, kh, kw, stride, pad[0], pad[1], Kp, N_.stream_ptr()),
                     "rb_col2im")
        return dx, dw, db, None, None


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
        if x.is_cuda and x.dtype == torch.bfloat16:
            return _Conv2dGemmFn.apply(x, self.weight.tensor, None if self.bias is None else self.bias.tensor, c.stride, pad)
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


N_.optional_sig("rb_max_pool2d_fwd", [_P, _P, _P, N_.c_ll, _I, _I, _I, _I, _I, _P])
N_.optional_sig("rb_max_pool2d_bwd", [_P, _P, _P, N_.c_ll, _I, _I, _I, _I, _I, _P])


class _MaxPool2dFn(torch.autograd.Function):
    """Max pooling of CUDA tensors (bf16 or fp32, NCHW) on the kernels of csrc/kernels/conv.cu: the forward keeps the
    position of every window's maximum, the backward gathers per input element (overlapping windows need no atomics)."""

    @staticmethod
    def forward(ctx, x, kernel, stride):
        x = x.contiguous()
        N, C, H, W = x.shape
        ho, wo = (H - kernel) // stride + 1, (W - kernel) // stride + 1
        y = torch.empty((N, C, ho, wo), dtype=x.dtype, device=x.device)
        idx = torch.empty((N, C, ho, wo), dtype=torch.int32, device=x.device)
        N_.check(N_.kernels().rb_max_pool2d_fwd(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N * C, H, W, kernel, stride,
                                                int(x.dtype == torch.bfloat16), N_.stream_ptr()), "rb_max_pool2d_fwd")
        ctx.save_for_backward(idx)
        ctx.geom = (N, C, H, W, kernel, stride)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        N, C, H, W, kernel, stride = ctx.geom
        dy = dy.contiguous()
        dx = torch.empty((N, C, H, W), dtype=dy.dtype, device=dy.device)
        N_.check(N_.kernels().rb_max_pool2d_bwd(dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N * C, H, W, kernel, stride,
                                                int(dy.dtype == torch.bfloat16), N_.stream_ptr()), "rb_max_pool2d_bwd")
        return dx, None, None


def max_pool2d(x: torch.Tensor, kernel: int = 2, stride: int | None = None) -> torch.Tensor:
    stride = stride or kernel
    if x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float32) and kernel <= min(x.shape[2], x.shape[3]):
        return _MaxPool2dFn.apply(x, kernel, stride)
    return F.max_pool2d(x, kernel, stride)


def global_max_pool2d(x: torch.Tensor) -> torch.Tensor:
    """[N, C, H, W] -> [N, C]: one window covering the whole image."""
    if x.is_cuda and x.dim() == 4 and x.shape[2] == x.shape[3] and x.dtype in (torch.bfloat16, torch.float32):
        return max_pool2d(x, x.shape[2]).reshape(x.shape[0], x.shape[1])
    return x.amax((2, 3))
