"""Fused optimizer steps over flat fp32 state."""
from __future__ import annotations

import math

import torch

from .. import _native as N

_scratch: dict = {}


def _f32_scratch(device, n: int) -> torch.Tensor:
    key = N.stream_key(device)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def adam_step(p, m, v, g, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step: int, decoupled=True,
              grad_scale: float = 1.0, p_lowp=None, max_grad_norm: float = 0.0, grad_norm=None, found_inf=None):
    """One Adam / AdamW step in place on flat tensors.  `p`, `m`, `v` fp32; `g` fp32 or bf16;
    `p_lowp` (bf16, optional) receives the rounded parameters.  `grad_norm` / `found_inf` are device
    scalars read by the kernel, so clipping and overflow-skip need no host synchronisation."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not p.is_cuda:
        if found_inf is not None and int(found_inf) != 0:
            return
        gs = grad_scale
        if max_grad_norm > 0 and grad_norm is not None:
            coef = max_grad_norm / (float(grad_norm) + 1e-6)
            if coef < 1.0:
                gs *= coef
        gf = g.float()
        if gs != 1.0:
            gf = gf * gs
        if not decoupled and weight_decay != 0.0:
            gf = gf + weight_decay * p
        m.mul_(beta1).add_(gf, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        # p -= lr * ((m / bc1) / (sqrt(v / bc2) + eps) + wd * p) with one temporary: sqrt(v / bc2) = sqrt(v) / sqrt(bc2)
        denom = v.sqrt().div_(math.sqrt(bc2)).add_(eps)
        if decoupled and weight_decay != 0.0:
            p.mul_(1.0 - lr * weight_decay)
        p.addcdiv_(m, denom, value=-lr / bc1)
        if p_lowp is not None:
            p_lowp.copy_(p.to(p_lowp.dtype))
        return
    a = N.RbAdamArgs(lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, int(decoupled), max_grad_norm)
    N.check(N.kernels().rb_adam_step(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                     int(g.dtype == torch.bfloat16), N.ptr(p_lowp), p.numel(), a, N.ptr(grad_norm),
                                     N.ptr(found_inf), N.stream_ptr()), "rb_adam_step")


def sgd_step(p, g, *, lr, momentum=0.0, weight_decay=0.0, mom=None, grad_scale=1.0, p_lowp=None):
    if not p.is_cuda:
        gf = g.float() * grad_scale + weight_decay * p
        if mom is not None and momentum != 0.0:
            mom.mul_(momentum).add_(gf)
            gf = mom
        p.add_(gf, alpha=-lr)
        if p_lowp is not None:
            p_lowp.copy_(p.to(p_lowp.dtype))
        return
    N.check(N.kernels().rb_sgd_step(p.data_ptr(), N.ptr(mom), g.data_ptr(), int(g.dtype == torch.bfloat16),
                                    N.ptr(p_lowp), p.numel(), lr, momentum, weight_decay, grad_scale,
                                    N.stream_ptr()), "rb_sgd_step")


def sumsq(x, out=None, found_inf=None, accumulate=False):
    """Sum of squares as a device fp32 scalar (ordered reduction); sets `found_inf` on a non-finite value."""
    if not x.is_cuda:
        r = (x.float() ** 2).sum()
        if found_inf is not None and not torch.isfinite(x.float()).all():
            found_inf.fill_(1)
        if out is not None:
            out.copy_(out + r if accumulate else r)
            return out
        return r
    x = x if x.is_contiguous() else x.contiguous()
    lib = N.kernels()
    if out is None:
        out = torch.zeros((), dtype=torch.float32, device=x.device)
    scratch = _f32_scratch(x.device, lib.rb_sumsq_scratch_floats())
    N.check(lib.rb_sumsq(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(), scratch.data_ptr(), out.data_ptr(),
                         N.ptr(found_inf), int(accumulate), N.stream_ptr()), "rb_sumsq")
    return out


def sqrt_scalar(x, out=None):
    if not x.is_cuda:
        if out is None:
            return x.sqrt()
        out.copy_(x.sqrt())
        return out
    out = out if out is not None else torch.empty_like(x)
    N.check(N.kernels().rb_sqrt_scalar(x.data_ptr(), out.data_ptr(), N.stream_ptr()), "rb_sqrt_scalar")
    return out


def cast_f32_to_bf16(src, dst=None):
    if not src.is_cuda:
        r = src.to(torch.bfloat16)
        if dst is not None:
            dst.copy_(r)
            return dst
        return r
    dst = dst if dst is not None else torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    N.check(N.kernels().rb_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), N.stream_ptr()),
            "rb_cast_f32_to_bf16")
    return dst
