"""LayerNorm / RMSNorm (bf16 activations, fp32 statistics) with explicit forward / backward entry points."""
from __future__ import annotations

import torch

from .. import _native as N

_scratch: dict = {}


def _partial_scratch(device, numel: int) -> torch.Tensor:
    """Grow-only fp32 scratch for the parameter-gradient partials, one per device and stream."""
    key = N.stream_key(device)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1 << 16), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def norm_forward(x2: torch.Tensor, gamma: torch.Tensor, beta, eps: float, rms: bool, out=None, want_stats: bool = True):
    """x2: [rows, n].  Returns (y, mean, rstd); mean is None for RMSNorm, and both are None on a CUDA tensor when
    `want_stats` is False (inference: nothing will run backward)."""
    rows, n = x2.shape
    if not x2.is_cuda:
        xf = x2.float()
        if rms:
            mean = None
            rstd = torch.rsqrt((xf * xf).mean(-1) + eps)
            y = xf * rstd[:, None] * gamma.float()
        else:
            mean = xf.mean(-1)
            var = ((xf - mean[:, None]) ** 2).mean(-1)
            rstd = torch.rsqrt(var + eps)
            y = (xf - mean[:, None]) * rstd[:, None] * gamma.float()
            if beta is not None:
                y = y + beta.float()
        y = y.to(x2.dtype)
        if out is not None:
            out.copy_(y)
            y = out
        return y, mean, rstd
    if x2.dtype != torch.bfloat16 or gamma.dtype != torch.bfloat16:
        raise TypeError("norm: CUDA tensors must be bf16")
    y = out if out is not None else torch.empty((rows, n), dtype=x2.dtype, device=x2.device)
    mean = rstd = None
    if want_stats:
        if rms:
            rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
        else:
            mean, rstd = torch.empty((2, rows), dtype=torch.float32, device=x2.device).unbind(0)
    if rows == 0:
        return y, mean, rstd
    N.check(N.kernels().rb_norm_fwd(x2.data_ptr(), x2.stride(0), gamma.data_ptr(), N.ptr(beta), y.data_ptr(),
                                    y.stride(0), N.ptr(mean), N.ptr(rstd), rows, n, eps, int(rms),
                                    N.stream_ptr()), "rb_norm_fwd")
    return y, mean, rstd


def norm_backward(dy2, x2, gamma, mean, rstd, rms: bool, dres=None, dgamma=None, dbeta=None, accumulate=False,
                  dx_out=None):
    """Returns (dx, dgamma, dbeta); dgamma/dbeta are fp32.  `dres` (same shape as dx) is added into dx."""
    rows, n = x2.shape
    if not x2.is_cuda:
        xf, g = x2.float(), dy2.float()
        m = torch.zeros(rows) if rms else mean
        xhat = (xf - m[:, None]) * rstd[:, None]
        dg = (g * xhat).sum(0)
        db = None if rms else g.sum(0)
        gd = g * gamma.float()
        s1 = torch.zeros(rows, 1) if rms else gd.mean(-1, keepdim=True)
        s2 = (gd * xhat).mean(-1, keepdim=True)
        dx = rstd[:, None] * (gd - s1 - xhat * s2)
        if dres is not None:
            dx = dx + dres.float()
        dx = dx.to(x2.dtype)
        if dx_out is not None:
            dx_out.copy_(dx)
            dx = dx_out
        if dgamma is not None:
            dgamma.copy_(dgamma + dg if accumulate else dg)
            dg = dgamma
        if dbeta is not None and db is not None:
            dbeta.copy_(dbeta + db if accumulate else db)
            db = dbeta
        return dx, dg, db
    lib = N.kernels()
    nparts = lib.rb_norm_bwd_num_partials(rows, n)
    partial = _partial_scratch(x2.device, 2 * nparts * n)
    dx = dx_out if dx_out is not None else torch.empty_like(x2)
    if dgamma is None:
        dgamma = torch.empty(n, dtype=torch.float32, device=x2.device)
        accumulate = False
    if dbeta is None and not rms:
        dbeta = torch.empty(n, dtype=torch.float32, device=x2.device)
    N.check(lib.rb_norm_bwd(dy2.data_ptr(), dy2.stride(0), x2.data_ptr(), x2.stride(0), gamma.data_ptr(),
                            N.ptr(mean), rstd.data_ptr(), N.ptr(dres), dres.stride(0) if dres is not None else 0,
                            dx.data_ptr(), dx.stride(0), dgamma.data_ptr(), N.ptr(dbeta), partial.data_ptr(),
                            rows, n, int(rms), int(accumulate), N.stream_ptr()), "rb_norm_bwd")
    return dx, dgamma, dbeta


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, mean, rstd = norm_forward(x2, gamma, beta, eps, rms)
        ctx.save_for_backward(x2, gamma, mean if mean is not None else rstd, rstd)
        ctx.rms = rms
        ctx.has_beta = beta is not None
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, gamma, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx, dg, db = norm_backward(dy2, x2, gamma, None if ctx.rms else mean, rstd, ctx.rms)
        return (dx.reshape(ctx.shape), dg.to(gamma.dtype), db.to(gamma.dtype) if (ctx.has_beta and db is not None) else None,
                None, None)


def _norm_inference(x, gamma, beta, eps, rms):
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = norm_forward(x2, gamma, beta, eps, rms, want_stats=False)[0]
    return y if x.dim() == 2 else y.reshape(x.shape)


def layer_norm(x, gamma, beta, eps: float = 1e-5):
    """Population variance, eps inside the square root (crates/nn/src/normalization.rs:87-158)."""
    if not N.wants_grad(x, gamma, beta):
        return _norm_inference(x, gamma, beta, eps, False)
    return _NormFn.apply(x, gamma, beta, eps, False)


def rms_norm(x, gamma, eps: float = 1e-5):
    if not N.wants_grad(x, gamma):
        return _norm_inference(x, gamma, None, eps, True)
    return _NormFn.apply(x, gamma, None, eps, True)
