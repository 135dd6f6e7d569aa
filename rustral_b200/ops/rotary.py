"""Rotary position embedding and SwiGLU (explicit forward / backward entry points + differentiable wrappers)."""
from __future__ import annotations

import torch

from .. import _native as N

N.optional_sig("rb_rope", [N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_int, N.c_int, N.c_int, N.c_ll, N.c_float,
                           N.c_int, N.c_void_p])
N.optional_sig("rb_swiglu_fwd", [N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_ll, N.c_int, N.c_void_p])
N.optional_sig("rb_swiglu_bwd", [N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_ll, N.c_int,
                                 N.c_void_p])


def _rope_ref(x3, pos, theta, inverse):
    T, H, D = x3.shape
    half = D // 2
    idx = torch.arange(half, dtype=torch.float32, device=x3.device)
    inv_freq = theta ** (-2.0 * idx / D)
    ang = pos.float()[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if inverse:
        s = -s
    x0, x1 = x3[..., :half].float(), x3[..., half:].float()
    return torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], -1).to(x3.dtype)


def rope_(x2: torch.Tensor, heads: int, head_dim: int, seq_len: int = 0, positions=None, pos_offset: int = 0,
          theta: float = 10000.0, inverse: bool = False) -> torch.Tensor:
    """In place on the first ``heads * head_dim`` columns of the 2-D tensor ``x2`` [tokens, >= heads*head_dim]."""
    tokens = x2.shape[0]
    if not x2.is_cuda:
        pos = positions if positions is not None else pos_offset + (torch.arange(tokens) % max(seq_len, 1))
        view = x2[:, :heads * head_dim].reshape(tokens, heads, head_dim)
        x2[:, :heads * head_dim] = _rope_ref(view, pos, theta, inverse).reshape(tokens, heads * head_dim)
        return x2
    if x2.dtype != torch.bfloat16 or x2.stride(1) != 1:
        raise TypeError("rope: bf16 rows with a contiguous last dimension are required")
    if positions is not None:
        positions = positions.to(torch.int64).contiguous()
    N.check(N.kernels().rb_rope(x2.data_ptr(), x2.stride(0), N.ptr(positions), tokens, heads, head_dim, seq_len,
                                pos_offset, theta, int(inverse), N.stream_ptr()), "rb_rope")
    return x2


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_len, positions, pos_offset, theta):
        # x: [B, S, H, D] (contiguous); returns a rotated copy
        B, S, H, D = x.shape
        y = x.contiguous().clone().reshape(B * S, H * D)
        rope_(y, H, D, seq_len, positions, pos_offset, theta, False)
        ctx.meta = (seq_len, positions, pos_offset, theta, x.shape)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        seq_len, positions, pos_offset, theta, shape = ctx.meta
        B, S, H, D = shape
        g = dy.contiguous().clone().reshape(B * S, H * D)
        rope_(g, H, D, seq_len, positions, pos_offset, theta, True)
        return g.reshape(shape), None, None, None, None


def rope(x, seq_len: int | None = None, positions=None, pos_offset: int = 0, theta: float = 10000.0):
    """Differentiable rotary embedding of [B, S, H, D]."""
    return _RopeFn.apply(x, seq_len if seq_len is not None else x.shape[1], positions, pos_offset, theta)


def swiglu_forward(gu2: torch.Tensor, out=None) -> torch.Tensor:
    tokens, F2 = gu2.shape
    F = F2 // 2
    if not gu2.is_cuda:
        g, u = gu2[:, :F].float(), gu2[:, F:].float()
        r = (g * torch.sigmoid(g) * u).to(gu2.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    out = out if out is not None else torch.empty((tokens, F), dtype=gu2.dtype, device=gu2.device)
    N.check(N.kernels().rb_swiglu_fwd(gu2.data_ptr(), gu2.stride(0), out.data_ptr(), out.stride(0), tokens, F,
                                      N.stream_ptr()), "rb_swiglu_fwd")
    return out


def swiglu_backward(dh2, gu2, out=None):
    tokens, F2 = gu2.shape
    F = F2 // 2
    if not gu2.is_cuda:
        g, u, d = gu2[:, :F].float(), gu2[:, F:].float(), dh2.float()
        s = torch.sigmoid(g)
        r = torch.cat([d * u * (s * (1 + g * (1 - s))), d * g * s], -1).to(gu2.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    out = out if out is not None else torch.empty_like(gu2)
    N.check(N.kernels().rb_swiglu_bwd(dh2.data_ptr(), dh2.stride(0), gu2.data_ptr(), gu2.stride(0), out.data_ptr(),
                                      out.stride(0), tokens, F, N.stream_ptr()), "rb_swiglu_bwd")
    return out


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu2 = gu.reshape(-1, gu.shape[-1])
        if not gu2.is_contiguous():
            gu2 = gu2.contiguous()
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return swiglu_forward(gu2).reshape(*gu.shape[:-1], gu.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dh):
        (gu2,) = ctx.saved_tensors
        dh2 = dh.reshape(-1, dh.shape[-1])
        if not dh2.is_contiguous():
            dh2 = dh2.contiguous()
        return swiglu_backward(dh2, gu2).reshape(ctx.shape)


def swiglu(gu):
    """``silu(gate) * up`` for ``gu = [gate | up]`` along the last dimension."""
    return _SwigluFn.apply(gu)
