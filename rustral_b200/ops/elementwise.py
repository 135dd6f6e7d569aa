"""Elementwise / reduction / data-movement ops (fp32 and bf16).

These mirror the reference's per-element tensor-op table (``TensorOps`` in crates/core/src/backend.rs:212-399,
WGSL entry points in crates/wgpu-backend/src/shaders.wgsl).  CUDA tensors run on the kernels in
``csrc/kernels/elementwise.cu``; CPU tensors on fp32 torch math.
"""
from __future__ import annotations

import math

import torch

from .. import _native as N

BINARY = {"add": 0, "mul": 1, "sub": 2, "div": 3, "maximum": 4}
UNARY = {"relu": 0, "sigmoid": 1, "tanh": 2, "exp": 3, "log": 4, "sqrt": 5, "neg": 6, "gelu": 7, "silu": 8, "copy": 9}
SCALAR = {"add_scalar": 0, "mul_scalar": 1, "gt_scalar": 2, "fill": 3}

_scratch: dict = {}


def _f32_scratch(device, n: int) -> torch.Tensor:
    key = N.stream_key(device)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 4096), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"elementwise kernels take fp32 or bf16, got {t.dtype}")


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


def _gelu_cpu(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


_CPU_UNARY = {
    "relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "exp": torch.exp, "log": torch.log,
    "sqrt": torch.sqrt, "neg": torch.neg, "gelu": _gelu_cpu, "silu": lambda x: x * torch.sigmoid(x),
    "copy": lambda x: x.clone(),
}
_CPU_BINARY = {"add": torch.add, "mul": torch.mul, "sub": torch.sub, "div": torch.div, "maximum": torch.maximum}


def binary(op: str, a, b, out=None):
    if a.shape != b.shape:
        raise ValueError(f"{op}: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
    if not a.is_cuda:
        r = _CPU_BINARY[op](a.float(), b.float()).to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, b = _c(a), _c(b)
    out = out if out is not None else torch.empty_like(a)
    N.check(N.kernels().rb_binary(BINARY[op], a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _dt(a),
                                  N.stream_ptr()), f"rb_binary[{op}]")
    return out


def unary(op: str, a, out=None):
    if not a.is_cuda:
        r = _CPU_UNARY[op](a.float()).to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a = _c(a)
    out = out if out is not None else torch.empty_like(a)
    N.check(N.kernels().rb_unary(UNARY[op], a.data_ptr(), out.data_ptr(), a.numel(), _dt(a), N.stream_ptr()),
            f"rb_unary[{op}]")
    return out


def scalar_op(op: str, a, s: float, out=None):
    if not a.is_cuda:
        af = a.float()
        r = {"add_scalar": lambda: af + s, "mul_scalar": lambda: af * s, "gt_scalar": lambda: (af > s).float(),
             "fill": lambda: torch.full_like(af, s)}[op]().to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a = _c(a)
    out = out if out is not None else torch.empty_like(a)
    N.check(N.kernels().rb_scalar(SCALAR[op], a.data_ptr(), float(s), out.data_ptr(), a.numel(), _dt(a),
                                  N.stream_ptr()), f"rb_scalar[{op}]")
    return out


def unary_bwd(op: str, x, dy, out=None):
    """dy * op'(x) for relu / sigmoid / tanh / gelu / silu."""
    if not x.is_cuda:
        from .matmul import act_grad_reference
        xf = x.float()
        if op == "sigmoid":
            s = torch.sigmoid(xf)
            g = s * (1 - s)
        elif op == "tanh":
            g = 1 - torch.tanh(xf) ** 2
        else:
            g = act_grad_reference(op, xf)
        r = (dy.float() * g).to(x.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    x, dy = _c(x), _c(dy)
    out = out if out is not None else torch.empty_like(x)
    N.check(N.kernels().rb_unary_bwd(UNARY[op], x.data_ptr(), dy.data_ptr(), out.data_ptr(), x.numel(), _dt(x),
                                     N.stream_ptr()), f"rb_unary_bwd[{op}]")
    return out


class _UnaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op):
        ctx.save_for_backward(x)
        ctx.op = op
        return unary(op, x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return unary_bwd(ctx.op, x, dy), None


def gelu(x):
    """tanh-approximated GELU (crates/ndarray-backend/src/lib.rs:565), differentiable."""
    return _UnaryFn.apply(x, "gelu") if N.wants_grad(x) else unary("gelu", x)


def relu(x):
    return _UnaryFn.apply(x, "relu") if N.wants_grad(x) else unary("relu", x)


def silu(x):
    return _UnaryFn.apply(x, "silu") if N.wants_grad(x) else unary("silu", x)


def add_row_vector(a, v):
    if not a.is_cuda:
        return (a.float() + v.float()).to(a.dtype)
    a, v = _c(a), _c(v)
    out = torch.empty_like(a)
    rows = a.numel() // a.shape[-1]
    N.check(N.kernels().rb_add_row_vector(a.data_ptr(), v.data_ptr(), out.data_ptr(), rows, a.shape[-1], _dt(a),
                                          N.stream_ptr()), "rb_add_row_vector")
    return out


def sum_dim0(a, out=None, accumulate: bool = False):
    """Column sums of a 2-D tensor, fp32 result, fixed summation order."""
    if not a.is_cuda:
        r = a.float().sum(0) if (a.requires_grad or _par_reduce()) else a.double().sum(0).float()
        if out is not None:
            out.copy_(out + r if accumulate else r)
            return out
        return r
    if a.stride(1) != 1:
        a = a.contiguous()
    rows, cols = a.shape
    if out is None:
        out = torch.empty(cols, dtype=torch.float32, device=a.device)
        accumulate = False
    if rows == 0:
        return out if accumulate else out.zero_()
    lib = N.kernels()
    slabs = lib.rb_sum_dim0_slabs()
    partial = _f32_scratch(a.device, slabs * cols)
    N.check(lib.rb_sum_dim0_staged(a.data_ptr(), a.stride(0), out.data_ptr(), partial.data_ptr(), rows, cols, _dt(a),
                                   int(accumulate), N.stream_ptr()), "rb_sum_dim0_staged")
    return out


def _par_reduce() -> bool:
    from ..core import parallel_reductions_enabled
    return parallel_reductions_enabled()


def sum_all(a):
    if not a.is_cuda:
        if a.requires_grad or _par_reduce():
            return a.float().sum()
        return a.double().sum().float()           # reproducible whatever the thread count (see core.parallel_reductions_enabled)
    a = _c(a)
    out = torch.empty((), dtype=torch.float32, device=a.device)
    scratch = _f32_scratch(a.device, 1024)
    N.check(N.kernels().rb_sum_all(a.data_ptr(), a.numel(), _dt(a), scratch.data_ptr(), out.data_ptr(),
                                   N.stream_ptr()), "rb_sum_all")
    return out


def transpose2d(a):
    if not a.is_cuda:
        return a.t().contiguous()
    a = _c(a)
    out = torch.empty((a.shape[1], a.shape[0]), dtype=a.dtype, device=a.device)
    N.check(N.kernels().rb_transpose(a.data_ptr(), out.data_ptr(), a.shape[0], a.shape[1], _dt(a), N.stream_ptr()),
            "rb_transpose")
    return out


def gather_rows(a, idx):
    if not a.is_cuda:
        return a[idx]
    a = _c(a)
    idx = _c(idx.to(torch.int64))
    out = torch.zeros((idx.numel(), a.shape[1]), dtype=a.dtype, device=a.device)
    N.check(N.kernels().rb_gather_rows(a.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), a.shape[1],
                                       a.shape[0], _dt(a), N.stream_ptr()), "rb_gather_rows")
    return out


def scatter_rows(a, idx, out):
    """out[idx[i], :] = a[i, :] (overwrite; duplicates: last writer wins, unordered)."""
    if not a.is_cuda:
        out[idx] = a
        return out
    a = _c(a)
    idx = _c(idx.to(torch.int64))
    N.check(N.kernels().rb_scatter_rows(a.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), a.shape[1],
                                        out.shape[0], _dt(a), N.stream_ptr()), "rb_scatter_rows")
    return out


def broadcast_to(a, rows: int, cols: int):
    a2 = a.reshape(-1, a.shape[-1]) if a.dim() > 1 else a.reshape(1, -1)
    if not a.is_cuda:
        return a2.repeat((rows + a2.shape[0] - 1) // a2.shape[0], (cols + a2.shape[1] - 1) // a2.shape[1])[:rows, :cols].contiguous()
    a2 = _c(a2)
    out = torch.empty((rows, cols), dtype=a.dtype, device=a.device)
    N.check(N.kernels().rb_broadcast_to(a2.data_ptr(), out.data_ptr(), a2.shape[0], a2.shape[1], rows, cols, _dt(a),
                                        N.stream_ptr()), "rb_broadcast_to")
    return out


def strided_copy(a, out):
    """2-D copy between tensors whose rows are contiguous but whose row pitches differ (slices, concat)."""
    if not a.is_cuda:
        out.copy_(a)
        return out
    assert a.dim() == 2 and out.shape == a.shape and a.stride(1) == 1 and out.stride(1) == 1
    N.check(N.kernels().rb_strided_copy(a.data_ptr(), a.stride(0), out.data_ptr(), out.stride(0), a.shape[0],
                                        a.shape[1], _dt(a), N.stream_ptr()), "rb_strided_copy")
    return out


def apply_mask(a, mask, mask_value: float):
    if not a.is_cuda:
        return torch.where(mask > 0, a, torch.full_like(a, mask_value))
    a, mask = _c(a), _c(mask.to(a.dtype))
    out = torch.empty_like(a)
    N.check(N.kernels().rb_apply_mask(a.data_ptr(), mask.data_ptr(), float(mask_value), out.data_ptr(), a.numel(),
                                      _dt(a), N.stream_ptr()), "rb_apply_mask")
    return out


def _pcg_hash_np(v):
    import numpy as np
    v = v.astype(np.uint32)
    state = v * np.uint32(747796405) + np.uint32(2891336453)
    word = ((state >> ((state >> np.uint32(28)) + np.uint32(4))) ^ state) * np.uint32(277803737)
    return (word >> np.uint32(22)) ^ word


def dropout_mask_reference(n: int, p: float, seed: int):
    """Keep-mask of the PCG-hash generator (rng=1), restated on the host for parity tests."""
    import numpy as np
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        h = _pcg_hash_np((np.uint64(seed & 0xFFFFFFFF) + idx * np.uint64(12345)).astype(np.uint32))
    u = h.astype(np.float32) * np.float32(1.0 / 4294967296.0)
    return torch.from_numpy((u >= np.float32(p)))


def dropout(a, p: float, training: bool = True, seed: int = 0, offset: int = 0, rng: str = "philox",
            return_mask: bool = False):
    """Inverted dropout; identity when not training or p == 0.  p must lie in [0, 1)."""
    if not (0.0 <= p < 1.0):
        raise ValueError(f"dropout probability must be in [0, 1), got {p}")
    if not training or p <= 0.0:
        return (a, None) if return_mask else a
    if not a.is_cuda:
        if rng == "pcg":
            keep = dropout_mask_reference(a.numel(), p, seed).reshape(a.shape)
        else:
            gen = torch.Generator().manual_seed(seed + offset)
            keep = torch.rand(a.shape, generator=gen) >= p
        r = (a.float() * keep.float() / (1.0 - p)).to(a.dtype)
        return (r, keep) if return_mask else r
    a = _c(a)
    out = torch.empty_like(a)
    mask = torch.empty(a.shape, dtype=torch.uint8, device=a.device) if return_mask else None
    N.check(N.kernels().rb_dropout(a.data_ptr(), out.data_ptr(), N.ptr(mask), a.numel(), float(p), seed, offset,
                                   1 if rng == "pcg" else 0, _dt(a), N.stream_ptr()), "rb_dropout")
    return (out, mask) if return_mask else out


def argmax_rows(a):
    a2 = a.reshape(-1, a.shape[-1])
    if not a.is_cuda:
        return a2.float().argmax(-1)
    if a2.stride(1) != 1:
        a2 = a2.contiguous()
    out = torch.empty(a2.shape[0], dtype=torch.int64, device=a.device)
    N.check(N.kernels().rb_argmax_rows(a2.data_ptr(), a2.stride(0), out.data_ptr(), a2.shape[0], a2.shape[1], _dt(a2),
                                       N.stream_ptr()), "rb_argmax_rows")
    return out
