"""The op tables a backend exposes (crates/core/src/backend.rs:212-675).

``TensorOps`` keeps the reference's method names (matmul, linear, softmax_dim, gather_rows, ...) so code written
against its ``ctx.backend().ops()`` idiom ports over; every method routes to ``rustral_b200.ops``: CUDA tensors
hit the sm_100a kernels, CPU tensors the fp32 reference math.  On CUDA, fp32 operands of GEMM-shaped ops are
rounded to bf16 (fp32 accumulate, fp32 result) because the tensor-core path is bf16.
"""
from __future__ import annotations

import torch

from .errors import InvalidArgument, ShapeMismatch


_OPS = None


def _ops_mod():
    """The kernel-wrapper package, imported on first use (it imports this package) and then kept: the op table is on the
    path of every small launch, where a `from .. import` statement per call is measurable."""
    global _OPS
    if _OPS is None:
        from .. import ops
        _OPS = ops
    return _OPS


class TensorOps:
    def __init__(self, backend):
        self.backend = backend

    # ---- construction / inspection -----------------------------------------------------------------
    def shape(self, t):
        return tuple(t.shape)

    def tensor_from_vec(self, values, shape):
        t = torch.as_tensor(values, dtype=torch.float32)
        n = 1
        for d in shape:
            n *= d
        if t.numel() != n:
            raise ShapeMismatch(shape, t.shape, "tensor_from_vec")
        return t.reshape(tuple(shape)).to(self.backend.device(), self.backend.dtype)

    def zeros(self, shape):
        return torch.zeros(tuple(shape), dtype=self.backend.dtype, device=self.backend.device())

    def tensor_to_vec(self, t):
        return t.detach().float().cpu().reshape(-1).tolist()

    def tensor_element(self, t, index: int):
        return float(t.detach().reshape(-1)[index].float().cpu())

    # ---- GEMM family ----------------------------------------------------------------------------------
    def _gemm(self, a, b_nk, bias=None, act="none"):
        ops = _ops_mod()
        if a.is_cuda and a.dtype == torch.float32:
            out = ops.gemm(ops.cast_f32_to_bf16(a.contiguous()), ops.cast_f32_to_bf16(b_nk.contiguous()),
                           bias=None if bias is None else ops.cast_f32_to_bf16(bias.contiguous()), act=act,
                           out_dtype=torch.float32)
            return out
        return ops.gemm(a.contiguous(), b_nk.contiguous(), bias=bias, act=act)

    def matmul(self, a, b):
        """[m,k] x [k,n]."""
        ops = _ops_mod()
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
            raise ShapeMismatch((a.shape[0], "k"), b.shape, "matmul")
        if a.is_cuda and a.dtype == torch.float32:
            return ops.gemm(ops.cast_f32_to_bf16(a.contiguous()), ops.cast_f32_to_bf16(b.contiguous()), b_mn=True,
                            out_dtype=torch.float32)
        return ops.gemm(a.contiguous(), b.contiguous(), b_mn=True)

    def linear(self, x, weight, bias=None):
        """x [batch,in] x weight[out,in]^T + bias."""
        return self._gemm(x, weight, bias)

    def transpose(self, a):
        ops = _ops_mod()
        return ops.transpose2d(a)

    # ---- elementwise ------------------------------------------------------------------------------------
    def _bin(self, op, a, b):
        ops = _ops_mod()
        return ops.binary(op, a, b)

    def add(self, a, b): return self._bin("add", a, b)
    def sub(self, a, b): return self._bin("sub", a, b)
    def mul(self, a, b): return self._bin("mul", a, b)
    def maximum(self, a, b): return self._bin("maximum", a, b)

    def div(self, a, b):
        if bool((b == 0).any()):
            raise InvalidArgument("div: division by zero")
        return self._bin("div", a, b)

    def _un(self, op, a):
        ops = _ops_mod()
        return ops.unary(op, a)

    def relu(self, a): return self._un("relu", a)
    def sigmoid(self, a): return self._un("sigmoid", a)
    def tanh(self, a): return self._un("tanh", a)
    def gelu(self, a): return self._un("gelu", a)
    def silu(self, a): return self._un("silu", a)
    def neg(self, a): return self._un("neg", a)
    def exp(self, a): return self._un("exp", a)

    def log(self, a):
        if bool((a <= 0).any()):
            raise InvalidArgument("log: non-positive input")
        return self._un("log", a)

    def sqrt(self, a):
        if bool((a < 0).any()):
            raise InvalidArgument("sqrt: negative input")
        return self._un("sqrt", a)

    def add_scalar(self, a, s):
        ops = _ops_mod()
        return ops.scalar_op("add_scalar", a, s)

    def mul_scalar(self, a, s):
        ops = _ops_mod()
        return ops.scalar_op("mul_scalar", a, s)

    def gt_scalar(self, a, s):
        ops = _ops_mod()
        return ops.scalar_op("gt_scalar", a, s)

    def add_row_vector(self, a, v):
        ops = _ops_mod()
        if a.shape[-1] != v.shape[-1]:
            raise ShapeMismatch((a.shape[-1],), v.shape, "add_row_vector")
        return ops.add_row_vector(a, v)

    def dropout(self, x, p: float, training: bool):
        ops = _ops_mod()
        import random
        return ops.dropout(x, p, training, seed=random.getrandbits(48))

    def dropout_with_seed(self, x, p: float, seed: int, training: bool = True):
        ops = _ops_mod()
        return ops.dropout(x, p, training, seed=seed)

    # ---- softmax / reductions ------------------------------------------------------------------------------
    def softmax(self, a):
        """Softmax over ALL elements (the reference's `softmax`); use softmax_dim for rows."""
        ops = _ops_mod()
        return ops.softmax(a.reshape(1, -1)).reshape(a.shape)

    def log_softmax(self, a):
        ops = _ops_mod()
        return ops.log_softmax(a.reshape(1, -1)).reshape(a.shape)

    def _dim_last(self, a, dim, fn):
        dim = dim % a.dim()
        if dim == a.dim() - 1:
            return fn(a)
        return fn(a.transpose(dim, -1).contiguous()).transpose(dim, -1).contiguous()

    def softmax_dim(self, a, dim: int):
        ops = _ops_mod()
        return self._dim_last(a, dim, ops.softmax)

    def log_softmax_dim(self, a, dim: int):
        ops = _ops_mod()
        return self._dim_last(a, dim, ops.log_softmax)

    def sum_all(self, a):
        ops = _ops_mod()
        return ops.sum_all(a)

    def sum_dim0(self, a):
        ops = _ops_mod()
        return ops.sum_dim0(a.reshape(a.shape[0], -1)).to(a.dtype).reshape(a.shape[1:])

    def sum_dim(self, a, dim: int, keepdim: bool = False):
        ops = _ops_mod()
        dim = dim % a.dim()
        moved = a.movedim(dim, 0).contiguous()
        r = ops.sum_dim0(moved.reshape(moved.shape[0], -1)).to(a.dtype).reshape(moved.shape[1:])
        return r.unsqueeze(dim) if keepdim else r

    def mean_dim(self, a, dim: int, keepdim: bool = False):
        return self.mul_scalar(self.sum_dim(a, dim, keepdim), 1.0 / a.shape[dim])

    def var_dim(self, a, dim: int, unbiased: bool = False, keepdim: bool = False):
        """Two-pass variance (crates/ndarray-backend/src/lib.rs:1392)."""
        mean = self.mean_dim(a, dim, keepdim=True)
        d = self.sub(a, mean.expand_as(a).contiguous())
        n = a.shape[dim] - (1 if unbiased else 0)
        return self.mul_scalar(self.sum_dim(self.mul(d, d), dim, keepdim), 1.0 / max(n, 1))

    def argmax(self, a):
        ops = _ops_mod()
        return int(ops.argmax_rows(a.reshape(1, -1))[0])

    def argmax_rows(self, a):
        ops = _ops_mod()
        return ops.argmax_rows(a)

    # ---- data movement -----------------------------------------------------------------------------------------
    def gather_rows(self, table, ids):
        ops = _ops_mod()
        ids = torch.as_tensor(ids, dtype=torch.int64, device=table.device)
        if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
            raise InvalidArgument("gather_rows: index out of range")
        return ops.gather_rows(table, ids)

    def broadcast_to(self, a, shape):
        ops = _ops_mod()
        if len(shape) == 2:
            return ops.broadcast_to(a, shape[0], shape[1])
        return a.expand(tuple(shape)).contiguous()

    def broadcast(self, a, shape):
        return self.broadcast_to(a, shape)

    def concat(self, tensors, dim: int = 0):
        ops = _ops_mod()
        ts = list(tensors)
        if ts[0].is_cuda and ts[0].dim() == 2 and dim in (1, -1):
            rows = ts[0].shape[0]
            out = torch.empty((rows, sum(t.shape[1] for t in ts)), dtype=ts[0].dtype, device=ts[0].device)
            c = 0
            for t in ts:
                ops.strided_copy(t.contiguous(), out[:, c:c + t.shape[1]])
                c += t.shape[1]
            return out
        return torch.cat(ts, dim)

    def slice(self, a, start: int, end: int, dim: int = 0):
        if not (0 <= start <= end <= a.shape[dim]):
            raise InvalidArgument(f"slice [{start},{end}) out of range for dim of size {a.shape[dim]}")
        return a.narrow(dim, start, end - start).contiguous()

    def reshape(self, a, shape):
        n = 1
        for d in shape:
            n *= d
        if n != a.numel():
            raise ShapeMismatch(shape, a.shape, "reshape")
        return a.reshape(tuple(shape))


class TensorInPlaceOps:
    """add_assign / mul_assign / axpy (crates/core/src/backend.rs:435)."""

    @staticmethod
    def add_assign(a, b):
        ops = _ops_mod()
        return ops.binary("add", a, b, out=a)

    @staticmethod
    def mul_assign(a, b):
        ops = _ops_mod()
        return ops.binary("mul", a, b, out=a)

    @staticmethod
    def axpy(alpha: float, x, y):
        """y += alpha * x"""
        ops = _ops_mod()
        return ops.binary("add", y, ops.scalar_op("mul_scalar", x, alpha), out=y)


class TensorView:
    """Zero-copy fp32 view of host tensors (crates/core/src/backend.rs:414-422).  Only tensors that live in host memory
    as contiguous fp32 can be viewed; device tensors are refused, as the reference's GPU backends refuse them: the
    caller makes the transfer explicit (`tensor.cpu()`) instead of paying for a hidden one."""

    @staticmethod
    def as_slice_f32(t):
        """A flat numpy float32 array sharing the tensor's memory (row-major)."""
        if t.is_cuda:
            raise InvalidArgument("as_slice_f32: the tensor lives on the GPU; copy it to the host explicitly")
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise InvalidArgument("as_slice_f32 needs a contiguous float32 tensor")
        return t.detach().reshape(-1).numpy()


class FusionOps:
    """Single-kernel linear + bias (+ activation): the GEMM epilogue does the rest (crates/core/src/backend.rs:475)."""

    def __init__(self, backend):
        self.backend = backend

    def fused_linear_bias(self, x, w, b):
        return self.backend.ops()._gemm(x, w, b, "none")

    def fused_linear_bias_relu(self, x, w, b):
        return self.backend.ops()._gemm(x, w, b, "relu")

    def fused_linear_bias_gelu(self, x, w, b):
        return self.backend.ops()._gemm(x, w, b, "gelu")

    def fused_linear_bias_silu(self, x, w, b):
        return self.backend.ops()._gemm(x, w, b, "silu")


class AttentionOps:
    """flash_attention_2(q, k, v, causal) on [B,S,H,D] (crates/core/src/backend.rs:551)."""

    def __init__(self, backend):
        self.backend = backend

    def flash_attention_2(self, q, k, v, causal: bool = False, scale=None):
        ops = _ops_mod()
        return ops.flash_attention(q, k, v, causal, scale)

    def flash_attention_2_with_mask(self, q, k, v, mask, scale=None):
        """Arbitrary additive mask [Sq,Sk]: computed with the reference math (fp32), O(S^2) memory."""
        import math
        B, Sq, H, D = q.shape
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
        rep = H // kf.shape[1]
        s = qf @ kf.repeat_interleave(rep, 1).transpose(-1, -2) * scale + mask.float()
        return (torch.softmax(s, -1) @ vf.repeat_interleave(rep, 1)).permute(0, 2, 1, 3).to(q.dtype)


class QuantizationOps:
    """Symmetric int8 quantisation (crates/core/src/backend.rs:615)."""

    def __init__(self, backend):
        self.backend = backend

    def quantize_int8(self, t):
        absmax = float(t.detach().abs().max())
        scale = absmax / 127.0 if absmax > 0 else 1.0
        q = torch.clamp(torch.round(t.float() / scale), -127, 127).to(torch.int8)
        return q, scale

    def dequantize_int8(self, q, scale: float, dtype=None):
        return (q.float() * scale).to(dtype or self.backend.dtype)

    def quantize_parameter_int8(self, p):
        return self.quantize_int8(p.tensor)

    def int8_matmul(self, qa, sa: float, qb, sb: float):
        """[m,k] int8 x [k,n] int8 -> fp32, exact integer accumulation."""
        acc = (qa.to(torch.int32).cpu() @ qb.to(torch.int32).cpu()).to(qa.device)
        return acc.float() * (sa * sb)
