"""Quantised matrix products: e4m3 x e4m3 on the tensor cores (`tcgen05.mma kind::f8f6f4`, fp32 accumulation, scales in
the epilogue) and exact int8 / group-wise int4 -> bf16 expansion ahead of the bf16 kernel.

The reference dequantises to f32 on the host and calls a plain matmul (crates/nn/src/quantization.rs:168-320
QuantizedLinear, :324-430 GPTQLinear).  CPU tensors follow the same arithmetic in fp32 and are the oracle of the GPU
tests.
"""
from __future__ import annotations

import torch

from .. import _native as N

P, c_int, c_ll = N.c_void_p, N.c_int, N.c_ll
N.optional_sig("rb_quantize_fp8_rows", [P, c_ll, P, c_ll, P, c_int, c_int, P])
N.optional_sig("rb_dequant_int8_bf16", [P, P, c_int, P, c_int, c_int, P])
N.optional_sig("rb_dequant_int4_bf16", [P, P, c_int, P, c_int, c_int, P])

E4M3_MAX = 448.0


def _e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """fp32 values rounded to the nearest e4m3 number (saturating at +-448), returned as fp32."""
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()


def quantize_fp8_rows(x: torch.Tensor, out: torch.Tensor | None = None, scales: torch.Tensor | None = None):
    """Row-wise dynamic e4m3 quantisation: returns (bytes [rows, n] as uint8, scales fp32 [rows]) with
    ``x ~= scales[:, None] * e4m3(bytes)``; ``scale = absmax / 448`` (1 for an all-zero row)."""
    assert x.dim() == 2
    rows, n = x.shape
    if not x.is_cuda:
        f = x.float()
        amax = f.abs().amax(1)
        sc = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q = (f * (1.0 / sc)[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
        if out is not None:
            out.copy_(q)
            q = out
        if scales is not None:
            scales.copy_(sc)
            sc = scales
        return q, sc
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    if x.stride(1) != 1:
        x = x.contiguous()
    if n % 16:
        raise ValueError("quantize_fp8_rows: the row length must be a multiple of 16")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.uint8, device=x.device)
    if scales is None:
        scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    N.check(N.kernels().rb_quantize_fp8_rows(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), scales.data_ptr(),
                                             rows, n, N.stream_ptr()), "rb_quantize_fp8_rows")
    return out, scales


def gemm_fp8(a8: torch.Tensor, a_scale, b8: torch.Tensor, b_scale, *, bias=None, act: str = "none", residual=None,
             out=None, out_dtype=torch.bfloat16, block_n: int = 0, b_e5m2: bool = False) -> torch.Tensor:
    """``out[i, j] = act(a_scale[i] * b_scale[j] * sum_k e4m3(a8[i, k]) * e4m3(b8[j, k]) + bias[j]) (+ residual)``.

    `a8` [M, K] and `b8` [N, K] hold e4m3 bytes (uint8 or torch.float8_e4m3fn; `b_e5m2`: `b8` holds e5m2 bytes); the
    scales are fp32 vectors or None."""
    assert a8.dim() == 2 and b8.dim() == 2 and a8.shape[1] == b8.shape[1]
    M, K = a8.shape
    Nn = b8.shape[0]
    if not a8.is_cuda:
        af = a8.view(torch.float8_e4m3fn).float()
        bf = b8.view(torch.float8_e5m2 if b_e5m2 else torch.float8_e4m3fn).float()
        y = af @ bf.t()
        if a_scale is not None:
            y = y * a_scale.float()[:, None]
        if b_scale is not None:
            y = y * b_scale.float()[None, :]
        if bias is not None:
            y = y + bias.float()
        if act != "none":
            from .matmul import act_reference
            y = act_reference(act, y)
        if residual is not None:
            y = y + residual.float()
        y = y.to(out_dtype if out is None else out.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if a8.stride(1) != 1 or b8.stride(1) != 1:
        raise ValueError("gemm_fp8: operands must have a contiguous last dimension")
    if K % 16:
        raise ValueError("gemm_fp8: K must be a multiple of 16")
    if out is None:
        out = torch.empty((M, Nn), dtype=out_dtype, device=a8.device)
    g = N.RbGemmArgs()
    g.a, g.b, g.d = a8.data_ptr(), b8.data_ptr(), out.data_ptr()
    g.bias, g.residual = N.ptr(bias), N.ptr(residual)
    g.lda, g.ldb, g.ldd = a8.stride(0), b8.stride(0), out.stride(0)
    g.ldr = residual.stride(0) if residual is not None else 0
    g.M, g.N, g.K = M, Nn, K
    g.act = N.ACT[act]
    g.out_f32 = int(out.dtype == torch.float32)
    g.alpha = 1.0
    g.block_n, g.splits = block_n, 1
    g.ab_fp8 = 2 if b_e5m2 else 1
    g.a_scale = None if a_scale is None else a_scale.data_ptr()
    g.b_scale = None if b_scale is None else b_scale.data_ptr()
    for t, nm in ((bias, "bias"), (residual, "residual")):
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"gemm_fp8: {nm} must be bf16")
    for t, n_, nm in ((a_scale, M, "a_scale"), (b_scale, Nn, "b_scale")):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n_ or not t.is_contiguous()):
            raise TypeError(f"gemm_fp8: {nm} must be a contiguous fp32 vector of {n_} elements")
    N.check(N.kernels().rb_gemm_bf16(g, N.stream_ptr()), "rb_gemm_bf16(fp8)")
    return out


def dequant_int8(q: torch.Tensor, zero_point=None, out=None) -> torch.Tensor:
    """int8 [rows, n] -> bf16 ``q - zero_point`` (exact); `zero_point`: None, a one-element or a per-row fp32 tensor."""
    rows, n = q.shape
    if not q.is_cuda:
        f = q.float()
        if zero_point is not None:
            f = f - zero_point.float().reshape(-1, 1)
        return f.to(torch.bfloat16)
    if n % 16 or not q.is_contiguous():
        raise ValueError("dequant_int8: rows must be contiguous with a length that is a multiple of 16")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=q.device)
    zp = None if zero_point is None else zero_point.to(device=q.device, dtype=torch.float32).reshape(-1).contiguous()
    per_row = int(zp is not None and zp.numel() == rows and rows > 1)
    N.check(N.kernels().rb_dequant_int8_bf16(q.data_ptr(), N.ptr(zp), per_row, out.data_ptr(), rows, n, N.stream_ptr()),
            "rb_dequant_int8_bf16")
    return out


def dequant_int4(packed: torch.Tensor, scales: torch.Tensor, group_size: int, out=None) -> torch.Tensor:
    """Nibbles [rows, n / 2] (element 2b in the low half of byte b, zero point 8) with fp32 scales [rows, n / group]
    -> bf16 ``(q - 8) * scale``."""
    rows, half = packed.shape
    n = half * 2
    if not packed.is_cuda:
        q = torch.empty((rows, n), dtype=torch.float32)
        q[:, 0::2] = (packed & 0xF).float()
        q[:, 1::2] = (packed >> 4).float()
        g = (q - 8.0).view(rows, n // group_size, group_size) * scales.float().unsqueeze(-1)
        return g.view(rows, n).to(torch.bfloat16)
    if n % 32 or group_size % 32 or n % group_size:
        raise ValueError("dequant_int4: row length and group size must be multiples of 32")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=packed.device)
    sc = scales.to(torch.float32).contiguous()
    N.check(N.kernels().rb_dequant_int4_bf16(packed.contiguous().data_ptr(), sc.data_ptr(), group_size, out.data_ptr(), rows, n,
                                             N.stream_ptr()), "rb_dequant_int4_bf16")
    return out
