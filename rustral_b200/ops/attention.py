"""Flash attention (causal / full, MHA / GQA) with a differentiable wrapper and a plain reference."""
from __future__ import annotations

import math

import torch

from .. import _native as N


def attention_reference(q, k, v, causal: bool, scale: float | None = None, kv_lens=None):
    """fp32 softmax(QK^T * scale + mask) V on [B, S, H, D] tensors (GQA: fewer K/V heads).  `kv_lens` ([B] integers):
    keys at positions >= kv_lens[b] are padding (a batch entry without any real key gives zero rows)."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf, vf = k.float().permute(0, 2, 1, 3), v.float().permute(0, 2, 1, 3)
    if H != Hk:                                             # grouped-query attention: every K/V head serves H / Hk query heads
        kf, vf = kf.repeat_interleave(H // Hk, dim=1), vf.repeat_interleave(H // Hk, dim=1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    if kv_lens is not None:
        pad = torch.arange(Sk, device=q.device)[None, :] >= kv_lens.to(q.device).long()[:, None]      # [B, Sk]
        s = s.masked_fill(pad[:, None, None, :], float("-inf"))
    p = torch.softmax(s, -1)
    if kv_lens is not None:
        p = torch.nan_to_num(p, nan=0.0)                      # rows without a visible key
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def _strides3(t):
    # [B, S, H, D] view -> element strides (batch, row, head)
    return (t.stride(0), t.stride(1), t.stride(2))


def _fill(args, q, k, v, o, causal, scale, kv_lens=None):
    B, Sq, H, D = q.shape
    if kv_lens is not None:
        if kv_lens.dtype != torch.int32 or not kv_lens.is_cuda or kv_lens.numel() != B or not kv_lens.is_contiguous():
            raise TypeError("attention: kv_lens must be a contiguous int32 CUDA tensor with one entry per batch element")
        args.kv_lens = kv_lens.data_ptr()
    else:
        args.kv_lens = None
    args.q, args.k, args.v, args.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        st = _strides3(t)
        arr = getattr(args, name)
        arr[0], arr[1], arr[2] = st
    args.batch, args.heads, args.kv_heads = B, H, k.shape[2]
    args.seq_q, args.seq_k, args.head_dim = Sq, k.shape[1], D
    args.causal, args.scale = int(causal), scale


N.optional_sig("rb_attention_fwd_tc", [N.C.POINTER(N.RbAttnArgs), N.c_void_p])
N.optional_sig("rb_attention_bwd_tc", [N.C.POINTER(N.RbAttnArgs), N.c_void_p])
N.optional_sig("rb_attention_fwd_tc2", [N.C.POINTER(N.RbAttnArgs), N.c_int, N.c_void_p])
N.optional_sig("rb_attention_bwd_tc2", [N.C.POINTER(N.RbAttnArgs), N.c_void_p])
N._LAUNCHES["rb_attention_bwd_tc2"] = 3
N._LAUNCHES["rb_attention_bwd_tc"] = 3

# "tc2": tcgen05 kernel with two query tiles per CTA in ping-pong (falls back to "tc" for shapes it does not take);
# "tc": one query tile per CTA; "mma": the mma.sync kernel.
FORWARD_IMPL = __import__("os").environ.get("RUSTRAL_ATTN_IMPL", "tc2")
# Share of the exponentials the "tc2" kernel computes with a polynomial on the FMA pipe: 0 (none) or 4 (every fourth
# pair).  Measured on B200, batch 32 x 12 heads x 1024 x 64 / batch 4 x 32 (8 KV) heads x 4096 x 128: 0 -> 191 us / 732 us,
# 4 -> 218 / 847; the one-tile "tc" kernel 220 / 1492.
FORWARD_POLY_EVERY = int(__import__("os").environ.get("RUSTRAL_ATTN_POLY", "0"))
# Backward: "tc2" keeps P and dS in TMEM and feeds the dV / dK / dQ products from there; "tc" stages them through shared
# memory.  Measured on the same two shapes: tc2 497 us / 2502 us, tc 574 / 3146.
BACKWARD_IMPL = __import__("os").environ.get("RUSTRAL_ATTN_BWD_IMPL", "mma" if FORWARD_IMPL == "mma" else "tc2")


def attention_forward(q, k, v, causal: bool, scale: float, out=None, want_lse: bool = True, impl: str | None = None,
                      kv_lens=None):
    """q: [B, Sq, H, D]; k, v: [B, Sk, Hkv, D] (any strides with a contiguous D).  Returns (o, lse).  `kv_lens`
    (int32 [B] on the device): number of real keys per batch entry, the rest is padding (second-generation kernels)."""
    B, Sq, H, D = q.shape
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or t.stride(3) != 1:
            raise TypeError("attention: bf16 tensors with a contiguous head dimension are required")
    o = out if out is not None else torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if want_lse else None
    a = N.RbAttnArgs()
    _fill(a, q, k, v, o, causal, scale, kv_lens)
    a.lse = N.ptr(lse)
    lib = N.kernels()
    which = impl or FORWARD_IMPL
    if kv_lens is not None and not which.startswith("tc2"):
        which = "tc2"
    if which.startswith("tc2") and hasattr(lib, "rb_attention_fwd_tc2"):
        poly = int(which[4:]) if len(which) > 4 else FORWARD_POLY_EVERY          # "tc2:4" selects the share explicitly
        rc = lib.rb_attention_fwd_tc2(a, poly, N.stream_ptr())
        if rc != -9:
            N.check(rc, "rb_attention_fwd_tc2")
            return o, lse
        which = "tc"
    if which == "tc" and hasattr(lib, "rb_attention_fwd_tc"):
        rc = lib.rb_attention_fwd_tc(a, N.stream_ptr())
        if rc != -9:
            N.check(rc, "rb_attention_fwd_tc")
            return o, lse
    N.check(lib.rb_attention_fwd(a, N.stream_ptr()), "rb_attention_fwd")
    return o, lse


def attention_backward(do, q, k, v, o, lse, causal: bool, scale: float, dq=None, dk=None, dv=None, impl: str | None = None,
                       kv_lens=None):
    B, Sq, H, D = q.shape
    if do.stride(3) != 1 or _strides3(do) != _strides3(o):
        do = _match(do, o)
    dq = dq if dq is not None else torch.empty_like(q)
    dk = dk if dk is not None else torch.empty_like(k)
    dv = dv if dv is not None else torch.empty_like(v)
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    a = N.RbAttnArgs()
    _fill(a, q, k, v, o, causal, scale, kv_lens)
    a.d_o = do.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    for name, t in (("dq_strides", dq), ("dk_strides", dk), ("dv_strides", dv)):
        st = _strides3(t)
        arr = getattr(a, name)
        arr[0], arr[1], arr[2] = st
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    lib = N.kernels()
    which = "tc2" if kv_lens is not None else (impl or BACKWARD_IMPL)
    if which == "tc2" and hasattr(lib, "rb_attention_bwd_tc2"):     # P / dS kept in TMEM (falls back to "tc")
        rc = lib.rb_attention_bwd_tc2(a, N.stream_ptr())
        if rc != -9:
            N.check(rc, "rb_attention_bwd_tc2")
            return dq, dk, dv
        which = "tc"
    if which == "tc" and hasattr(lib, "rb_attention_bwd_tc"):
        rc = lib.rb_attention_bwd_tc(a, N.stream_ptr())
        if rc != -9:
            N.check(rc, "rb_attention_bwd_tc")
            return dq, dk, dv
    N.check(lib.rb_attention_bwd(a, N.stream_ptr()), "rb_attention_bwd")
    return dq, dk, dv


def _match(do, o):
    """A copy of `do` laid out with the strides of `o` (the kernel reads both with one stride set)."""
    buf = torch.empty_strided(o.shape, o.stride(), dtype=do.dtype, device=do.device)
    buf.copy_(do)
    return buf


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, kv_lens=None):
        o, lse = attention_forward(q, k, v, causal, scale, kv_lens=kv_lens)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale, ctx.kv_lens = causal, scale, kv_lens
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(do, q, k, v, o, lse, ctx.causal, ctx.scale, kv_lens=ctx.kv_lens)
        return dq, dk, dv, None, None, None


def flash_attention(q, k, v, causal: bool = True, scale: float | None = None, kv_lens=None):
    """Differentiable attention on [B, S, H, D] tensors.  CUDA: tiled flash kernels; CPU: reference math.
    `kv_lens` ([B] integers): number of real keys per batch entry (key-padding mask given as lengths)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if not q.is_cuda:
        return attention_reference(q, k, v, causal, scale, kv_lens)
    if kv_lens is not None:
        kv_lens = kv_lens.to(device=q.device, dtype=torch.int32).contiguous()
    D = q.shape[-1]
    in_dtype = q.dtype
    if in_dtype != torch.bfloat16:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    if D not in (64, 128):
        # The kernels take head dimensions 64 and 128.  Zero columns change neither QK^T nor the kept
        # columns of PV, so other sizes run padded (the scale stays that of the true head dimension).
        if D > 128:
            raise ValueError(f"flash_attention: head dimension {D} > 128 is not supported")
        Dp = 64 if D < 64 else 128
        pad = lambda t: torch.nn.functional.pad(t, (0, Dp - D))
        o = _FlashFn.apply(pad(q), pad(k), pad(v), causal, scale, kv_lens)[..., :D]
    else:
        q, k, v = (t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v))
        o = _FlashFn.apply(q, k, v, causal, scale, kv_lens)
    return o if in_dtype == torch.bfloat16 else o.to(in_dtype)
