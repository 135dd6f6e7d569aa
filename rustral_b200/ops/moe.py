"""Mixture-of-experts ops: top-k routing, the token -> expert permutation, grouped expert GEMMs, combine, and a
differentiable expert-MLP layer built from them.

On CUDA the expert matmuls run as ONE grouped tcgen05 GEMM per projection over the permuted token buffer (expert
segments are padded to whole 128-row tiles, the tile scheduler reads the tile -> expert table from device memory,
so there is no host synchronisation on the routing result).  CPU tensors take the reference math.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N
from . import rotary
from .matmul import gemm, act_reference, act_grad_reference

P, I, F, LL = N.c_void_p, N.c_int, N.c_float, N.c_ll
N.optional_sig("rb_moe_route", [P, I, I, I, I, P, P, P, P])
N.optional_sig("rb_moe_route_bwd", [P, P, P, P, P, I, I, I, I, F, P, P])
N.optional_sig("rb_moe_plan", [P, I, I, I, P, P, P, P, P, P, I, P])
N.optional_sig("rb_moe_gather", [P, P, P, P, I, I, I, P, P])
N.optional_sig("rb_moe_combine", [P, P, P, P, P, I, I, I, P])
N.optional_sig("rb_moe_weight_grad", [P, P, P, P, I, I, I, P])

ROW_ALIGN = 128


def route(logits: torch.Tensor, k: int, renorm: bool = True):
    """logits fp32 [T, E] -> (idx int32 [T, k], w fp32 [T, k], probs fp32 [T, E])."""
    T, E = logits.shape
    if not logits.is_cuda:
        probs = torch.softmax(logits.float(), -1)
        # descending probability, ties to the lower index: stable sort of the negated values
        order = torch.sort(-probs, dim=-1, stable=True).indices[:, :k]
        w = probs.gather(1, order)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        return order.to(torch.int32), w, probs
    logits = logits.float().contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    probs = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    N.check(N.kernels().rb_moe_route(logits.data_ptr(), T, E, k, int(renorm), idx.data_ptr(), w.data_ptr(), probs.data_ptr(),
                                     N.stream_ptr()), "rb_moe_route")
    return idx, w, probs


def route_backward(probs, idx, w, dw, counts, renorm: bool, aux_grad_scale: float):
    """dlogits fp32 [T, E] from dw [T, k] and the load-balancing loss E * sum_e f_e P_e scaled by aux_grad_scale."""
    T, E = probs.shape
    k = idx.shape[1]
    if not probs.is_cuda:
        dp = torch.zeros_like(probs)
        li = idx.long()
        if renorm:
            S = probs.gather(1, li).sum(-1, keepdim=True)
            dot = (dw * w).sum(-1, keepdim=True)
            dp.scatter_add_(1, li, (dw - dot) / S)
        else:
            dp.scatter_add_(1, li, dw)
        dp = dp + aux_grad_scale * E * (counts.float() / (T * k))[None, :] / T
        return probs * (dp - (dp * probs).sum(-1, keepdim=True))
    out = torch.empty_like(probs)
    N.check(N.kernels().rb_moe_route_bwd(probs.data_ptr(), idx.data_ptr(), w.data_ptr(), dw.contiguous().data_ptr(),
                                         counts.data_ptr(), T, E, k, int(renorm), float(aux_grad_scale), out.data_ptr(),
                                         N.stream_ptr()), "rb_moe_route_bwd")
    return out


@dataclass
class MoEPlan:
    counts: torch.Tensor        # int32 [E]
    offsets: torch.Tensor       # int32 [E + 1], multiples of 128
    slot_pos: torch.Tensor      # int32 [T * k]
    row_slot: torch.Tensor      # int32 [max_rows], -1 = padding
    tile_expert: torch.Tensor   # int32 [max_rows / 128]
    num_tiles: torch.Tensor     # int32 [1]
    max_rows: int
    num_experts: int
    k: int


def plan(idx: torch.Tensor, num_experts: int) -> MoEPlan:
    T, k = idx.shape
    E = num_experts
    max_rows = (T * k + E * ROW_ALIGN + 127) // 128 * 128
    dev = idx.device
    if not idx.is_cuda:
        flat = idx.reshape(-1).long()
        counts = torch.bincount(flat, minlength=E).to(torch.int32)
        padded = (counts + ROW_ALIGN - 1) // ROW_ALIGN * ROW_ALIGN
        offsets = torch.zeros(E + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(padded, 0)
        order = torch.sort(flat, stable=True).indices           # slots grouped by expert, ascending inside
        rank = torch.arange(T * k) - torch.repeat_interleave(torch.cumsum(counts.long(), 0) - counts.long(), counts.long())
        slot_pos = torch.empty(T * k, dtype=torch.int32)
        slot_pos[order] = (offsets[:-1].long()[flat[order]] + rank).to(torch.int32)
        row_slot = torch.full((max_rows,), -1, dtype=torch.int32)
        row_slot[slot_pos.long()] = torch.arange(T * k, dtype=torch.int32)
        tile_expert = torch.full((max_rows // 128,), -1, dtype=torch.int32)
        ntiles = int(offsets[-1]) // 128
        tile_expert[:ntiles] = torch.repeat_interleave(torch.arange(E, dtype=torch.int32), (padded // 128).long())
        return MoEPlan(counts, offsets, slot_pos, row_slot, tile_expert, torch.tensor([ntiles], dtype=torch.int32), max_rows, E, k)
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
    pl = MoEPlan(i32(E), i32(E + 1), i32(T * k), i32(max_rows), i32(max_rows // 128), i32(1), max_rows, E, k)
    N.check(N.kernels().rb_moe_plan(idx.contiguous().data_ptr(), T, E, k, pl.counts.data_ptr(), pl.offsets.data_ptr(),
                                    pl.slot_pos.data_ptr(), pl.row_slot.data_ptr(), pl.tile_expert.data_ptr(),
                                    pl.num_tiles.data_ptr(), max_rows, N.stream_ptr()), "rb_moe_plan")
    return pl


def gather(x: torch.Tensor, pl: MoEPlan, slot_scale=None) -> torch.Tensor:
    """x [T, d] -> permuted [max_rows, d] (rows past the last expert segment are left untouched / zero)."""
    T, d = x.shape
    if not x.is_cuda:
        xp = torch.zeros((pl.max_rows, d), dtype=x.dtype)
        ok = pl.row_slot >= 0
        src = x[(pl.row_slot[ok] // pl.k).long()].float()
        if slot_scale is not None:
            src = src * slot_scale.reshape(-1)[pl.row_slot[ok].long()][:, None]
        xp[ok] = src.to(x.dtype)
        return xp
    xp = torch.zeros((pl.max_rows, d), dtype=x.dtype, device=x.device)   # rows past the last segment stay zero
    N.check(N.kernels().rb_moe_gather(x.contiguous().data_ptr(), pl.row_slot.data_ptr(), N.ptr(slot_scale), xp.data_ptr(),
                                      pl.max_rows, pl.k, d, pl.offsets[pl.num_experts:].data_ptr(), N.stream_ptr()),
            "rb_moe_gather")
    return xp


def combine(yp: torch.Tensor, pl: MoEPlan, w=None, residual=None) -> torch.Tensor:
    d = yp.shape[1]
    T = pl.slot_pos.numel() // pl.k
    if not yp.is_cuda:
        rows = yp[pl.slot_pos.long()].float().view(T, pl.k, d)
        ww = torch.ones(T, pl.k) if w is None else w.float()
        y = (rows * ww[:, :, None]).sum(1)
        if residual is not None:
            y = y + residual.float()
        return y.to(yp.dtype)
    y = torch.empty((T, d), dtype=yp.dtype, device=yp.device)
    N.check(N.kernels().rb_moe_combine(yp.data_ptr(), pl.slot_pos.data_ptr(), N.ptr(w), N.ptr(residual), y.data_ptr(), T, pl.k, d,
                                       N.stream_ptr()), "rb_moe_combine")
    return y


def weight_grad(dy: torch.Tensor, yp: torch.Tensor, pl: MoEPlan) -> torch.Tensor:
    """dw[t, j] = <dy[t], yp[slot_pos[t*k+j]]>."""
    T, d = dy.shape
    if not dy.is_cuda:
        rows = yp[pl.slot_pos.long()].float().view(T, pl.k, d)
        return (rows * dy.float()[:, None, :]).sum(-1)
    dw = torch.empty((T, pl.k), dtype=torch.float32, device=dy.device)
    N.check(N.kernels().rb_moe_weight_grad(dy.contiguous().data_ptr(), yp.data_ptr(), pl.slot_pos.data_ptr(), dw.data_ptr(), T,
                                           pl.k, d, N.stream_ptr()), "rb_moe_weight_grad")
    return dw


def _segments(pl: MoEPlan):
    off = pl.offsets.tolist()
    cnt = pl.counts.tolist()
    return [(off[e], cnt[e]) for e in range(pl.num_experts)]


def grouped_gemm(xp: torch.Tensor, W: torch.Tensor, pl: MoEPlan, *, b_mn: bool = False, act: str = "none", aux_out=None,
                 aux_in=None, out: torch.Tensor | None = None, arrived=None) -> torch.Tensor:
    """Per-expert matmul over the permuted buffer.  b_mn False: W [E, N, K], y = xp @ W[e]^T.  b_mn True: W [E, K, N]
    (the dgrad form: y = xp @ W[e]).  `arrived` = (counters, expected): int32 device tensors with one entry per
    128-row tile of `xp`; the kernel starts on a tile once its counter has reached the expected number of rows (rows
    that other ranks are still storing into `xp`; see parallel/expert_parallel.py)."""
    E = pl.num_experts
    rows = xp.shape[0]
    Nn = W.shape[2] if b_mn else W.shape[1]
    K = xp.shape[1]
    if not xp.is_cuda:
        y = torch.zeros((rows, Nn), dtype=xp.dtype)
        for e, (o, c) in enumerate(_segments(pl)):
            if c == 0:
                continue
            seg = gemm(xp[o:o + c], W[e], b_mn=b_mn, act=act, aux_in=None if aux_in is None else aux_in[o:o + c],
                       aux_out=None if aux_out is None else aux_out[o:o + c])
            y[o:o + c] = seg
        return y
    y = out if out is not None else torch.empty((rows, Nn), dtype=xp.dtype, device=xp.device)
    W2 = W.reshape(-1, W.shape[2])
    g = N.RbGemmArgs()
    g.a, g.b, g.d = xp.data_ptr(), W2.data_ptr(), y.data_ptr()
    g.aux_in, g.aux_out = N.ptr(aux_in), N.ptr(aux_out)
    g.lda, g.ldb, g.ldd = xp.stride(0), W2.stride(0), y.stride(0)
    g.ld_aux_in = aux_in.stride(0) if aux_in is not None else 0
    g.ld_aux_out = aux_out.stride(0) if aux_out is not None else 0
    g.M, g.N, g.K = rows, Nn, K
    g.a_mn_major, g.b_mn_major = 0, int(b_mn)
    g.act, g.alpha, g.splits = N.ACT[act], 1.0, 1
    g.group_mode, g.num_experts = 1, E
    g.tile_expert, g.num_m_tiles = pl.tile_expert.data_ptr(), pl.num_tiles.data_ptr()
    g.b_expert_rows = W.shape[1]
    if arrived is not None:
        g.tile_arrived, g.tile_expected = arrived[0].data_ptr(), arrived[1].data_ptr()
    N.check(N.kernels().rb_gemm_bf16(g, N.stream_ptr()), "rb_gemm_bf16[grouped]")
    return y


def grouped_wgrad(dyp: torch.Tensor, xp: torch.Tensor, pl: MoEPlan, out: torch.Tensor | None = None,
                  accumulate: bool = False) -> torch.Tensor:
    """dW[e] = dyp[seg_e]^T @ xp[seg_e]  ->  [E, N, K] (fp32 or the dtype of `out`)."""
    E = pl.num_experts
    Nn, K = dyp.shape[1], xp.shape[1]
    if out is None:
        out = torch.zeros((E, Nn, K), dtype=torch.float32, device=xp.device)
        accumulate = False
    if not xp.is_cuda:
        for e, (o, c) in enumerate(_segments(pl)):
            v = dyp[o:o + c].float().t() @ xp[o:o + c].float() if c else torch.zeros(Nn, K)
            out[e] = (out[e].float() + v if accumulate else v).to(out.dtype)
        return out
    g = N.RbGemmArgs()
    g.a, g.b, g.d = dyp.data_ptr(), xp.data_ptr(), out.data_ptr()
    g.lda, g.ldb, g.ldd = dyp.stride(0), xp.stride(0), K
    g.M, g.N, g.K = Nn, K, xp.shape[0]
    g.a_mn_major, g.b_mn_major = 1, 1
    g.out_f32, g.accumulate, g.alpha, g.splits = int(out.dtype == torch.float32), int(accumulate), 1.0, 1
    g.group_mode, g.num_experts = 2, E
    g.expert_offsets = pl.offsets.data_ptr()
    g.d_expert_stride = Nn * K
    N.check(N.kernels().rb_gemm_bf16(g, N.stream_ptr()), "rb_gemm_bf16[grouped wgrad]")
    return out


class _MoEMlpFn(torch.autograd.Function):
    """y = sum_j w_j * Expert_{idx_j}(x) with experts W1 [E, F(or 2F), d], W2 [E, d, F]; returns (y, aux_loss).

    kind "swiglu": W1 stacks gate and up ([E, 2F, d]);  kind "gelu": W1 [E, F, d], tanh-GELU, no biases."""

    @staticmethod
    def forward(ctx, x, router_w, w1, w2, k, kind, renorm):
        T, d = x.shape
        E = router_w.shape[0]
        logits = gemm(x, router_w, out_dtype=torch.float32)
        idx, w, probs = route(logits, k, renorm)
        pl = plan(idx, E)
        xp = gather(x, pl)
        if kind == "swiglu":
            gu = grouped_gemm(xp, w1, pl)
            h = rotary.swiglu_forward(gu)
            saved_pre = gu
        else:
            pre = torch.empty((pl.max_rows, w1.shape[1]), dtype=x.dtype, device=x.device)
            h = grouped_gemm(xp, w1, pl, act="gelu", aux_out=pre)
            saved_pre = pre
        yp = grouped_gemm(h, w2, pl)
        y = combine(yp, pl, w)
        f = pl.counts.float() / float(T * k)
        aux = (f * probs.mean(0)).sum() * E
        ctx.save_for_backward(x, router_w, w1, w2, idx, w, probs, xp, saved_pre, h, yp)
        ctx.pl, ctx.k, ctx.kind, ctx.renorm = pl, k, kind, renorm
        return y, aux

    @staticmethod
    def backward(ctx, dy, daux):
        x, router_w, w1, w2, idx, w, probs, xp, pre, h, yp = ctx.saved_tensors
        pl, k, kind = ctx.pl, ctx.k, ctx.kind
        T, d = x.shape
        dy = dy.contiguous()
        dw = weight_grad(dy, yp, pl)                                   # [T, k]
        dyp = gather(dy, pl, slot_scale=w.reshape(-1).contiguous())      # w_j * dy at every slot
        dw2 = grouped_wgrad(dyp, h, pl)
        dh = grouped_gemm(dyp, w2, pl, b_mn=True)
        if kind == "swiglu":
            dpre = rotary.swiglu_backward(dh, pre)
        else:
            from .elementwise import unary_bwd
            dpre = unary_bwd("gelu", pre, dh)
        dw1 = grouped_wgrad(dpre, xp, pl)
        dxp = grouped_gemm(dpre, w1, pl, b_mn=True)
        dx_experts = combine(dxp, pl, None)
        aux_scale = float(daux) if daux is not None else 0.0
        dlogits = route_backward(probs, idx, w, dw, pl.counts, ctx.renorm, aux_scale)
        dl = dlogits.to(x.dtype)
        dx = gemm(dl, router_w, b_mn=True, out_dtype=x.dtype) if dl.shape[1] % 8 == 0 and x.is_cuda else \
            (dlogits @ router_w.float()).to(x.dtype)
        from .elementwise import binary
        dx = binary("add", dx.contiguous(), dx_experts)
        drw = (dlogits.t() @ x.float()).to(router_w.dtype) if not x.is_cuda or dl.shape[1] % 8 else \
            gemm(dl, x, a_mn=True, b_mn=True, out_dtype=router_w.dtype)
        return dx, drw, dw1.to(w1.dtype), dw2.to(w2.dtype), None, None, None


def moe_mlp(x, router_w, w1, w2, k: int = 2, kind: str = "swiglu", renorm: bool = True):
    """Differentiable top-k expert MLP on [T, d] tokens.  Returns (y [T, d], aux load-balancing loss)."""
    return _MoEMlpFn.apply(x, router_w, w1, w2, k, kind, renorm)
