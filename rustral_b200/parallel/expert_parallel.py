"""Expert parallelism with dispatch and combine over NVLink peer memory.

Experts are split over the ranks of a group (`E / W` consecutive experts per rank, the mapping of the reference's
`ExpertParallel`, crates/nn/src/moe.rs:478-520, which stops at the mapping and moves no tokens).  One layer call does:

  route            local tokens -> top-k experts and weights (ops.moe.route, one kernel)
  plan             every rank learns every rank's per-expert counts (one tiny all-gather of E integers), from which
                   each rank derives, without a host sync, where each of its (token, choice) pairs lands in the owner's
                   receive buffer (expert segments padded to 128 rows, sources in rank order inside a segment) and the
                   tile -> expert table of its own grouped GEMM
  dispatch         `rb_ep_push_rows`: token rows are stored straight into the owner's receive buffer (peer stores);
                   that buffer IS the A operand of the grouped tcgen05 GEMM, there is no intermediate permuted copy.
                   Every stored row adds one to the counter of its 128-row tile on the owner, and the owner's GEMM waits
                   (bounded) per tile until the tile's counter reaches the number of rows the plan expects there, so
                   it works on the tiles that are complete while other ranks are still storing the rest: there is no
                   barrier between dispatch and the first expert GEMM (`RUSTRAL_EP_GRANULAR=0` restores it)
  experts          grouped GEMM -> SwiGLU / GELU -> grouped GEMM on the local experts
  combine          `rb_ep_pull_combine`: every rank pulls its tokens' expert outputs from the owners' output buffers
                   (peer loads) and applies the routing weights in choice order (deterministic)

The backward pass is the mirror image with the same three kernels (push of w * dy, pull of dx, pull-dot for the
routing-weight gradients).  Flags on a signal pad order the phases; every wait is bounded.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import moe as M
from ..ops import rotary
from ..ops.elementwise import unary_bwd, binary
from ..ops.matmul import gemm
from .symm import SignalPad, SymmetricBuffer

P, I = N.c_void_p, N.c_int
N.optional_sig("rb_ep_push_rows", [P, I, I, I, P, P, P, P, P, P])
N.optional_sig("rb_ep_pull_combine", [P, I, I, I, P, P, P, P, P, P])
N.optional_sig("rb_ep_pull_dot", [P, P, I, I, I, P, P, P, P])
N.optional_sig("rb_ep_zero_padding", [P, P, P, I, I, P])


@dataclass
class EPPlan:
    dest_rank: torch.Tensor       # int32 [T * k]
    dest_row: torch.Tensor        # int32 [T * k]
    counts_global: torch.Tensor   # int32 [E]: tokens per expert over all ranks (for the load-balancing loss)
    recv: M.MoEPlan               # grouped-GEMM plan of this rank's receive buffer (local experts)
    tokens: int
    k: int
    dropped: torch.Tensor | None = None   # number of this rank's (token, choice) pairs beyond the capacity (device scalar)
    tile_rows: torch.Tensor | None = None  # int32 [cap / 128]: rows every 128-row tile of the receive buffer is going to get


class FusedEP:
    """Buffers and flags of one expert-parallel group.  `max_tokens` is the largest number of local tokens of a call.
    Without a `capacity_factor` the receive buffers hold the worst case (every pair of every rank routed here) and no
    token is ever dropped; with one they hold `capacity_factor * max_tokens * k` rows (the balanced share times the
    factor) and pairs that would land beyond that are dropped, on every rank alike (`EPPlan.dropped` counts them)."""

    def __init__(self, group, device, num_experts: int, d_model: int, max_tokens: int, k: int, limit_ms: int = 5000,
                 capacity_factor: float | None = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("the number of experts must be divisible by the expert-parallel size")
        self.device = torch.device(device)
        self.E, self.El, self.d, self.k = num_experts, num_experts // self.world, d_model, k
        self.limit_ms = limit_ms
        rows = self.world * max_tokens * k if capacity_factor is None else int(capacity_factor * max_tokens * k)
        cap = min(rows, self.world * max_tokens * k) + self.El * M.ROW_ALIGN
        self.cap = (cap + 127) // 128 * 128
        nbytes = self.cap * d_model * 2
        self.pad = SignalPad(group, self.device)
        # x in / y out (forward), dy in / dx out (backward); all peer-visible
        self.bufs = {name: SymmetricBuffer(nbytes, group, self.device) for name in ("x", "y", "dy", "dx")}
        # rows arrived per 128-row tile of the two buffers that peers push into
        self.granular = __import__("os").environ.get("RUSTRAL_EP_GRANULAR", "1") != "0"
        self.counts = {name: SymmetricBuffer(4 * (self.cap // 128), group, self.device) for name in ("x", "dy")}
        self.epoch = 0

    def view(self, name: str) -> torch.Tensor:
        return self.bufs[name].view(torch.bfloat16, self.cap * self.d).view(self.cap, self.d)

    def sync(self) -> None:
        """All ranks' work enqueued so far is complete before any rank's later work starts."""
        self.epoch += 1
        self.pad.signal_all(0, self.epoch)
        self.pad.wait_all(0, self.epoch, self.limit_ms)

    # ---------------------------------------------------------------------------------------------- planning
    def plan(self, idx: torch.Tensor) -> EPPlan:
        T, k = idx.shape
        W, El, E = self.world, self.El, self.E
        local = M.plan(idx, E)
        table = torch.empty((W, E), dtype=torch.int32, device=idx.device)
        dist.all_gather_into_tensor(table, local.counts, group=self.group)
        table = table.long()
        seg = table.sum(0)                                             # rows per expert over all sources
        padded = (seg + 127) // 128 * 128
        pr = padded.view(W, El)
        off = (torch.cumsum(pr, 1) - pr).reshape(-1)                   # segment start inside its owner's buffer
        base = off + table[:self.rank].sum(0)                          # this rank's rows start after lower ranks' rows
        e = idx.reshape(-1).long()
        pos = local.slot_pos.long() - local.offsets.long()[e]          # position inside this rank's group for expert e
        row = base[e] + pos
        fits = row < self.cap                                         # the same answer on every rank
        dest_row = torch.where(fits, row, torch.full_like(row, -1)).to(torch.int32)
        dest_rank = (e // El).to(torch.int32)
        dropped = (~fits).sum()
        # receive side (segments cut at the capacity)
        recv_off = torch.zeros(El + 1, dtype=torch.int64, device=idx.device)
        recv_off[1:] = torch.cumsum(pr[self.rank], 0)
        recv_off = recv_off.clamp(max=self.cap)
        my_counts = torch.minimum(seg.view(W, El)[self.rank], self.cap - recv_off[:-1]).clamp(min=0).to(torch.int32)
        tiles = torch.arange(self.cap // 128, device=idx.device) * 128
        te = torch.bucketize(tiles, recv_off[1:], right=True)
        tile_expert = torch.where(tiles < recv_off[-1], te, torch.full_like(te, -1)).to(torch.int32)
        num_tiles = (recv_off[-1:] // 128).to(torch.int32)
        recv = M.MoEPlan(my_counts, recv_off.to(torch.int32), None, None, tile_expert, num_tiles, self.cap, El, k)
        # rows each tile receives: the part of its expert's segment [start, start + count) that falls into the tile
        seg_end = recv_off[:-1] + my_counts.long()
        tile_rows = (seg_end[te.clamp(max=El - 1)] - tiles).clamp(min=0, max=128)
        tile_rows = torch.where(tiles < recv_off[-1], tile_rows, torch.zeros_like(tile_rows)).to(torch.int32)
        return EPPlan(dest_rank, dest_row, seg.to(torch.int32), recv, T, k, dropped, tile_rows)

    # ---------------------------------------------------------------------------------------------- transport
    def push(self, src: torch.Tensor, pl: EPPlan, to: str, scale=None):
        """Rows of `src` [T, d] into the owners' buffer `to`.  Returns (this rank's buffer, arrived): with tile-granular
        dispatch `arrived` = (counters, expected rows) for the first grouped GEMM that reads the buffer, which waits per
        tile, and the buffer is complete only once that GEMM has run; otherwise `arrived` is None and the buffer is
        complete on return."""
        cnt = self.counts[to]
        counters = cnt.view(torch.int32, self.cap // 128)
        if self.granular:
            counters.zero_()                          # before the barrier: nobody adds to them until it has passed
        self.sync()                                   # the owners are done with the previous contents
        buf = self.bufs[to]
        N.check(N.kernels().rb_ep_push_rows(src.contiguous().data_ptr(), pl.tokens, pl.k, self.d, pl.dest_rank.data_ptr(),
                                            pl.dest_row.data_ptr(), N.ptr(scale), buf.ptrs_dev.data_ptr(),
                                            cnt.ptrs_dev.data_ptr() if self.granular else None, N.stream_ptr()),
                "rb_ep_push_rows")
        if not self.granular:
            self.sync()                               # every rank's rows have landed
        mine = self.view(to)
        # the padding rows of every expert segment are this rank's to clear (no peer writes them)
        N.check(N.kernels().rb_ep_zero_padding(mine.data_ptr(), pl.recv.offsets.data_ptr(), pl.recv.counts.data_ptr(),
                                               self.El, self.d, N.stream_ptr()), "rb_ep_zero_padding")
        return mine, ((counters, pl.tile_rows) if self.granular else None)

    def pull(self, pl: EPPlan, frm: str, w=None, residual=None, synced: bool = False) -> torch.Tensor:
        if not synced:
            self.sync()                               # the owners' outputs are complete
        out = torch.empty((pl.tokens, self.d), dtype=torch.bfloat16, device=self.device)
        N.check(N.kernels().rb_ep_pull_combine(out.data_ptr(), pl.tokens, pl.k, self.d, pl.dest_rank.data_ptr(),
                                               pl.dest_row.data_ptr(), N.ptr(w), N.ptr(residual),
                                               self.bufs[frm].ptrs_dev.data_ptr(), N.stream_ptr()), "rb_ep_pull_combine")
        return out

    def pull_dot(self, dy: torch.Tensor, pl: EPPlan, frm: str) -> torch.Tensor:
        dw = torch.empty((pl.tokens, pl.k), dtype=torch.float32, device=self.device)
        N.check(N.kernels().rb_ep_pull_dot(dw.data_ptr(), dy.contiguous().data_ptr(), pl.tokens, pl.k, self.d,
                                           pl.dest_rank.data_ptr(), pl.dest_row.data_ptr(),
                                           self.bufs[frm].ptrs_dev.data_ptr(), N.stream_ptr()), "rb_ep_pull_dot")
        return dw

    def close(self) -> None:
        for b in list(self.bufs.values()) + list(self.counts.values()):
            b.close()
        self.pad.close()


class _EPMoEMlpFn(torch.autograd.Function):
    """y = sum_j w_j Expert_{idx_j}(x) with the experts spread over the group; w1 [E_local, F or 2F, d], w2 [E_local, d, F]."""

    @staticmethod
    def forward(ctx, x, router_w, w1, w2, k, kind, renorm, ep: FusedEP):
        T, d = x.shape
        E = router_w.shape[0]
        logits = gemm(x, router_w, out_dtype=torch.float32)
        idx, w, probs = M.route(logits, k, renorm)
        pl = ep.plan(idx)
        xp, arrived = ep.push(x, pl, "x")
        if kind == "swiglu":
            pre = M.grouped_gemm(xp, w1, pl.recv, arrived=arrived)
            h = rotary.swiglu_forward(pre)
        else:
            pre = torch.empty((ep.cap, w1.shape[1]), dtype=x.dtype, device=x.device)
            h = M.grouped_gemm(xp, w1, pl.recv, act="gelu", aux_out=pre, arrived=arrived)
        M.grouped_gemm(h, w2, pl.recv, out=ep.view("y"))
        y = ep.pull(pl, "y", w=w)
        f = pl.counts_global.float() / float(max(1, T * k * ep.world))
        aux = (f * probs.mean(0)).sum() * E
        # xp and yp live in buffers that the next layer overwrites: keep copies for the backward pass
        ctx.save_for_backward(x, router_w, w1, w2, idx, w, probs, xp.clone(), pre, h)
        ctx.pl, ctx.k, ctx.kind, ctx.renorm, ctx.ep = pl, k, kind, renorm, ep
        return y, aux

    @staticmethod
    def backward(ctx, dy, daux):
        x, router_w, w1, w2, idx, w, probs, xp, pre, h = ctx.saved_tensors
        pl, k, kind, ep = ctx.pl, ctx.k, ctx.kind, ctx.ep
        dy = dy.contiguous()
        # the owners recompute their expert outputs for the routing-weight gradient
        ep.sync()
        M.grouped_gemm(h, w2, pl.recv, out=ep.view("y"))
        dyp, arrived = ep.push(dy, pl, "dy", scale=w.reshape(-1).contiguous())  # w_j * dy at every slot
        dh = M.grouped_gemm(dyp, w2, pl.recv, b_mn=True, arrived=arrived)        # waits per tile; dyp is complete after it
        dw2 = M.grouped_wgrad(dyp, h, pl.recv)
        dpre = rotary.swiglu_backward(dh, pre) if kind == "swiglu" else unary_bwd("gelu", pre, dh)
        dw1 = M.grouped_wgrad(dpre, xp, pl.recv)
        M.grouped_gemm(dpre, w1, pl.recv, b_mn=True, out=ep.view("dx"))
        dx_experts = ep.pull(pl, "dx")                                           # barrier inside: the owners' y and dx are complete
        dw = ep.pull_dot(dy, pl, "y")                                            # [T, k]
        aux_scale = float(daux) if daux is not None else 0.0
        T = x.shape[0]
        # load-balancing term: f uses the global counts, scaled to the local token count convention of route_backward
        counts_local_equiv = (pl.counts_global.float() / ep.world).to(torch.int32)
        dlogits = M.route_backward(probs, idx, w, dw, counts_local_equiv, ctx.renorm, aux_scale)
        dl = dlogits.to(x.dtype)
        if dl.shape[1] % 8 == 0:
            dx = gemm(dl, router_w, b_mn=True, out_dtype=x.dtype)
            drw = gemm(dl, x, a_mn=True, b_mn=True, out_dtype=router_w.dtype)
        else:
            dx = (dlogits @ router_w.float()).to(x.dtype)
            drw = (dlogits.t() @ x.float()).to(router_w.dtype)
        dx = binary("add", dx.contiguous(), dx_experts)
        return dx, drw, dw1.to(w1.dtype), dw2.to(w2.dtype), None, None, None, None


def ep_moe_mlp(x, router_w, w1_local, w2_local, ep: FusedEP, k: int = 2, kind: str = "swiglu", renorm: bool = True):
    """Differentiable expert-parallel top-k MLP on this rank's [T, d] tokens.  Returns (y, aux load-balancing loss).
    The router weight gradient is local (sum it over the data-parallel group like any replicated parameter); the
    expert weight gradients already contain every rank's tokens."""
    return _EPMoEMlpFn.apply(x, router_w, w1_local, w2_local, k, kind, renorm, ep)
