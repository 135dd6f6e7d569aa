"""Tensor-parallel GEMMs fused with their collectives over NVLink peer memory.

Two primitives, both one launch of the tcgen05 GEMM (csrc/kernels/gemm_tcgen05.cu, `peer_mode` 1 and 2):

* ``ag_gemm``  : ``Y[M, N] = act(allgather_rows(X_local) @ W^T + b)``.  Every rank publishes its row shard
  ``X_local[M / W, K]`` in symmetric memory.  Inside the GEMM the epilogue warps first pull the remote 128-row
  blocks of X over NVLink into a local ``[M, K]`` buffer (plain peer loads, in the order the tiles will be
  consumed), raise a per-block flag, and the TMA producer of whichever CTA needs a block waits for that flag.
  The tile schedule starts at the rank's own rows, so tensor-core work begins at once and the transfer of the
  other rows hides behind it.
* ``gemm_rs``  : ``Y_local[M / W, N] = reduce_scatter_rows(X @ W^T) (+ residual)``.  The epilogue stores every
  output row block straight into the receive slot of the rank that owns those rows (peer stores from the TMEM
  read-back, no intermediate full-size product); after one flag exchange a small kernel adds the W slots in
  rank order in fp32, so the result is bit-identical on every run.

No TMA descriptor ever covers a peer's memory: remote data moves with ordinary loads and stores, TMA only reads
this GPU's buffers.  Each primitive double-buffers its symmetric workspace by call parity; together with the
flag exchange before (ag) or after (rs) the kernel this is enough to keep a fast rank from overwriting data a
slow rank still reads.

The reference's tensor parallelism is forward-only over host slices (crates/distributed/src/tensor_parallel.rs:125-241);
it has no fused communication kernels.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops.elementwise import unary_bwd
from ..ops.matmul import gemm
from .symm import SignalPad, SymmetricBuffer

N.optional_sig("rb_tp_reduce_slots", [N.c_void_p, N.c_int, N.c_ll, N.c_void_p, N.c_void_p, N.c_void_p])

ROW_BLOCK = 128


class _AgWorkspace:
    def __init__(self, ctx: "FusedTP", rows: int, k: int, channel: int):
        self.shard = [SymmetricBuffer(rows * k * 2, ctx.group, ctx.device) for _ in range(2)]
        self.a_full = torch.empty((rows * ctx.world, k), dtype=torch.bfloat16, device=ctx.device)
        self.flags = torch.zeros(rows * ctx.world // ROW_BLOCK, dtype=torch.int32, device=ctx.device)
        self.epoch = 0
        self.channel = channel


class _RsWorkspace:
    def __init__(self, ctx: "FusedTP", rows: int, n: int, channel: int):
        self.slots = [SymmetricBuffer(ctx.world * rows * n * 2, ctx.group, ctx.device) for _ in range(2)]
        self.epoch = 0
        self.channel = channel


class WeightShard:
    """A row shard [N / W, K] of a weight that lives in symmetric memory (so peers can pull it from inside a GEMM),
    with this rank's landing buffer for the gathered [N, K] weight and its per-block counters."""

    def __init__(self, ctx: "FusedTP", rows: int, k: int, channel: int, full: torch.Tensor | None = None):
        self.rows, self.k = rows, k
        self.buf = SymmetricBuffer(rows * k * 2, ctx.group, ctx.device)
        self.tensor = self.buf.view(torch.bfloat16, rows * k).view(rows, k)
        # landing buffer of the gathered weight: private, or one shared by every shard of this shape (`pooled`), in
        # which case it only holds this weight until the next gather of that shape
        self.pooled = full is not None
        self.full = full if full is not None else torch.empty((rows * ctx.world, k), dtype=torch.bfloat16, device=ctx.device)
        self.flags = torch.zeros(rows * ctx.world // ROW_BLOCK, dtype=torch.int32, device=ctx.device)
        self.epoch = 0
        self.channel = channel


class FusedTP:
    """Workspaces and flags of the fused tensor-parallel GEMMs for one tensor-parallel group.

    Workspaces are created on first use for each (rows per rank, width) pair; creation is collective, so every
    rank must issue the same sequence of calls (which tensor-parallel layers do by construction)."""

    def __init__(self, group=None, device=None, limit_ms: int = 5000):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.limit_ms = limit_ms
        self.pad = SignalPad(group, self.device)
        self._ws: dict = {}
        self._full_pool: dict = {}

    def _workspace(self, kind: str, rows: int, width: int):
        key = (kind, rows, width)
        ws = self._ws.get(key)
        if ws is None:
            channel = len(self._ws)
            if (channel + 1) * self.world * 4 > self.pad.nbytes:
                raise N.NativeError("FusedTP: out of signal channels")
            ws = (_AgWorkspace if kind == "ag" else _RsWorkspace)(self, rows, width, channel)
            self._ws[key] = ws
        return ws

    def supports(self, rows_per_rank: int) -> bool:
        return rows_per_rank > 0 and rows_per_rank % ROW_BLOCK == 0

    # ------------------------------------------------------------------------------------------ all-gather -> GEMM
    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None, act: str = "none",
                aux_out=None, out=None):
        """Returns (Y[M, N], X_full[M, K]).  X_full is the workspace the kernel gathered into: valid until the next
        ag_gemm call with the same (rows, K); clone it to keep it.  `w` is [N, K], or [K, N] with `b_mn`."""
        rows, k = x_local.shape
        if not self.supports(rows):
            raise ValueError(f"ag_gemm: rows per rank ({rows}) must be a multiple of {ROW_BLOCK}")
        ws = self._workspace("ag", rows, k)
        ws.epoch += 1
        par = ws.epoch & 1
        shard = ws.shard[par].view(torch.bfloat16, rows * k).view(rows, k)
        shard.copy_(x_local)
        ws.a_full[self.rank * rows:(self.rank + 1) * rows].copy_(x_local)
        # every rank's shard is in place before any rank's kernel reads it
        self.pad.signal_all(ws.channel, ws.epoch)
        self.pad.wait_all(ws.channel, ws.epoch, self.limit_ms)
        y = gemm(ws.a_full, w, b_mn=b_mn, bias=bias, act=act, aux_out=aux_out, out=out, out_dtype=torch.bfloat16,
                 peer={"mode": 1, "world": self.world, "rank": self.rank, "rows_per_rank": rows, "epoch": ws.epoch,
                       "ready_flags": ws.flags.data_ptr(), "peer_ptrs": ws.shard[par].peer_ptrs})
        return y, ws.a_full

    # ------------------------------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, residual=None, out=None):
        """Y_local[M / W, N] = sum over ranks of (X_r @ W_r^T)[own rows] (+ residual).  `x` is [M, K_local]
        (or [K_local, M] with `a_mn`)."""
        m = x.shape[1] if a_mn else x.shape[0]
        n = w.shape[1] if b_mn else w.shape[0]
        if m % self.world or not self.supports(m // self.world):
            raise ValueError(f"gemm_rs: M / world ({m} / {self.world}) must be a multiple of {ROW_BLOCK}")
        rows = m // self.world
        ws = self._workspace("rs", rows, n)
        ws.epoch += 1
        par = ws.epoch & 1
        slots = ws.slots[par]
        local_view = slots.view(torch.bfloat16, m * n).view(m, n)
        gemm(x, w, a_mn=a_mn, b_mn=b_mn, out=local_view,
             peer={"mode": 2, "world": self.world, "rank": self.rank, "rows_per_rank": rows, "epoch": ws.epoch,
                   "ready_flags": None, "peer_ptrs": slots.peer_ptrs})
        # every rank's partial rows have landed in this rank's slots
        self.pad.signal_all(ws.channel, ws.epoch)
        self.pad.wait_all(ws.channel, ws.epoch, self.limit_ms)
        if out is None:
            out = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)
        N.check(N.kernels().rb_tp_reduce_slots(slots.local_ptr, self.world, rows * n, N.ptr(residual), out.data_ptr(),
                                               N.stream_ptr()), "rb_tp_reduce_slots")
        return out

    # ------------------------------------------------------------------------------------------ weight all-gather -> GEMM
    def shard_weight(self, w_shard: torch.Tensor, pooled: bool = False) -> WeightShard:
        """Moves this rank's row shard of a weight into symmetric memory (collective; same order on every rank).
        `pooled`: all shards of one shape share a single landing buffer for the gathered weight, so a rank holds one
        gathered weight per shape instead of one per layer (the backward pass gathers again)."""
        rows, k = w_shard.shape
        if not self.supports(rows):
            raise ValueError(f"shard_weight: rows per rank ({rows}) must be a multiple of {ROW_BLOCK}")
        key = ("w", len(self._ws))
        channel = len(self._ws)
        if (channel + 1) * self.world * 4 > self.pad.nbytes:
            raise N.NativeError("FusedTP: out of signal channels")
        full = None
        if pooled:
            full = self._full_pool.get((rows, k))
            if full is None:
                full = torch.empty((rows * self.world, k), dtype=torch.bfloat16, device=self.device)
                self._full_pool[(rows, k)] = full
        ws = WeightShard(self, rows, k, channel, full)
        ws.tensor.copy_(w_shard)
        self._ws[key] = ws
        return ws

    def fsdp_gemm(self, x: torch.Tensor, ws: WeightShard, *, bias=None, act: str = "none", aux_out=None, out=None):
        """Y[M, N] = act(X @ allgather_rows(W_shard)^T + b): the ZeRO-3 / FSDP parameter all-gather fused into the GEMM
        that consumes it.  Returns (Y, W_full); W_full stays valid until the next call with the same shard."""
        ws.epoch += 1
        ws.full[self.rank * ws.rows:(self.rank + 1) * ws.rows].copy_(ws.tensor)
        # every rank has finished writing its shard (optimizer step) before any rank pulls it
        self.pad.signal_all(ws.channel, ws.epoch)
        self.pad.wait_all(ws.channel, ws.epoch, self.limit_ms)
        y = gemm(x, ws.full, bias=bias, act=act, aux_out=aux_out, out=out, out_dtype=torch.bfloat16,
                 peer={"mode": 3, "world": self.world, "rank": self.rank, "rows_per_rank": ws.rows, "epoch": ws.epoch,
                       "ready_flags": ws.flags.data_ptr(), "peer_ptrs": ws.buf.peer_ptrs})
        return y, ws.full

    def close(self) -> None:
        for ws in self._ws.values():
            if isinstance(ws, WeightShard):
                ws.buf.close()
                continue
            for buf in (ws.shard if isinstance(ws, _AgWorkspace) else ws.slots):
                buf.close()
        self._ws = {}
        self.pad.close()


class ColumnSeqParallelFn(torch.autograd.Function):
    """y[M, n_local] = act(allgather_rows(x_local) W^T + b); the backward pass is the mirrored GEMM -> reduce-scatter."""

    @staticmethod
    def forward(ctx, x_local, w, bias, act, tp: FusedTP):
        need_pre = act != "none"
        M = x_local.shape[0] * tp.world
        pre = torch.empty((M, w.shape[0]), dtype=torch.bfloat16, device=w.device) if need_pre else None
        y, x_full = tp.ag_gemm(x_local, w, bias=bias, act=act, aux_out=pre)
        ctx.save_for_backward(x_full.clone(), w, pre)
        ctx.act, ctx.tp, ctx.has_bias = act, tp, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w, pre = ctx.saved_tensors
        dy = dy.contiguous()
        dz = unary_bwd(ctx.act, pre, dy) if pre is not None else dy
        dw = gemm(dz, x_full, a_mn=True, b_mn=True, out_dtype=torch.bfloat16)      # [n_local, K] = dz^T x
        db = dz.float().sum(0).to(dz.dtype) if ctx.has_bias else None
        dx_local = ctx.tp.gemm_rs(dz, w, b_mn=True)                                # rows of dz @ W, summed over ranks
        return dx_local, dw, db, None, None


class RowSeqParallelFn(torch.autograd.Function):
    """y_local[M / W, N] = reduce_scatter_rows(x W^T) (+ residual); backward is all-gather -> GEMM."""

    @staticmethod
    def forward(ctx, x, w, residual, tp: FusedTP):
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.has_res = tp, residual is not None
        return tp.gemm_rs(x, w, residual=residual)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        dy_local = dy_local.contiguous()
        dx, dy_full = ctx.tp.ag_gemm(dy_local, w, b_mn=True)                       # [M, k_local] = allgather(dy) @ W
        dw = gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=torch.bfloat16)      # [N, k_local] = dy^T x
        return dx, dw, (dy_local if ctx.has_res else None), None


class FSDPLinearFn(torch.autograd.Function):
    """y = act(x W^T + b) with W row-sharded over the data-parallel ranks (FSDP / ZeRO-3).

    Forward: the parameter all-gather runs inside the GEMM (peer mode 3).  Backward: dx uses the gathered weight the
    forward left in this rank's landing buffer; the weight gradient dW = dy^T x is reduce-scattered from inside its
    GEMM (peer mode 2), so each rank ends with the summed gradient of its own shard.  Returns dW for `w_shard_param`
    (a tensor of the shard's shape that only carries the gradient)."""

    @staticmethod
    def forward(ctx, x, w_shard_param, bias, act, tp: FusedTP, ws: WeightShard):
        x2 = x.reshape(-1, x.shape[-1])
        need_pre = act != "none"
        pre = torch.empty((x2.shape[0], ws.rows * tp.world), dtype=torch.bfloat16, device=x.device) if need_pre else None
        y, w_full = tp.fsdp_gemm(x2, ws, bias=bias, act=act, aux_out=pre)
        ctx.save_for_backward(x2, pre)
        ctx.w_full, ctx.act, ctx.tp, ctx.has_bias, ctx.x_shape, ctx.ws = w_full, act, tp, bias is not None, x.shape, ws
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dz = unary_bwd(ctx.act, pre, dy2) if pre is not None else dy2
        if ctx.ws.pooled:
            # the shared landing buffer has been reused since the forward pass: gather this weight again
            dist.all_gather_into_tensor(ctx.w_full, ctx.ws.tensor.detach(), group=ctx.tp.group)
        dx = gemm(dz, ctx.w_full, b_mn=True, out_dtype=torch.bfloat16)                # [M, K] = dz @ W
        dw_shard = ctx.tp.gemm_rs(dz, x2, a_mn=True, b_mn=True)                       # rows of dz^T x, summed over ranks
        db = dz.float().sum(0).to(dz.dtype) if ctx.has_bias else None
        return dx.reshape(ctx.x_shape), dw_shard, db, None, None, None
