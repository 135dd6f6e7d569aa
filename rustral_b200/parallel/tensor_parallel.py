"""Tensor parallelism (crates/distributed/src/tensor_parallel.rs:28-375).

Column-parallel linears shard the output features (each rank owns out/W rows of W), row-parallel linears shard the
input features (each rank owns in/W columns and produces a partial sum).  Between a column- and a row-parallel
pair the activation stays sharded by features; with `sequence_parallel=True` the activations OUTSIDE the pair are
sharded by sequence, so the collectives become all-gather (before the column layer) and reduce-scatter (after the
row layer) instead of one all-reduce.

Differences from the reference, on purpose: both layers are differentiable (the reference is forward-only), each
rank initialises ITS shard of one global weight (the reference seeds every rank identically, tensor_parallel.rs:74-75),
and the column-parallel gather concatenates along the feature dimension (the reference concatenates rank-major and
reshapes, which scrambles batches larger than one, :139-149).
"""
from __future__ import annotations

import enum

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, InvalidArgument
from .process_group import ProcessGroup


class ParallelStyle(enum.Enum):
    COLUMN = "column"
    ROW = "row"


class _AllGatherLastDim(torch.autograd.Function):
    """Forward: concatenate feature shards; backward: keep this rank's slice."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return torch.cat(pg.all_gather(x.contiguous()), -1)

    @staticmethod
    def backward(ctx, g):
        n = g.shape[-1] // ctx.pg.world_size
        return g[..., ctx.pg.rank * n:(ctx.pg.rank + 1) * n].contiguous(), None


class _AllReduce(torch.autograd.Function):
    """Forward: sum over ranks; backward: identity (every rank gets the same upstream gradient)."""

    @staticmethod
    def forward(ctx, x, pg):
        y = x.clone()
        pg.all_reduce_sum(y, "tp_row")
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """Forward: identity; backward: sum the input gradients of all ranks (entry of a column-parallel region)."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return x

    @staticmethod
    def backward(ctx, g):
        y = g.clone()
        ctx.pg.all_reduce_sum(y, "tp_copy_bwd")
        return y, None


class _GatherSeq(torch.autograd.Function):
    """Sequence-parallel entry: all-gather along dim 0 forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return torch.cat(pg.all_gather(x.contiguous()), 0)

    @staticmethod
    def backward(ctx, g):
        return ctx.pg.reduce_scatter(g.contiguous()), None


class _ReduceScatterSeq(torch.autograd.Function):
    """Sequence-parallel exit: reduce-scatter along dim 0 forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return pg.reduce_scatter(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return torch.cat(ctx.pg.all_gather(g.contiguous()), 0), None


class TensorParallelLinear(Module, Trainable, Saveable):
    """Parameter names: weight (the local shard), bias (column: local slice; row: full, added once)."""

    def __init__(self, style: ParallelStyle, weight: Parameter, bias, process_group: ProcessGroup, in_dim: int, out_dim: int,
                 gather_output: bool = False, input_is_parallel: bool = True, sequence_parallel: bool = False,
                 activation: str = "none"):
        self.fused_tp = None     # a parallel.fused_tp.FusedTP: sequence-parallel layers then run the fused kernels
        self.style, self.weight, self.bias, self._pg = style, weight, bias, process_group
        self.in_dim, self.out_dim = in_dim, out_dim
        self.gather_output, self.input_is_parallel, self.sequence_parallel = gather_output, input_is_parallel, sequence_parallel
        self.activation = activation

    @staticmethod
    def _full_weight(backend, in_dim, out_dim, seed, scale):
        g = torch.Generator().manual_seed(seed)
        return torch.randn(out_dim, in_dim, generator=g) * scale

    @classmethod
    def column_parallel(cls, backend, in_dim: int, out_dim: int, pg: ProcessGroup, bias: bool = False, seed: int = 42,
                        scale: float = 0.02, gather_output: bool = False, sequence_parallel: bool = False, activation="none"):
        W, r = pg.world_size, pg.rank
        if out_dim % W:
            raise InvalidArgument("out_dim must be divisible by the tensor-parallel size")
        n = out_dim // W
        w = cls._full_weight(backend, in_dim, out_dim, seed, scale)[r * n:(r + 1) * n]
        wp = Parameter("weight", w.to(backend.device(), backend.dtype))
        bp = backend.constant_parameter("bias", (n,), 0.0) if bias else None
        return cls(ParallelStyle.COLUMN, wp, bp, pg, in_dim, out_dim, gather_output, True, sequence_parallel, activation)

    @classmethod
    def row_parallel(cls, backend, in_dim: int, out_dim: int, pg: ProcessGroup, bias: bool = False, seed: int = 42,
                     scale: float = 0.02, input_is_parallel: bool = True, sequence_parallel: bool = False):
        W, r = pg.world_size, pg.rank
        if in_dim % W:
            raise InvalidArgument("in_dim must be divisible by the tensor-parallel size")
        n = in_dim // W
        w = cls._full_weight(backend, in_dim, out_dim, seed, scale)[:, r * n:(r + 1) * n].contiguous()
        wp = Parameter("weight", w.to(backend.device(), backend.dtype))
        bp = backend.constant_parameter("bias", (out_dim,), 0.0) if bias else None
        return cls(ParallelStyle.ROW, wp, bp, pg, in_dim, out_dim, False, input_is_parallel, sequence_parallel)

    def use_fused(self, fused_tp) -> "TensorParallelLinear":
        """Route the sequence-parallel forward and backward through the fused all-gather->GEMM / GEMM->reduce-scatter
        kernels of `fused_tp` (CUDA, rows per rank a multiple of 128; other inputs keep the collective path)."""
        self.fused_tp = fused_tp
        return self

    def _fused_forward(self, x, residual):
        from .fused_tp import ColumnSeqParallelFn, RowSeqParallelFn
        tp = self.fused_tp
        b = None if self.bias is None else self.bias.tensor
        x2 = x.reshape(-1, x.shape[-1])
        if self.style is ParallelStyle.COLUMN:
            y = ColumnSeqParallelFn.apply(x2, self.weight.tensor, b, self.activation, tp)
            return y.reshape(x.shape[0] * tp.world, *x.shape[1:-1], y.shape[-1])
        res2 = None
        if residual is not None and b is None:
            res2 = residual.reshape(-1, residual.shape[-1])
        y = RowSeqParallelFn.apply(x2, self.weight.tensor, res2, tp)
        y = y.reshape(x.shape[0] // tp.world, *x.shape[1:-1], y.shape[-1])
        if b is not None:
            y = y + b
            if residual is not None:
                y = y + residual
        return y

    def _can_fuse(self, x) -> bool:
        if self.fused_tp is None or not self.sequence_parallel or not x.is_cuda or x.dtype != torch.bfloat16:
            return False
        rows = x.numel() // x.shape[-1]
        if self.style is ParallelStyle.COLUMN:
            return self.fused_tp.supports(rows)
        return self.input_is_parallel and rows % self.fused_tp.world == 0 and self.fused_tp.supports(rows // self.fused_tp.world)

    def forward(self, x, ctx: ForwardCtx | None = None, residual=None):
        pg = self._pg
        if self._can_fuse(x):
            return self._fused_forward(x, residual)
        b = None if self.bias is None else self.bias.tensor
        if self.style is ParallelStyle.COLUMN:
            x = _GatherSeq.apply(x, pg) if self.sequence_parallel else _CopyToTP.apply(x, pg)
            y = ops.linear(x, self.weight.tensor, b, self.activation)
            return _AllGatherLastDim.apply(y, pg) if self.gather_output else y
        if not self.input_is_parallel:
            n = self.in_dim // pg.world_size
            x = x[..., pg.rank * n:(pg.rank + 1) * n].contiguous()
        y = ops.linear(x, self.weight.tensor, None)
        y = _ReduceScatterSeq.apply(y, pg) if self.sequence_parallel else _AllReduce.apply(y, pg)
        if b is not None:
            y = y + b
        if residual is not None:
            y = y + residual
        return y

    def __call__(self, x, ctx=None, residual=None):
        return self.forward(x, ctx, residual)

    def _children(self):
        yield "weight", self.weight
        if self.bias is not None:
            yield "bias", self.bias


class AllGatherOp:
    def __init__(self, pg: ProcessGroup, dim: int = -1):
        self.pg, self.dim = pg, dim

    def execute(self, t):
        return torch.cat(self.pg.all_gather(t.contiguous()), self.dim)


class AllReduceOp:
    def __init__(self, pg: ProcessGroup, op: str = "sum"):
        self.pg, self.op = pg, op

    def execute(self, t):
        if self.op == "max":
            return torch.stack(self.pg.all_gather(t)).amax(0)
        y = t.clone()
        self.pg.all_reduce_sum(y)
        return y / self.pg.world_size if self.op == "mean" else y


def _vocab_parallel_cross_entropy_cuda(local_logits, targets, pg: ProcessGroup, vocab_start: int):
    """CUDA path: the fused loss kernel yields this shard's log-sum-exp and target logit per row, two small
    collectives combine them over the ranks, a second kernel writes (softmax - onehot) for this shard."""
    from .. import _native as N
    from ..ops.loss import cross_entropy_fwd_bwd
    rows, n = local_logits.shape
    local_t = targets.to(torch.int64) - vocab_start
    mine = (local_t >= 0) & (local_t < n)
    t_masked = torch.where(mine, local_t, torch.full_like(local_t, -100))
    loss_l, lse_l, _ = cross_entropy_fwd_bwd(local_logits, t_masked, want_grad=False)      # loss = lse - z_target (owned rows)
    target_logit = torch.where(mine, lse_l - loss_l, torch.zeros_like(lse_l))
    lse = torch.logsumexp(torch.stack(pg.all_gather(lse_l)), 0)
    pg.all_reduce_sum(target_logit, "vp_target")
    grad = torch.empty_like(local_logits)
    N.optional_sig("rb_cross_entropy_grad_lse", [N.c_void_p, N.c_ll, N.c_void_p, N.c_void_p, N.c_void_p, N.c_ll, N.c_int,
                                                 N.c_int, N.c_float, N.c_void_p])
    N.check(N.kernels().rb_cross_entropy_grad_lse(local_logits.data_ptr(), local_logits.stride(0), t_masked.data_ptr(),
                                                  lse.data_ptr(), grad.data_ptr(), grad.stride(0), rows, n, 1.0,
                                                  N.stream_ptr()), "rb_cross_entropy_grad_lse")
    return lse - target_logit, grad


def vocab_parallel_cross_entropy(local_logits: torch.Tensor, targets: torch.Tensor, pg: ProcessGroup, vocab_start: int):
    """Cross-entropy over a vocabulary sharded across the TP group: local_logits [rows, V/W].  Returns (loss [rows],
    dlogits_local [rows, V/W]).  CUDA bf16 shards whose width is a multiple of 8 take the native kernels; everything
    else the tensor-op form below (two small collectives for max and sum-exp plus one for the target logit)."""
    if local_logits.is_cuda and local_logits.dtype == torch.bfloat16 and local_logits.shape[1] % 8 == 0 and \
            local_logits.stride(1) == 1 and local_logits.stride(0) % 8 == 0:
        return _vocab_parallel_cross_entropy_cuda(local_logits, targets, pg, vocab_start)
    lf = local_logits.float()
    rows, n = lf.shape
    gmax = lf.amax(-1)
    gmax = torch.stack(pg.all_gather(gmax)).amax(0)
    se = torch.exp(lf - gmax[:, None]).sum(-1)
    pg.all_reduce_sum(se, "vp_sumexp")
    lse = gmax + torch.log(se)
    local_t = targets - vocab_start
    mine = (local_t >= 0) & (local_t < n)
    tl = torch.where(mine, lf.gather(1, local_t.clamp(0, n - 1)[:, None])[:, 0], torch.zeros_like(lse))
    pg.all_reduce_sum(tl, "vp_target")
    loss = lse - tl
    grad = torch.exp(lf - lse[:, None])
    grad[mine, local_t[mine]] -= 1.0
    return loss, grad
