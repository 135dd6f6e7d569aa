"""Expert-choice routing (crates/nn/src/expert_choice.rs:39-430): every expert picks its top-c tokens, so load is
balanced by construction and a token may be served by zero or several experts."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N_
from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, InvalidArgument

_P, _I = N_.c_void_p, N_.c_int
N_.optional_sig("rb_ec_select", [_P, _I, _I, _I, _P, _P, _P])
N_.optional_sig("rb_ec_table", [_P, _I, _I, _I, _P, _P])
N_.optional_sig("rb_ec_combine", [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
N_.optional_sig("rb_ec_combine_bwd", [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P])


def ec_select(probs: torch.Tensor, cap: int):
    """Per expert (column of `probs` [T, E], fp32) the `cap` tokens with the largest probability, in ascending token
    order; ties at the threshold go to the lower token index.  Returns (idx int64 [E, cap], gate fp32 [E, cap])."""
    T, E = probs.shape
    if probs.is_cuda:
        p = probs.detach().float().contiguous()
        idx = torch.empty((E, cap), dtype=torch.int64, device=probs.device)
        gate = torch.empty((E, cap), dtype=torch.float32, device=probs.device)
        N_.check(N_.kernels().rb_ec_select(p.data_ptr(), T, E, cap, idx.data_ptr(), gate.data_ptr(), N_.stream_ptr()), "rb_ec_select")
        return idx, gate
    pt = probs.detach().float().t()                                         # [E, T]
    order = torch.argsort(pt, dim=1, descending=True, stable=True)[:, :cap]  # stable: ties keep the lower index first
    idx = torch.sort(order, dim=1).values
    return idx, pt.gather(1, idx)


def ec_table(idx: torch.Tensor, T: int) -> torch.Tensor:
    """table[t, e] = position of token t in expert e's list (int32), -1 when expert e did not choose it."""
    E, cap = idx.shape
    if idx.is_cuda:
        table = torch.empty((T, E), dtype=torch.int32, device=idx.device)
        N_.check(N_.kernels().rb_ec_table(idx.data_ptr(), T, E, cap, table.data_ptr(), N_.stream_ptr()), "rb_ec_table")
        return table
    table = torch.full((T, E), -1, dtype=torch.int32)
    table[idx.reshape(-1), torch.arange(E).repeat_interleave(cap)] = torch.arange(cap, dtype=torch.int32).repeat(E)
    return table


def _combine(y, gate, table, T, out_f32=False):
    E = table.shape[1]
    cap = y.shape[0] // E
    out = torch.empty((T, y.shape[1]), dtype=torch.float32 if out_f32 else torch.bfloat16, device=y.device)
    N_.check(N_.kernels().rb_ec_combine(y.data_ptr(), N_.ptr(gate), table.data_ptr(), out.data_ptr(), T, E, cap, y.shape[1], int(out_f32),
                                        N_.stream_ptr()), "rb_ec_combine")
    return out


class _EcGatherFn(torch.autograd.Function):
    """rows[e * cap + s] = x[idx[e, s]]; backward: every token sums the gradients of the rows it was copied to, in expert
    order (the combine kernel with unit weights)."""

    @staticmethod
    def forward(ctx, x2, idx_flat, table):
        ctx.save_for_backward(table)
        ctx.T = x2.shape[0]
        return ops.gather_rows(x2.contiguous(), idx_flat)

    @staticmethod
    def backward(ctx, drows):
        (table,) = ctx.saved_tensors
        return _combine(drows.contiguous(), None, table, ctx.T), None, None


class _EcCombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_all, gate_flat, idx_flat, table, T):
        y_all, gate_flat = y_all.contiguous(), gate_flat.contiguous()
        ctx.save_for_backward(y_all, gate_flat, idx_flat)
        ctx.T = T
        return _combine(y_all, gate_flat, table, T)

    @staticmethod
    def backward(ctx, dout):
        y_all, gate_flat, idx_flat = ctx.saved_tensors
        n, d = y_all.shape
        dy = torch.empty_like(y_all)
        dgate = torch.empty(n, dtype=torch.float32, device=y_all.device)
        N_.check(N_.kernels().rb_ec_combine_bwd(dout.contiguous().data_ptr(), idx_flat.data_ptr(), gate_flat.data_ptr(), y_all.data_ptr(),
                                                dy.data_ptr(), dgate.data_ptr(), n, ctx.T, d, N_.stream_ptr()), "rb_ec_combine_bwd")
        return dy, dgate, None, None, None


class _EcGateFn(torch.autograd.Function):
    """The chosen probabilities as a differentiable function of `probs`: the gradient of probs[t, e] is the gradient of
    the gate at table[t, e] (or zero), a gather, so no scattered accumulation is needed."""

    @staticmethod
    def forward(ctx, probs, gate_sel, table):
        ctx.save_for_backward(table)
        return gate_sel.reshape(-1).clone()

    @staticmethod
    def backward(ctx, dgate):
        (table,) = ctx.saved_tensors
        T, E = table.shape
        cap = dgate.numel() // E
        pos = torch.arange(E, device=table.device)[None, :] * cap + table.clamp_min(0).long()
        return torch.where(table >= 0, dgate[pos], torch.zeros((), dtype=dgate.dtype, device=dgate.device)), None, None


@dataclass
class ExpertChoiceConfig:
    d_model: int
    num_experts: int
    expert_hidden_dim: int
    tokens_per_expert: int = 8
    all_to_all: bool = True          # with expert parallelism: dispatch by all-to-all (rustral_b200.parallel.expert_parallel)
    capacity_factor: float = 1.0

    def capacity(self) -> int:
        return max(1, int(self.tokens_per_expert * self.capacity_factor))

    def validate_for_batch(self, num_tokens: int) -> None:
        if num_tokens < self.capacity():
            raise InvalidArgument(f"{num_tokens} tokens are fewer than the expert capacity {self.capacity()}")


@dataclass
class ExpertChoiceStats:
    min_tokens: int
    max_tokens: int
    avg_tokens: float
    imbalance: float
    unrouted_tokens: int


class ExpertChoiceRouter(Module, Trainable, Saveable):
    def __init__(self, config: ExpertChoiceConfig, router: Parameter):
        self.config = config
        self.router = router
        self.last_stats: ExpertChoiceStats | None = None

    @classmethod
    def new(cls, backend, config: ExpertChoiceConfig, seed: int = 42):
        return cls(config, backend.normal_parameter("router", (config.num_experts, config.d_model), seed, 0.02))

    def select(self, x2):
        """Returns (token index [E, c], gate weight [E, c], probs [T, E])."""
        c = self.config
        logits = ops.gemm(x2.contiguous(), self.router.tensor, out_dtype=torch.float32)
        probs = ops.softmax(logits)
        cap = min(c.capacity(), x2.shape[0])
        vals, idx = torch.topk(probs.t(), cap, dim=-1)          # per expert: its highest-affinity tokens
        return idx, vals, probs

    def assignments(self, x) -> "ExpertAssignments":
        """The routing decision for `x` as explicit (token, expert, weight) records."""
        x2 = x.reshape(-1, self.config.d_model)
        idx, gate, _ = self.select(x2)
        return ExpertAssignments.from_selection(idx, gate, x2.shape[0])

    def _forward_native(self, x, x2, expert_fn):
        """bf16 CUDA tensors: selection, row gather, combine and their backward passes are the kernels of
        csrc/kernels/expert_choice.cu; the experts see one contiguous [capacity, d] block each."""
        c = self.config
        T, E = x2.shape[0], c.num_experts
        cap = min(c.capacity(), T)
        w = self.router.tensor.to(x2.dtype)
        if E % 8:                                   # the GEMM's output rows need a 16-byte pitch: zero rows up to a multiple of 8
            w = torch.nn.functional.pad(w, (0, 0, 0, (-E) % 8))
        logits = ops.linear(x2, w)[:, :E].float()
        probs = ops.softmax(logits)
        idx, gate_sel = ec_select(probs, cap)
        table = ec_table(idx, T)
        idx_flat = idx.reshape(-1)
        gate = _EcGateFn.apply(probs, gate_sel, table)
        rows = _EcGatherFn.apply(x2, idx_flat, table)
        y_all = torch.cat([expert_fn(e, rows[e * cap:(e + 1) * cap]).to(x2.dtype) for e in range(E)], 0)
        out = _EcCombineFn.apply(y_all, gate, idx_flat, table, T)
        self.last_stats = ExpertChoiceStats(cap, cap, float(cap), 1.0, int((table.max(1).values < 0).sum()))
        return out.to(x.dtype).reshape(x.shape)

    def forward(self, x, expert_fn, ctx: ForwardCtx):
        """expert_fn(e, tokens [n, d]) -> [n, d].  Output: sum over choosing experts of gate * expert output."""
        c = self.config
        x2 = x.reshape(-1, c.d_model)
        c.validate_for_batch(x2.shape[0])
        if x2.is_cuda and x2.dtype == torch.bfloat16 and c.d_model % 8 == 0:
            return self._forward_native(x, x2, expert_fn)
        idx, gate, probs = self.select(x2)
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x2.device)
        served = torch.zeros(x2.shape[0], dtype=torch.int32, device=x2.device)
        for e in range(c.num_experts):
            rows = ops.gather_rows(x2.contiguous(), idx[e]) if not x2.requires_grad else x2[idx[e]]
            y = expert_fn(e, rows)
            # An expert's chosen tokens are distinct (top-c of one row of the affinity matrix), so its contribution is
            # added with a gather, an addition and a plain scatter: no floating-point atomics, and the experts are
            # folded in index order, so the result is the same on every run.
            out.index_put_((idx[e],), out[idx[e]] + y.float() * gate[e][:, None])
            served.index_put_((idx[e],), served[idx[e]] + 1)
        per = [int(idx.shape[1])] * c.num_experts
        self.last_stats = ExpertChoiceStats(min(per), max(per), sum(per) / len(per), 1.0, int((served == 0).sum()))
        return out.to(x.dtype).reshape(x.shape)


@dataclass
class TokenAssignment:
    token_idx: int
    expert_idx: int
    weight: float


@dataclass
class ExpertAssignments:
    """Who serves whom after expert-choice routing (crates/nn/src/expert_choice.rs:359-372): `assignments[e]` lists the
    tokens expert `e` took with their gate weights."""
    assignments: list
    num_tokens: int

    @classmethod
    def from_selection(cls, idx: torch.Tensor, gate: torch.Tensor, num_tokens: int) -> "ExpertAssignments":
        """`idx` / `gate`: [experts, capacity] as returned by `ExpertChoiceRouter.select`."""
        rows = [[TokenAssignment(int(t), e, float(w)) for t, w in zip(idx[e].tolist(), gate[e].tolist())] for e in range(idx.shape[0])]
        return cls(rows, num_tokens)

    def tokens_of(self, expert: int) -> list:
        return [a.token_idx for a in self.assignments[expert]]

    def experts_of(self, token: int) -> list:
        return [a.expert_idx for row in self.assignments for a in row if a.token_idx == token]

    def unrouted_tokens(self) -> list:
        seen = {a.token_idx for row in self.assignments for a in row}
        return [t for t in range(self.num_tokens) if t not in seen]


@dataclass
class RoutingComparison:
    """Analytic comparison of token-choice vs expert-choice load for T tokens."""
    token_choice_max_load: float
    expert_choice_max_load: float

    @classmethod
    def compare(cls, num_tokens: int, num_experts: int, top_k: int, observed_max_fraction: float):
        return cls(observed_max_fraction * num_tokens * top_k, num_tokens * top_k / num_experts)
