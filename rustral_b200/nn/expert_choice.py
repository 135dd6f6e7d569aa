"""Expert-choice routing (crates/nn/src/expert_choice.rs:39-430): every expert picks its top-c tokens, so load is
balanced by construction and a token may be served by zero or several experts."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, InvalidArgument


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

    def forward(self, x, expert_fn, ctx: ForwardCtx):
        """expert_fn(e, tokens [n, d]) -> [n, d].  Output: sum over choosing experts of gate * expert output."""
        c = self.config
        x2 = x.reshape(-1, c.d_model)
        c.validate_for_batch(x2.shape[0])
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
class RoutingComparison:
    """Analytic comparison of token-choice vs expert-choice load for T tokens."""
    token_choice_max_load: float
    expert_choice_max_load: float

    @classmethod
    def compare(cls, num_tokens: int, num_experts: int, top_k: int, observed_max_fraction: float):
        return cls(observed_max_fraction * num_tokens * top_k, num_tokens * top_k / num_experts)
