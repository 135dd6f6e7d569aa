"""Mixture-of-experts layers (crates/nn/src/moe.rs:32-470).

Real top-k routing (the reference's gating hands out experts as `i % E`, moe.rs:122-141), sparse dispatch (the
reference sends every token to every expert, :344-348), the standard load-balancing loss E * sum_e f_e P_e (the
reference's variant chunks probabilities by row, :146-165), and capacity handling.  Expert weights are stacked
([E, F, d]) so one grouped GEMM serves all experts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, InvalidArgument
from ..ops import moe as moe_ops


@dataclass
class MoEConfig:
    d_model: int
    num_experts: int
    expert_dim: int
    top_k: int = 2
    capacity_factor: float = 1.0
    dropout: float = 0.0
    aux_loss_coef: float = 0.01
    activation: str = "gelu"          # "gelu" (reference's Expert: fc1 -> GELU -> fc2) or "swiglu"
    renormalize: bool = True

    def with_top_k(self, k: int):
        self.top_k = k
        return self

    def with_capacity_factor(self, f: float):
        self.capacity_factor = f
        return self

    def expert_capacity(self, num_tokens: int) -> int:
        return int(math.ceil(num_tokens * self.top_k * self.capacity_factor / self.num_experts))


@dataclass
class GatingOutput:
    indices: torch.Tensor      # int32 [T, k]
    weights: torch.Tensor      # fp32 [T, k]
    probs: torch.Tensor        # fp32 [T, E]
    aux_loss: torch.Tensor


@dataclass
class MoEOutput:
    output: torch.Tensor
    aux_loss: torch.Tensor


@dataclass
class MoEStats:
    tokens_per_expert: list
    load_imbalance: float      # max / mean
    dropped_tokens: int

    @classmethod
    def from_counts(cls, counts, capacity: int | None = None):
        c = [int(v) for v in counts]
        mean = sum(c) / max(1, len(c))
        dropped = sum(max(0, v - capacity) for v in c) if capacity else 0
        return cls(c, (max(c) / mean) if mean > 0 else 0.0, dropped)


class TopKGating(Module, Trainable, Saveable):
    """gate_proj: Linear(d_model -> num_experts, no bias); per-token softmax then top-k."""

    def __init__(self, config: MoEConfig, gate_proj: Parameter):
        self.config = config
        self.gate_proj = gate_proj

    @classmethod
    def new(cls, backend, config: MoEConfig, seed: int = 42):
        return cls(config, backend.normal_parameter("gate_proj", (config.num_experts, config.d_model), seed, 0.02))

    def forward(self, x2, ctx: ForwardCtx) -> GatingOutput:
        c = self.config
        logits = ops.gemm(x2.contiguous(), self.gate_proj.tensor, out_dtype=torch.float32)
        idx, w, probs = moe_ops.route(logits, c.top_k, c.renormalize)
        counts = torch.bincount(idx.reshape(-1).long().cpu(), minlength=c.num_experts).to(probs.device)
        f = counts.float() / float(idx.numel())
        aux = (f * probs.mean(0)).sum() * c.num_experts
        return GatingOutput(idx, w, probs, aux)

    def _children(self):
        yield "gate_proj", self.gate_proj


class Expert(Module, Trainable, Saveable):
    """One expert as a standalone module: fc1 -> GELU -> fc2 (kept for API parity and tests)."""

    def __init__(self, fc1: Parameter, fc2: Parameter):
        self.fc1, self.fc2 = fc1, fc2

    def forward(self, x, ctx: ForwardCtx):
        return ops.linear(ops.gelu(ops.linear(x, self.fc1.tensor)), self.fc2.tensor)


class ExpertLayer(Module, Trainable, Saveable):
    """Gate + stacked experts.  Parameter names: gate.gate_proj, experts_w1 [E, F(2F), d], experts_w2 [E, d, F]."""

    def __init__(self, config: MoEConfig, gate: TopKGating, w1: Parameter, w2: Parameter):
        self.config = config
        self.gate = gate
        self.experts_w1, self.experts_w2 = w1, w2

    @classmethod
    def new(cls, backend, config: MoEConfig, seed: int = 42):
        c = config
        f1 = 2 * c.expert_dim if c.activation == "swiglu" else c.expert_dim
        return cls(c, TopKGating.new(backend, c, seed),
                   backend.normal_parameter("experts_w1", (c.num_experts, f1, c.d_model), seed + 1, 0.02),
                   backend.normal_parameter("experts_w2", (c.num_experts, c.d_model, c.expert_dim), seed + 2, 0.02))

    def forward(self, x, ctx: ForwardCtx) -> MoEOutput:
        """x: [..., d_model]; every leading dimension is a token dimension."""
        c = self.config
        x2 = x.reshape(-1, c.d_model)
        with ctx.profile("moe", x2.shape):
            y, aux = moe_ops.moe_mlp(x2.contiguous(), self.gate.gate_proj.tensor, self.experts_w1.tensor,
                                     self.experts_w2.tensor, c.top_k, c.activation, c.renormalize)
        return MoEOutput(y.reshape(x.shape), aux * c.aux_loss_coef)

    def expert(self, e: int) -> Expert:
        """A view of expert `e` as a standalone module (GELU kind only)."""
        return Expert(Parameter("fc1", self.experts_w1.tensor[e]), Parameter("fc2", self.experts_w2.tensor[e]))

    def stats(self, x) -> MoEStats:
        g = self.gate.forward(x.reshape(-1, self.config.d_model), ForwardCtx.inference())
        counts = torch.bincount(g.indices.reshape(-1).long().cpu(), minlength=self.config.num_experts)
        return MoEStats.from_counts(counts.tolist(), self.config.expert_capacity(g.indices.shape[0]))


class ExpertParallel:
    """Expert placement over ranks: expert e lives on rank e % world_size (crates/nn/src/moe.rs:408-433)."""

    def __init__(self, num_experts: int, world_size: int, rank: int = 0):
        if world_size <= 0 or num_experts % world_size:
            raise InvalidArgument("num_experts must be a positive multiple of world_size")
        self.num_experts, self.world_size, self.rank = num_experts, world_size, rank

    def rank_of(self, expert: int) -> int:
        return expert % self.world_size

    def local_experts(self, rank: int | None = None) -> list:
        r = self.rank if rank is None else rank
        return [e for e in range(self.num_experts) if e % self.world_size == r]

    def is_local(self, expert: int) -> bool:
        return self.rank_of(expert) == self.rank
