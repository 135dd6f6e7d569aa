"""Shared + routed experts, DeepSeek-style (crates/nn/src/shared_expert.rs:44-420).

Shared experts see every token; routed experts are chosen per token by real top-k routing.  Experts are SwiGLU
MLPs with the SiLU in place (the reference's ExpertMLP multiplies gate and up without it, shared_expert.rs:158-168);
routed compute is one grouped GEMM per projection instead of one tiny GEMM per (token, expert)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable
from ..ops import moe as moe_ops
from .linear import LinearBuilder


@dataclass
class SharedExpertConfig:
    d_model: int
    num_shared: int
    num_routed: int
    expert_hidden_dim: int
    top_k: int = 2
    shared_weight: float = 1.0
    routed_weight: float = 1.0
    use_residual: bool = True
    renormalize: bool = False        # the reference does not renormalise the selected weights


class ExpertMLP(Module, Trainable, Saveable):
    """down( silu(gate(x)) * up(x) ); gate and up share one stacked weight."""

    def __init__(self, gate_up, down):
        self.gate_up, self.down = gate_up, down

    @classmethod
    def new(cls, backend, d_model: int, hidden: int, seed: int = 42):
        return cls(LinearBuilder(d_model, 2 * hidden).seed(seed).scale(0.02).build(backend),
                   LinearBuilder(hidden, d_model).seed(seed + 1).scale(0.02).build(backend))

    def forward(self, x, ctx: ForwardCtx):
        return self.down(ops.swiglu(self.gate_up(x, ctx)), ctx)


@dataclass
class SharedExpertStats:
    tokens_per_routed_expert: list
    load_balance_score: float      # mean / max, 1.0 = perfectly even


class SharedExpertLayer(Module, Trainable, Saveable):
    def __init__(self, config, shared_experts, router: Parameter, routed_w1: Parameter, routed_w2: Parameter, output_proj):
        self.config = config
        self.shared_experts = shared_experts
        self.router = router
        self.routed_w1, self.routed_w2 = routed_w1, routed_w2
        self.output_proj = output_proj
        self.last_aux_loss = None

    @classmethod
    def new(cls, backend, config: SharedExpertConfig, seed: int = 42):
        c = config
        shared = [ExpertMLP.new(backend, c.d_model, c.expert_hidden_dim, seed + 10 * i) for i in range(c.num_shared)]
        return cls(c, shared, backend.normal_parameter("router", (c.num_routed, c.d_model), seed + 1000, 0.02),
                   backend.normal_parameter("routed_w1", (c.num_routed, 2 * c.expert_hidden_dim, c.d_model), seed + 1001, 0.02),
                   backend.normal_parameter("routed_w2", (c.num_routed, c.d_model, c.expert_hidden_dim), seed + 1002, 0.02),
                   LinearBuilder(c.d_model, c.d_model).seed(seed + 1003).scale(0.02).build(backend))

    def forward(self, x, ctx: ForwardCtx):
        c = self.config
        x2 = x.reshape(-1, c.d_model).contiguous()
        shared = None
        for ex in self.shared_experts:
            y = ex(x2, ctx)
            shared = y if shared is None else shared + y
        if shared is not None and c.num_shared > 1:
            shared = shared * (1.0 / c.num_shared)
        routed, aux = moe_ops.moe_mlp(x2, self.router.tensor, self.routed_w1.tensor, self.routed_w2.tensor, c.top_k,
                                      "swiglu", c.renormalize)
        self.last_aux_loss = aux
        y = routed * c.routed_weight
        if shared is not None:
            y = y + shared * c.shared_weight
        if c.use_residual:
            y = y + x2
        return self.output_proj(y, ctx).reshape(x.shape)

    def routing(self, x) -> "HybridRouting":
        """The gates of `x` spelled out (crates/nn/src/shared_expert.rs:122-127): every token passes through the shared
        experts with weight `shared_weight`; `routed_gates` is the router's softmax over the routed experts and
        `top_k_indices` / `top_k_weights` what was kept of it."""
        c = self.config
        x2 = x.reshape(-1, c.d_model).contiguous()
        logits = ops.gemm(x2, self.router.tensor, out_dtype=torch.float32)
        idx, w, probs = moe_ops.route(logits, c.top_k, c.renormalize)
        return HybridRouting(torch.full((x2.shape[0],), float(c.shared_weight)), probs.detach().float().cpu(),
                             idx.detach().long().cpu(), (w.detach().float() * c.routed_weight).cpu())

    def stats(self, x) -> SharedExpertStats:
        c = self.config
        logits = ops.gemm(x.reshape(-1, c.d_model).contiguous(), self.router.tensor, out_dtype=torch.float32)
        idx, _, _ = moe_ops.route(logits, c.top_k, c.renormalize)
        counts = torch.bincount(idx.reshape(-1).long().cpu(), minlength=c.num_routed).tolist()
        mx = max(counts) or 1
        return SharedExpertStats(counts, (sum(counts) / len(counts)) / mx)


@dataclass
class HybridRouting:
    shared_gate: torch.Tensor        # [tokens]
    routed_gates: torch.Tensor       # [tokens, num_routed]
    top_k_indices: torch.Tensor      # [tokens, top_k]
    top_k_weights: torch.Tensor      # [tokens, top_k]


@dataclass
class SharedAndRoutedConfig:
    shared: int
    routed: int
    active_routed: int

    def active_fraction(self) -> float:
        return (self.shared + self.active_routed) / (self.shared + self.routed)
