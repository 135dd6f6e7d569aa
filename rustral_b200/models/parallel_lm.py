"""Llama-style decoder language model for tensor-, pipeline- and expert-parallel training.

One class covers the dense model (RMSNorm, rotary GQA attention, SwiGLU MLP) and the mixture-of-experts variant
(top-k SwiGLU experts in place of the MLP).  It is written against the differentiable ops of `rustral_b200.ops`, so
torch.autograd drives the backward pass while every matmul, attention, norm, rotary, SwiGLU, routing and loss kernel
is one of the framework's own.

Parallel layouts:

* tensor parallel with sequence parallelism: between blocks a rank holds a contiguous block of the (batch * seq)
  rows; QKV and gate/up are column-parallel (all-gather of the rows fused into the GEMM), the output and down
  projections are row-parallel (reduce-scatter fused into the GEMM epilogue), see parallel/fused_tp.py.  The LM head
  is column-parallel over the vocabulary with a vocabulary-parallel cross-entropy.  Without a `fused_tp` context the
  same maths runs over ProcessGroup collectives (the baseline the fused kernels are measured against).
* pipeline parallel: a stage owns a contiguous range of blocks (`first_layer`, `last_layer`), optionally the
  embedding and the head; `embed` / `blocks` / `loss` are the pieces parallel/pipeline_parallel.py schedules.
* expert parallel: the experts of every MoE block are spread over the ranks of `ep` (parallel/expert_parallel.py);
  attention and the dense parameters are replicated and their gradients averaged over the group.

The reference has no such model: its tensor-parallel layers are forward-only over host slices
(crates/distributed/src/tensor_parallel.rs:119-173), its MoE routes with host loops (crates/nn/src/moe.rs:277-370).
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import ops
from ..ops import moe as moe_ops
from ..ops import rotary


@dataclass
class ParallelLMConfig:
    vocab_size: int = 32000
    d_model: int = 512
    n_layer: int = 4
    n_head: int = 8
    n_kv_head: int = 8
    ffn_hidden: int = 1536
    seq_len: int = 512
    rope_theta: float = 500000.0
    eps: float = 1e-5
    num_experts: int = 0          # > 0: every block's MLP is a top-k mixture of SwiGLU experts
    top_k: int = 2
    aux_coef: float = 0.01
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    def params_per_layer(self) -> int:
        d, hd = self.d_model, self.head_dim
        attn = d * (self.n_head + 2 * self.n_kv_head) * hd + self.n_head * hd * d
        mlp = 3 * d * self.ffn_hidden * max(1, self.num_experts) + (self.num_experts * d if self.num_experts else 0)
        return attn + mlp + 2 * d

    def num_params(self) -> int:
        return self.n_layer * self.params_per_layer() + 2 * self.vocab_size * self.d_model + self.d_model

    def flops_per_token(self) -> float:
        """Training FLOPs per token (forward + backward = 3 x forward), active parameters only, causal attention."""
        d, hd = self.d_model, self.head_dim
        attn_proj = d * (self.n_head + 2 * self.n_kv_head) * hd + self.n_head * hd * d
        mlp = 3 * d * self.ffn_hidden * (self.top_k if self.num_experts else 1)
        dense = self.n_layer * (attn_proj + mlp) + self.vocab_size * d
        attn = self.n_layer * 2 * self.seq_len * d * 0.5 * 2          # QK^T and PV, causal half
        return 6.0 * dense + 3.0 * attn


def llama_8b(**kw) -> ParallelLMConfig:
    base = dict(vocab_size=128256, d_model=4096, n_layer=32, n_head=32, n_kv_head=8, ffn_hidden=14336, seq_len=4096,
                rope_theta=500000.0)
    base.update(kw)
    return ParallelLMConfig(**base)


def moe_24l(**kw) -> ParallelLMConfig:
    base = dict(vocab_size=32000, d_model=2048, n_layer=24, n_head=16, n_kv_head=16, ffn_hidden=8192, seq_len=2048,
                num_experts=8, top_k=2, aux_coef=0.01)
    base.update(kw)
    return ParallelLMConfig(**base)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy over rows with the vocabulary split over the tensor-parallel group."""

    @staticmethod
    def forward(ctx, local_logits, targets, pg, vocab_start):
        from ..parallel.tensor_parallel import vocab_parallel_cross_entropy
        loss, grad = vocab_parallel_cross_entropy(local_logits, targets, pg, vocab_start)
        ctx.save_for_backward((grad / loss.numel()).to(local_logits.dtype))
        return loss.mean()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return grad * g.to(grad.dtype), None, None, None


class ParallelDecoderLM:
    """Parameters live in `self.params` (bf16 leaves); `self.replicated` names those every tensor-parallel rank holds
    in full and sees different rows of (their gradients are summed over the group by `sync_grads`)."""

    def __init__(self, cfg: ParallelLMConfig, device, *, tp_pg=None, fused_tp=None, ep=None, dp_group=None,
                 first_layer: int = 0, last_layer: int | None = None, has_embed: bool = True, has_head: bool = True,
                 seed: int = 0, fsdp=None, cp=None, cp_striped: bool = True):
        """`fsdp` (a parallel.fused_tp.FusedTP over the data-parallel group): ZeRO-3 for the block weights.  Each rank
        keeps 1/W of the rows of every projection in symmetric memory; the forward all-gathers them inside the
        consuming GEMM and the weight gradient is reduce-scattered inside its GEMM (FSDPLinearFn).

        `cp` (a parallel.peer_ring.PeerRing): context parallelism.  Every rank of the ring holds 1/W of the tokens of
        each sequence (striped: token t on rank t mod W, which balances causal attention; or contiguous), runs all
        layers on them, and attention pulls the other ranks' K / V over NVLink.  Parameters are replicated over the
        ring, so `dp_group` must span it: their gradients are averaged like data-parallel gradients."""
        self.cfg, self.device = cfg, torch.device(device)
        self.tp_pg, self.fused_tp, self.ep, self.dp_group = tp_pg, fused_tp, ep, dp_group
        self.fsdp = fsdp
        self.cp, self.cp_striped = cp, cp_striped
        if cp is not None and (tp_pg is not None or ep is not None or fsdp is not None):
            raise ValueError("context parallelism is combined with plain data parallelism only")
        if cp is not None and dp_group is None:
            raise ValueError("context parallelism needs dp_group (a group spanning the ring) for the gradient average")
        self.fsdp_shards: dict = {}
        if fsdp is not None and (tp_pg is not None or ep is not None):
            raise ValueError("fsdp is combined with plain data parallelism only")
        self.tp = tp_pg.world_size if tp_pg is not None else 1
        self.tp_rank = tp_pg.rank if tp_pg is not None else 0
        self.first_layer = first_layer
        self.last_layer = cfg.n_layer if last_layer is None else last_layer
        self.has_embed, self.has_head = has_embed, has_head
        if cfg.n_head % self.tp or cfg.n_kv_head % self.tp or cfg.ffn_hidden % self.tp or cfg.vocab_size % self.tp:
            raise ValueError("heads, KV heads, FFN width and vocabulary must be divisible by the tensor-parallel size")
        self.params: dict = {}
        self.replicated: set = set()
        self.expert_names: set = set()
        self._init(seed)

    # ------------------------------------------------------------------------------------------------ parameters
    def _rand(self, shape, seed, std=None):
        g = torch.Generator(device=self.device).manual_seed(seed)
        std = self.cfg.init_std if std is None else std
        t = torch.empty(shape, dtype=torch.float32, device=self.device).normal_(0.0, std, generator=g)
        return t.to(torch.bfloat16).requires_grad_()

    def _weight(self, name: str, shape, sd, tp_rank: int, std):
        """A block projection: the tensor-parallel shard, or with `fsdp` this data-parallel rank's row shard of it,
        stored in symmetric memory (the parameter IS the symmetric buffer, so optimizer updates are visible to peers)."""
        if self.fsdp is None:
            return self._rand(shape, sd(name, tp_rank), std)
        W, r = self.fsdp.world, self.fsdp.rank
        rows = shape[0] // W
        if shape[0] % W or not self.fsdp.supports(rows):
            raise ValueError(f"fsdp: {name} has {shape[0]} rows, not a multiple of 128 x {W}")
        shard = self._rand((rows, shape[1]), sd(name, r), std).detach()
        ws = self.fsdp.shard_weight(shard, pooled=True)
        self.fsdp_shards[name] = ws
        return ws.tensor.requires_grad_()

    def _init(self, seed: int) -> None:
        c, tp, r = self.cfg, self.tp, self.tp_rank
        d, hd = c.d_model, c.head_dim
        hq, hk, f = c.n_head // tp, c.n_kv_head // tp, c.ffn_hidden // tp
        P = self.params
        # a shard's seed depends on (parameter, shard) only, so a gathered checkpoint is the same for every layout
        sd = lambda name, shard=0: (zlib.crc32(f"{seed}/{name}".encode()) & 0x7FFFFFFF) * 64 + shard
        if self.has_embed:
            P["wte"] = self._rand((c.vocab_size, d), sd("wte"))
            self.replicated.add("wte")
        for l in range(self.first_layer, self.last_layer):
            p = f"l{l}."
            P[p + "attn_norm"] = torch.ones(d, dtype=torch.bfloat16, device=self.device, requires_grad=True)
            P[p + "wqkv"] = self._weight(p + "wqkv", ((hq + 2 * hk) * hd, d), sd, r, None)
            P[p + "wo"] = self._weight(p + "wo", (d, hq * hd), sd, r, c.init_std / math.sqrt(2 * c.n_layer))
            P[p + "mlp_norm"] = torch.ones(d, dtype=torch.bfloat16, device=self.device, requires_grad=True)
            self.replicated.update({p + "attn_norm", p + "mlp_norm"})
            if c.num_experts:
                el = c.num_experts // (self.ep.world if self.ep is not None else 1)
                er = self.ep.rank if self.ep is not None else 0
                P[p + "router"] = self._rand((c.num_experts, d), sd(p + "router"))
                P[p + "w1"] = self._rand((el, 2 * c.ffn_hidden, d), sd(p + "w1", er))
                P[p + "w2"] = self._rand((el, d, c.ffn_hidden), sd(p + "w2", er), c.init_std / math.sqrt(2 * c.n_layer))
                self.replicated.add(p + "router")
                self.expert_names.update({p + "w1", p + "w2"})
            else:
                P[p + "wgu"] = self._weight(p + "wgu", (2 * f, d), sd, r, None)
                P[p + "wdown"] = self._weight(p + "wdown", (d, f), sd, r, c.init_std / math.sqrt(2 * c.n_layer))
        if self.has_head:
            P["final_norm"] = torch.ones(d, dtype=torch.bfloat16, device=self.device, requires_grad=True)
            P["head"] = self._rand((c.vocab_size // tp, d), sd("head", r))
            self.replicated.add("final_norm")

    def parameters(self):
        return list(self.params.values())

    # ------------------------------------------------------------------------------------------------ checkpoints
    def _shard_plan(self) -> dict:
        """local parameter name -> function(full state dict) giving this rank's tensor, for dense (non-MoE) models.
        The full state uses the checkpoint names of the single-GPU engine (tok_embed.embed, layers.N.attn.wq.weight,
        ..., ffn.gate_up.weight, head.weight), which is also what utils.hf.convert_hf_llama produces."""
        c, tp, r = self.cfg, self.tp, self.tp_rank
        hd = c.head_dim
        hq, hk, f, v = c.n_head // tp, c.n_kv_head // tp, c.ffn_hidden // tp, c.vocab_size // tp
        rows = lambda t, n: t[r * n:(r + 1) * n]
        plan = {}
        if self.has_embed:
            plan["wte"] = lambda s: s["tok_embed.embed"]
        if self.has_head:
            plan["final_norm"] = lambda s: s["final_norm.weight"]
            plan["head"] = lambda s: rows(s["head.weight"], v)
        for l in range(self.first_layer, self.last_layer):
            p, q = f"l{l}.", f"layers.{l}."
            plan[p + "attn_norm"] = lambda s, q=q: s[q + "ln1.weight"]
            plan[p + "mlp_norm"] = lambda s, q=q: s[q + "ln2.weight"]
            plan[p + "wqkv"] = lambda s, q=q: torch.cat([rows(s[q + "attn.wq.weight"], hq * hd), rows(s[q + "attn.wk.weight"], hk * hd),
                                                         rows(s[q + "attn.wv.weight"], hk * hd)], 0)
            plan[p + "wo"] = lambda s, q=q: s[q + "attn.wo.weight"][:, r * hq * hd:(r + 1) * hq * hd]
            plan[p + "wgu"] = lambda s, q=q: torch.cat([rows(s[q + "ffn.gate_up.weight"][:c.ffn_hidden], f),
                                                        rows(s[q + "ffn.gate_up.weight"][c.ffn_hidden:], f)], 0)
            plan[p + "wdown"] = lambda s, q=q: s[q + "ffn.down.weight"][:, r * f:(r + 1) * f]
        return plan

    def load_state_dict(self, state: dict) -> None:
        """Loads an UNSHARDED dense checkpoint: every rank reads the full state and keeps its tensor-parallel /
        pipeline (/ FSDP row) shard.  Strict for the parameters this rank owns: a missing tensor or a shape mismatch
        raises before anything is written."""
        if self.cfg.num_experts:
            raise ValueError("load_state_dict covers dense models; expert weights have no single-GPU checkpoint format")
        staged = {}
        for name, pick in self._shard_plan().items():
            try:
                t = pick(state)
            except KeyError as e:
                raise KeyError(f"checkpoint is missing {e.args[0]!r} (needed for {name})") from None
            if name in self.fsdp_shards:
                W, rr = self.fsdp.world, self.fsdp.rank
                n = t.shape[0] // W
                t = t[rr * n:(rr + 1) * n]
            if tuple(t.shape) != tuple(self.params[name].shape):
                raise ValueError(f"{name}: checkpoint gives {tuple(t.shape)}, the model holds {tuple(self.params[name].shape)}")
            staged[name] = t
        with torch.no_grad():
            for name, t in staged.items():
                self.params[name].copy_(t.to(self.params[name].device, self.params[name].dtype))

    def gather_state_dict(self) -> dict:
        """Collective over the tensor-parallel group: the unsharded checkpoint (fp32, single-GPU engine names) of a
        dense model that is sharded over tensor-parallel ranks, assembled on every rank.  The inverse of
        `load_state_dict`; pipeline stages return the layers (and embedding / head) they own."""
        if self.cfg.num_experts or self.fsdp is not None:
            raise ValueError("gather_state_dict covers dense tensor- / pipeline-parallel models")
        c, P, tp = self.cfg, self.params, self.tp
        hd = c.head_dim
        hq, hk, f = c.n_head // tp, c.n_kv_head // tp, c.ffn_hidden // tp
        f32 = lambda t: t.detach().float().cpu().clone()

        def gather(t):
            """Every rank's copy of a sharded tensor, in rank order."""
            if tp == 1:
                return [f32(t)]
            return [f32(x) for x in self.tp_pg.all_gather(t.detach().contiguous())]
        out = {}
        if self.has_embed:
            out["tok_embed.embed"] = f32(P["wte"])
        if self.has_head:
            out["final_norm.weight"] = f32(P["final_norm"])
            out["head.weight"] = torch.cat(gather(P["head"]), 0)
        for l in range(self.first_layer, self.last_layer):
            p, q = f"l{l}.", f"layers.{l}."
            parts = gather(P[p + "wqkv"])
            out[q + "attn.wq.weight"] = torch.cat([x[:hq * hd] for x in parts], 0)
            out[q + "attn.wk.weight"] = torch.cat([x[hq * hd:(hq + hk) * hd] for x in parts], 0)
            out[q + "attn.wv.weight"] = torch.cat([x[(hq + hk) * hd:] for x in parts], 0)
            out[q + "attn.wo.weight"] = torch.cat(gather(P[p + "wo"]), 1)
            parts = gather(P[p + "wgu"])
            out[q + "ffn.gate_up.weight"] = torch.cat([x[:f] for x in parts] + [x[f:] for x in parts], 0)
            out[q + "ffn.down.weight"] = torch.cat(gather(P[p + "wdown"]), 1)
            out[q + "ln1.weight"], out[q + "ln2.weight"] = f32(P[p + "attn_norm"]), f32(P[p + "mlp_norm"])
        return out

    def state_dict(self) -> dict:
        """The unsharded checkpoint of a model held by ONE rank (no tensor / pipeline / FSDP sharding): fp32 tensors
        under the single-GPU engine's names."""
        if self.tp != 1 or self.fsdp is not None or self.cfg.num_experts or not (self.has_embed and self.has_head) or \
                self.first_layer != 0 or self.last_layer != self.cfg.n_layer:
            raise ValueError("state_dict exports unsharded dense models only")
        c, P = self.cfg, self.params
        hd = c.head_dim
        qe, ke = c.n_head * hd, (c.n_head + c.n_kv_head) * hd
        f32 = lambda t: t.detach().float().cpu().clone()
        out = {"tok_embed.embed": f32(P["wte"]), "final_norm.weight": f32(P["final_norm"]), "head.weight": f32(P["head"])}
        for l in range(c.n_layer):
            p, q = f"l{l}.", f"layers.{l}."
            w = f32(P[p + "wqkv"])
            out[q + "attn.wq.weight"], out[q + "attn.wk.weight"], out[q + "attn.wv.weight"] = w[:qe].clone(), w[qe:ke].clone(), w[ke:].clone()
            out[q + "attn.wo.weight"] = f32(P[p + "wo"])
            out[q + "ffn.gate_up.weight"], out[q + "ffn.down.weight"] = f32(P[p + "wgu"]), f32(P[p + "wdown"])
            out[q + "ln1.weight"], out[q + "ln2.weight"] = f32(P[p + "attn_norm"]), f32(P[p + "mlp_norm"])
        return out

    def local_param_count(self) -> int:
        return sum(p.numel() for p in self.params.values())

    # ------------------------------------------------------------------------------------------------ layers
    def _fsdp_linear(self, x, name: str):
        from ..parallel.fused_tp import FSDPLinearFn
        return FSDPLinearFn.apply(x, self.params[name], None, "none", self.fsdp, self.fsdp_shards[name])

    def _col(self, x, name: str):
        """Column-parallel projection of sequence-sharded rows: [R / tp, d] -> [R, n / tp]."""
        if name in self.fsdp_shards:
            return self._fsdp_linear(x, name)
        w = self.params[name]
        if self.tp == 1:
            return ops.linear(x, w)
        if self.fused_tp is not None and self.fused_tp.supports(x.shape[0]):
            from ..parallel.fused_tp import ColumnSeqParallelFn
            return ColumnSeqParallelFn.apply(x, w, None, "none", self.fused_tp)
        from ..parallel.tensor_parallel import _GatherSeq
        return ops.linear(_GatherSeq.apply(x, self.tp_pg), w)

    def _row(self, x, name: str, residual):
        """Row-parallel projection back to sequence-sharded rows: [R, k / tp] -> [R / tp, d] (+ residual)."""
        if name in self.fsdp_shards:
            return self._fsdp_linear(x, name) + residual
        w = self.params[name]
        if self.tp == 1:
            return ops.linear(x, w, None, "none", residual)
        if self.fused_tp is not None and x.shape[0] % self.tp == 0 and self.fused_tp.supports(x.shape[0] // self.tp):
            from ..parallel.fused_tp import RowSeqParallelFn
            return RowSeqParallelFn.apply(x, w, residual, self.fused_tp)
        from ..parallel.tensor_parallel import _ReduceScatterSeq
        return _ReduceScatterSeq.apply(ops.linear(x, w), self.tp_pg) + residual

    def _block(self, l: int, x, batch: int, seq: int, positions=None):
        c, P, p = self.cfg, self.params, f"l{l}."
        hd = c.head_dim
        hq, hk = c.n_head // self.tp, c.n_kv_head // self.tp
        h = ops.rms_norm(x, P[p + "attn_norm"], c.eps)
        qkv = self._col(h, p + "wqkv")                                   # [B*S, (hq + 2 hk) * hd]
        q = rotary.rope(qkv[:, :hq * hd].reshape(batch, seq, hq, hd), seq, positions=positions, theta=c.rope_theta)
        k = rotary.rope(qkv[:, hq * hd:(hq + hk) * hd].reshape(batch, seq, hk, hd), seq, positions=positions,
                        theta=c.rope_theta)
        v = qkv[:, (hq + hk) * hd:].reshape(batch, seq, hk, hd)
        if self.cp is not None:
            o = self.cp.attention(q, k, v.contiguous(), causal=True, striped=self.cp_striped)
        else:
            o = ops.flash_attention(q, k, v, True)
        x = self._row(o.reshape(batch * seq, hq * hd), p + "wo", x)
        h = ops.rms_norm(x, P[p + "mlp_norm"], c.eps)
        aux = None
        if c.num_experts:
            if self.ep is not None:
                from ..parallel.expert_parallel import ep_moe_mlp
                y, aux = ep_moe_mlp(h, P[p + "router"], P[p + "w1"], P[p + "w2"], self.ep, c.top_k, "swiglu")
            else:
                y, aux = moe_ops.moe_mlp(h, P[p + "router"], P[p + "w1"], P[p + "w2"], c.top_k, "swiglu")
            x = x + y
        else:
            gu = self._col(h, p + "wgu")
            x = self._row(rotary.swiglu(gu), p + "wdown", x)
        return x, aux

    # ------------------------------------------------------------------------------------------------ forward
    def local_rows(self, batch: int, seq: int) -> slice:
        rows = batch * seq
        if rows % self.tp:
            raise ValueError("batch * seq must be divisible by the tensor-parallel size")
        n = rows // self.tp
        return slice(self.tp_rank * n, (self.tp_rank + 1) * n)

    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, S] (the same on every tensor-parallel rank) -> this rank's rows [B*S / tp, d]."""
        B, S = ids.shape
        flat = ids.reshape(-1)[self.local_rows(B, S)].contiguous()
        return ops.embedding(flat, self.params["wte"])

    def cp_positions(self, seq: int) -> torch.Tensor:
        """Positions (int64, ascending) of the tokens this context-parallel rank holds of a `seq`-token sequence."""
        W, r = self.cp.world, self.cp.rank
        if seq % W:
            raise ValueError("the sequence length must be divisible by the context-parallel size")
        if self.cp_striped:
            return torch.arange(r, seq, W, device=self.device)
        return torch.arange(r * (seq // W), (r + 1) * (seq // W), device=self.device)

    def blocks(self, x, batch: int, seq: int, positions=None):
        """`positions` (int64 [batch * seq], context parallelism): the position of every local token in its sequence."""
        aux_total = None
        for l in range(self.first_layer, self.last_layer):
            x, aux = self._block(l, x, batch, seq, positions)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        return x, aux_total

    def loss(self, x, targets: torch.Tensor) -> torch.Tensor:
        """x: this rank's rows after the last block; targets [B, S] (all rows)."""
        c = self.cfg
        h = ops.rms_norm(x, self.params["final_norm"], c.eps)
        logits = self._col(h, "head")                          # [B*S, V / tp]
        t = targets.reshape(-1)
        if self.tp == 1:
            return ops.cross_entropy(logits, t)
        return _VocabParallelCE.apply(logits, t, self.tp_pg, self.tp_rank * (c.vocab_size // self.tp))

    def forward_loss(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S + 1] -> scalar training loss (next-token cross-entropy + aux_coef * load-balancing loss)."""
        ids, targets = tokens[:, :-1], tokens[:, 1:]
        B, S = ids.shape
        positions = None
        if self.cp is not None:                      # this rank's tokens of every sequence; the loss is their mean
            pos = self.cp_positions(S)
            ids, targets = ids[:, pos].contiguous(), targets[:, pos].contiguous()
            S = pos.numel()
            positions = pos.repeat(B)
        x, aux = self.blocks(self.embed(ids), B, S, positions)
        loss = self.loss(x, targets)
        if aux is not None:
            loss = loss + self.cfg.aux_coef * aux / (self.last_layer - self.first_layer)
        return loss

    # ------------------------------------------------------------------------------------------------ gradients
    def sync_grads(self, main_grads: dict) -> None:
        """Sum the gradients of replicated parameters over the tensor-parallel group; average dense gradients over
        the data / expert-parallel group and rescale the expert gradients (which already hold every rank's tokens)."""
        if self.tp > 1:
            for name in sorted(self.replicated):
                if name in main_grads:
                    dist.all_reduce(main_grads[name], group=self.tp_pg.group)
        if self.fsdp is not None:
            world = self.fsdp.world
            for name in sorted(main_grads):
                g = main_grads[name]
                if name not in self.fsdp_shards:                 # replicated: average over the data-parallel ranks
                    dist.all_reduce(g, group=self.fsdp.group)
                g.mul_(1.0 / world)                              # sharded: already summed inside the wgrad GEMM
            return
        if self.dp_group is not None or self.ep is not None:
            group = self.dp_group if self.dp_group is not None else self.ep.group
            world = dist.get_world_size(group)
            for name in sorted(main_grads):
                g = main_grads[name]
                if name in self.expert_names and self.ep is not None:
                    g.mul_(1.0 / world)
                else:
                    dist.all_reduce(g, group=group)
                    g.mul_(1.0 / world)


class MixedPrecisionAdamW:
    """AdamW on fp32 master weights with bf16 working copies (one fused kernel per tensor), gradients accumulated
    in fp32 across micro-batches.

    `zero1_group`: ZeRO-1 over that data-parallel group for the replicated (non-expert) parameters, in the reference's
    form (crates/distributed/src/zero.rs:72-123): every such parameter has one owner rank (round-robin in name
    order); only the owner keeps its fp32 master copy and Adam moments and runs the update, then broadcasts the new
    bf16 values.  Expert parameters are already unique to their rank and are always updated locally."""

    def __init__(self, model: ParallelDecoderLM, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, zero1_group=None, use_zero1: bool = False):
        self.model, self.lr, self.betas, self.eps, self.wd = model, lr, betas, eps, weight_decay
        self.zero1 = use_zero1
        self.zero1_group = zero1_group
        self.owner: dict = {}
        if use_zero1:
            world, rank = dist.get_world_size(zero1_group), dist.get_rank(zero1_group)
            dense = [n for n in sorted(model.params) if n not in model.expert_names]
            self.owner = {n: i % world for i, n in enumerate(dense)}
            self._rank = rank
        owned = lambda n: (not use_zero1) or n in model.expert_names or self.owner[n] == self._rank
        self.master = {n: p.detach().float() for n, p in model.params.items() if owned(n)}
        self.m = {n: torch.zeros_like(v) for n, v in self.master.items()}
        self.v = {n: torch.zeros_like(v) for n, v in self.master.items()}
        self.main_grads = {n: torch.zeros(p.shape, dtype=torch.float32, device=p.device) for n, p in model.params.items()}
        self.step_count = 0

    def state_bytes(self) -> int:
        """Bytes of optimizer state held by this rank (master weights + both moments)."""
        return sum(3 * v.numel() * 4 for v in self.master.values())

    def accumulate(self) -> None:
        """Fold the bf16 `.grad` of the micro-batch just finished into the fp32 accumulators."""
        for n, p in self.model.params.items():
            if p.grad is not None:
                self.main_grads[n].add_(p.grad)
                p.grad = None

    def step(self, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        self.model.sync_grads(self.main_grads)
        for n, p in self.model.params.items():
            if n in self.master:
                decay = self.wd if p.dim() >= 2 else 0.0
                ops.adam_step(self.master[n].view(-1), self.m[n].view(-1), self.v[n].view(-1), self.main_grads[n].view(-1),
                              lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=decay,
                              step=self.step_count, grad_scale=grad_scale, p_lowp=p.data.view(-1))
            self.main_grads[n].zero_()
        if self.zero1:
            for n in sorted(self.owner):                      # the owner publishes the updated working copy
                src = self.owner[n]
                if self.zero1_group is not None:
                    src = dist.get_global_rank(self.zero1_group, src)
                dist.broadcast(self.model.params[n].data, src=src, group=self.zero1_group)
