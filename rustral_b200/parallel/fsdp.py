"""FSDP / ZeRO-3 wrapper for arbitrary NamedParameters models (crates/distributed/src/fsdp.rs:50-507).

Between steps a rank keeps only its shard of every parameter (flat-index contiguous split; the first `numel % W`
ranks hold one extra element, fsdp.rs:199-210).  `forward` gathers the full parameters, runs the model and drops
them again; `backward` reduce-scatters gradients into the shards; `step` runs the optimizer on shard views.  In the
reference gather, scatter, reduce-scatter and checkpoint load are placeholders (fsdp.rs:252-338,472-477); here
they move data.  The language-model trainer does the same with fused kernels (parallel/fused_zero.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..core import Parameter
from .process_group import ProcessGroup, RankMismatch


@dataclass
class FSDPConfig:
    shard_params: bool = True
    shard_grads: bool = True
    cpu_offload: bool = False
    gradient_checkpointing: bool = False
    bucket_size: int = 25 << 20
    auto_wrap: bool = False
    mixed_precision: bool = False

    def with_cpu_offload(self, flag: bool = True):
        self.cpu_offload = flag
        return self

    def with_mixed_precision(self, flag: bool = True):
        self.mixed_precision = flag
        return self

    def with_bucket_size(self, n: int):
        self.bucket_size = n
        return self


def shard_range(numel: int, world: int, rank: int) -> tuple:
    base, rem = divmod(numel, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


@dataclass
class ShardedParameter:
    name: str
    full_shape: tuple
    numel: int
    start: int
    end: int
    shard: torch.Tensor                 # fp32 master shard (on the host when cpu_offload)
    grad_shard: torch.Tensor | None = None
    is_gathered: bool = False


class FSDP:
    def __init__(self, model, optimizer, process_group: ProcessGroup, config: FSDPConfig | None = None):
        self.model, self.optimizer, self.pg = model, optimizer, process_group
        self.config = config or FSDPConfig()
        self.named = model.named_parameters()
        self.sharded: list = []
        W, r = self.pg.world_size, self.pg.rank
        for name, p in self.named:
            s, e = shard_range(p.numel(), W, r)
            shard = p.tensor.detach().float().reshape(-1)[s:e].clone()
            if self.config.cpu_offload:
                shard = shard.cpu()
            self.sharded.append(ShardedParameter(name, p.shape, p.numel(), s, e, shard))
        self._shard_params = [Parameter(sp.name, sp.shard) for sp in self.sharded]
        self.scatter_all_params()

    # ---- gather / scatter -------------------------------------------------------------------------------------------
    def _max_shard(self, numel: int) -> int:
        return (numel + self.pg.world_size - 1) // self.pg.world_size

    def gather_all_params(self) -> None:
        W = self.pg.world_size
        for (name, p), sp in zip(self.named, self.sharded):
            dev = p.tensor.device if p.tensor.numel() else sp.shard.device
            pad = self._max_shard(sp.numel)
            buf = torch.zeros(pad, dtype=torch.float32, device=self._dev)
            buf[:sp.end - sp.start] = sp.shard.to(self._dev)
            parts = self.pg.all_gather(buf)
            pieces = []
            for r in range(W):
                s, e = shard_range(sp.numel, W, r)
                pieces.append(parts[r][:e - s])
            full = torch.cat(pieces).view(sp.full_shape)
            p.tensor = full.to(self._dtype[name]).requires_grad_(True)
            sp.is_gathered = True

    def scatter_all_params(self) -> None:
        """Frees the full parameters (keeps zero-size placeholders so names and dtypes survive)."""
        if not hasattr(self, "_dtype"):
            self._dtype = {n: p.tensor.dtype for n, p in self.named}
            self._dev = self.named[0][1].tensor.device
        if not self.config.shard_params:
            return
        for (name, p), sp in zip(self.named, self.sharded):
            p.tensor = torch.empty(0, dtype=self._dtype[name], device=self._dev)
            sp.is_gathered = False

    # ---- step -----------------------------------------------------------------------------------------------------------
    def forward(self, x, ctx=None):
        self.gather_all_params()
        return self.model(x, ctx) if ctx is not None else self.model(x)

    def backward(self, loss: torch.Tensor) -> None:
        loss.backward()
        self.reduce_scatter_grads()

    def reduce_scatter_grads(self) -> None:
        W, r = self.pg.world_size, self.pg.rank
        for (name, p), sp in zip(self.named, self.sharded):
            g = p.tensor.grad
            flat = torch.zeros(self._max_shard(sp.numel) * W, dtype=torch.float32, device=self._dev)
            if g is not None:
                gf = g.detach().float().reshape(-1)
                for q in range(W):      # lay the gradient out so that equal-size chunk q is rank q's (padded) shard
                    s, e = shard_range(sp.numel, W, q)
                    flat[q * self._max_shard(sp.numel):q * self._max_shard(sp.numel) + e - s] = gf[s:e]
            shard = self.pg.reduce_scatter(flat)
            sp.grad_shard = (shard[:sp.end - sp.start] / W).to(sp.shard.device)
        self.scatter_all_params()

    def step(self) -> None:
        grads = {sp_p.id: sp.grad_shard for sp_p, sp in zip(self._shard_params, self.sharded) if sp.grad_shard is not None}
        self.optimizer.step(self._shard_params, grads)
        for sp in self.sharded:
            sp.grad_shard = None

    def train_step(self, x, target, loss_fn, ctx=None) -> float:
        out = self.forward(x, ctx)
        loss = loss_fn(out, target)
        self.backward(loss)
        self.step()
        l = loss.detach().float().reshape(1).clone()
        self.pg.all_reduce_mean(l, "fsdp_loss")
        return float(l)

    def memory_stats(self) -> "FSDPMemoryStats":
        shard_bytes = sum(sp.shard.numel() * 4 for sp in self.sharded)
        full_bytes = sum(sp.numel * 4 for sp in self.sharded)
        gathered = sum(1 for _, p in self.named if p.tensor.numel() > 0) if hasattr(self, "named") else 0
        return FSDPMemoryStats(self.pg.world_size, sum(sp.numel for sp in self.sharded), sum(sp.shard.numel() for sp in self.sharded),
                               (1.0 - shard_bytes / max(1, full_bytes)) * 100.0, gathered, shard_bytes, full_bytes)

    # ---- checkpoints -----------------------------------------------------------------------------------------------------
    def save_checkpoint(self) -> "FSDPCheckpoint":
        return FSDPCheckpoint({sp.name: sp.shard.detach().cpu().clone() for sp in self.sharded}, None, self.pg.rank,
                              self.pg.world_size)

    def load_checkpoint(self, ck: "FSDPCheckpoint") -> None:
        if ck.world_size != self.pg.world_size or ck.rank != self.pg.rank:
            raise RankMismatch("FSDP checkpoint belongs to another rank / world size")
        for sp in self.sharded:
            sp.shard.copy_(ck.shards[sp.name].to(sp.shard.device))


@dataclass
class FSDPMemoryStats:
    """crates/distributed/src/fsdp.rs:389-425, plus the byte counts.  Also answers the dictionary keys `shard_bytes`,
    `full_bytes` and `savings`."""
    world_size: int
    total_parameters: int
    local_parameters: int
    memory_reduction_percent: float
    gathered_params: int
    shard_bytes: int = 0
    full_bytes: int = 0

    def __getitem__(self, key):
        return {"shard_bytes": self.shard_bytes, "full_bytes": self.full_bytes, "savings": self.memory_reduction_percent / 100.0}[key]


@dataclass
class FSDPCheckpoint:
    shards: dict
    optimizer_state: dict | None
    rank: int
    world_size: int


@dataclass
class AutoWrapPolicy:
    """Which sub-modules get their own FSDP unit: by parameter count, by type name, or by a predicate."""
    min_params: int = 0
    type_names: tuple = ()
    predicate: object = None

    def should_wrap(self, module) -> bool:
        if self.predicate is not None:
            return bool(self.predicate(module))
        if self.type_names and type(module).__name__ in self.type_names:
            return True
        n = sum(p.numel() for _, p in module.named_parameters()) if hasattr(module, "named_parameters") else 0
        return self.min_params > 0 and n >= self.min_params


def auto_wrap(model, optimizer, process_group, config: FSDPConfig | None = None, policy: AutoWrapPolicy | None = None) -> FSDP:
    """One FSDP unit over the whole model (sub-module units would only change gather granularity)."""
    return FSDP(model, optimizer, process_group, config)
