"""ZeRO-1 / ZeRO-2 optimizers over named Parameters (crates/distributed/src/zero.rs:24-345).

All parameters are viewed as one flat index space cut into `world` equal contiguous shards (padded); a rank keeps
Adam state only for its shard.  ZeRO-1: gradients are all-reduced, each rank updates its shard, parameters are
all-gathered.  ZeRO-2: gradients are reduce-scattered, so a rank only ever holds its shard of the reduced
gradient (the reference all-reduces a copy and discards it, zero.rs:265-278, and broadcasts every parameter from
its owner one by one, :104-123).  The GPU hot path of the language-model trainer uses the fused kernels of
rustral_b200/parallel/fused_zero.py; this class is the general-purpose optimizer for arbitrary models.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from .process_group import ProcessGroup


class ZeroOptimizer:
    stage = 1

    def __init__(self, named_params, process_group: ProcessGroup, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, decoupled: bool = True):
        self.named = list(named_params)
        self.pg = process_group
        self.lr, self.betas, self.eps, self.weight_decay, self.decoupled = lr, betas, eps, weight_decay, decoupled
        W = self.pg.world_size
        self.total = sum(p.numel() for _, p in self.named)
        self.padded = (self.total + W - 1) // W * W
        self.shard_len = self.padded // W
        self.lo = self.pg.rank * self.shard_len
        dev = self.named[0][1].tensor.device
        flat = self._flatten([p.tensor.detach().float() for _, p in self.named], dev)
        self.master = flat[self.lo:self.lo + self.shard_len].clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.t = 0

    def _flatten(self, tensors, dev):
        flat = torch.zeros(self.padded, dtype=torch.float32, device=dev)
        off = 0
        for t in tensors:
            flat[off:off + t.numel()] = t.reshape(-1)
            off += t.numel()
        return flat

    def _grad_shard(self, flat_grad):
        self.pg.all_reduce_sum(flat_grad, "zero1_grads")
        flat_grad.div_(self.pg.world_size)
        return flat_grad[self.lo:self.lo + self.shard_len]

    def step(self) -> None:
        dev = self.master.device
        grads = [(p.tensor.grad if p.tensor.grad is not None else torch.zeros_like(p.tensor)).detach().float()
                 for _, p in self.named]
        g = self._grad_shard(self._flatten(grads, dev)).contiguous()
        self.t += 1
        ops.adam_step(self.master, self.m, self.v, g, lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                      weight_decay=self.weight_decay, step=self.t, decoupled=self.decoupled)
        full = torch.cat(self.pg.all_gather(self.master))
        off = 0
        with torch.no_grad():
            for _, p in self.named:
                n = p.numel()
                p.tensor.copy_(full[off:off + n].view(p.shape).to(p.tensor.dtype))
                off += n

    def zero_grad(self) -> None:
        for _, p in self.named:
            p.zero_grad()

    # ---- checkpoints: keyed by rank + flat range, reloadable on the same world size ------------------------------
    def save_checkpoint(self) -> dict:
        return {"rank": self.pg.rank, "world_size": self.pg.world_size, "t": self.t, "lr": self.lr,
                "master": self.master.cpu(), "m": self.m.cpu(), "v": self.v.cpu(), "shard": [self.lo, self.shard_len]}

    def load_checkpoint(self, ck: dict) -> None:
        from .process_group import RankMismatch
        if ck["world_size"] != self.pg.world_size or ck["rank"] != self.pg.rank:
            raise RankMismatch("ZeRO checkpoint belongs to another rank / world size")
        dev = self.master.device
        self.master, self.m, self.v = ck["master"].to(dev), ck["m"].to(dev), ck["v"].to(dev)
        self.t, self.lr = ck["t"], ck["lr"]


class Zero2Optimizer(ZeroOptimizer):
    stage = 2

    def _grad_shard(self, flat_grad):
        shard = self.pg.reduce_scatter(flat_grad)
        shard.div_(self.pg.world_size)
        return shard


@dataclass
class ZeroMemoryStats:
    """Bytes per rank for P parameters, bf16 working copy + fp32 master + two Adam moments (zero.rs:286-345)."""
    params: float
    grads: float
    optimizer: float

    @property
    def total(self) -> float:
        return self.params + self.grads + self.optimizer

    @classmethod
    def baseline(cls, P: int):
        return cls(2.0 * P, 4.0 * P, 12.0 * P)

    @classmethod
    def zero1(cls, P: int, W: int):
        return cls(2.0 * P, 4.0 * P, 12.0 * P / W)

    @classmethod
    def zero2(cls, P: int, W: int):
        return cls(2.0 * P, 4.0 * P / W, 12.0 * P / W)

    @classmethod
    def zero3(cls, P: int, W: int):
        return cls(2.0 * P / W, 4.0 * P / W, 12.0 * P / W)


@dataclass
class ZeRoMemoryStats:
    """Per-rank megabytes under the reference's accounting (crates/distributed/src/zero.rs:286-345): parameters of
    `param_size_bytes` each, Adam's two moments of the same size, gradients of the same size; `memory_saved_percent` is
    against holding all of it on every rank.  `ZeroMemoryStats` above is this package's own bf16 + fp32-master model."""
    local_params_mb: float
    local_optimizer_states_mb: float
    local_gradients_mb: float
    total_params_mb: float
    memory_saved_percent: float

    @classmethod
    def _make(cls, total_params: int, param_size_bytes: int, world_size: int, shard_grads: bool, shard_params: bool = True):
        mb = total_params * param_size_bytes / (1024.0 * 1024.0)
        lp = mb / world_size if shard_params else mb
        lo = 2.0 * mb / world_size
        lg = mb / world_size if shard_grads else mb
        return cls(lp, lo, lg, mb, (1.0 - (lp + lo + lg) / (4.0 * mb)) * 100.0 if mb else 0.0)

    @classmethod
    def zero1(cls, total_params: int, param_size_bytes: int, world_size: int):
        return cls._make(total_params, param_size_bytes, world_size, shard_grads=False)

    @classmethod
    def zero2(cls, total_params: int, param_size_bytes: int, world_size: int):
        return cls._make(total_params, param_size_bytes, world_size, shard_grads=True)


@dataclass
class ZeroCheckpoint:
    """A rank's optimizer shard as a typed record (crates/distributed/src/zero.rs:208-217): `ZeroCheckpoint.of(opt)` wraps
    `opt.save_checkpoint()`, `restore(opt)` loads it back and refuses another rank or world size."""
    rank: int
    world_size: int
    inner: dict

    @classmethod
    def of(cls, opt: ZeroOptimizer) -> "ZeroCheckpoint":
        ck = opt.save_checkpoint()
        return cls(ck["rank"], ck["world_size"], ck)

    def restore(self, opt: ZeroOptimizer) -> None:
        opt.load_checkpoint(self.inner)
