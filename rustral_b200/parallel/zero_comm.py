"""Gradient reduction + sharded optimizer step + parameter gather for data-parallel ranks (ZeRO).

Two interchangeable implementations behind one interface:

* ``NcclZeroComm``  -- library collectives (reduce-scatter, all-gather over NCCL, or gloo for CPU ranks).  This is
  the measured baseline and the path CPU-rank tests use.
* ``FusedZeroComm`` -- the peer-memory kernels of ``csrc/comm``: every rank reads its gradient shard from all
  peers over NVLink, reduces in fp32, applies AdamW to its fp32 master shard and pushes the updated bf16
  parameters into every peer's working copy, all in one kernel (see rustral_b200/parallel/symm.py).

Shard geometry: the flat parameter index space is padded to a multiple of world * 128 and cut into equal
contiguous ranges, rank r owning [r * n/W, (r+1) * n/W) (the reference shards by flat index as well,
crates/distributed/src/fsdp.rs:199-210, handing the remainder to the first ranks instead of padding).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops


class NcclZeroComm:
    def __init__(self, trainer):
        self.t = trainer
        P = trainer.engine.params
        self.grad_shard = torch.zeros(trainer.shard_len, dtype=torch.float32, device=trainer.device)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=trainer.device)
        self.norm = torch.zeros((), dtype=torch.float32, device=trainer.device)

    def reduce_and_step(self, loss: torch.Tensor, lr):
        t = self.t
        eng, P = t.engine, t.engine.params
        pg = t.pg
        # gradients: sum over ranks, each rank keeps its shard
        if P.grad.is_cuda:
            dist.reduce_scatter_tensor(self.grad_shard, P.grad, op=dist.ReduceOp.SUM, group=pg)
        else:   # gloo has no reduce-scatter: all-reduce and keep the shard
            dist.all_reduce(P.grad, group=pg)
            self.grad_shard.copy_(P.grad[t.shard])
        P.grad[t.shard].copy_(self.grad_shard)
        # global gradient norm from the shards
        ops.sumsq(self.grad_shard, out=self.norm_sq.view(()))
        dist.all_reduce(self.norm_sq, group=pg)
        ops.optim.sqrt_scalar(self.norm_sq.view(()), out=self.norm)
        eng.optimizer_step(lr, shard=t.shard, grad_norm=self.norm)
        # parameters: every rank gathers the updated working copy
        if P.lowp.is_cuda:
            dist.all_gather_into_tensor(P.lowp, P.lowp[t.shard].clone(), group=pg)
        else:
            parts = [torch.empty(t.shard_len, dtype=P.lowp.dtype) for _ in range(t.world)]
            dist.all_gather(parts, P.lowp[t.shard].clone(), group=pg)
            P.lowp.copy_(torch.cat(parts))
        lbuf = loss.reshape(1).clone()
        dist.all_reduce(lbuf, group=pg)
        return lbuf.view(())


    def gather_master(self) -> None:
        """Every rank updated only its shard of the fp32 master copy: collect the shards (for checkpoints)."""
        t = self.t
        P = t.engine.params
        parts = [torch.empty(t.shard_len, dtype=torch.float32, device=P.master.device) for _ in range(t.world)]
        dist.all_gather(parts, P.master[t.shard].clone(), group=t.pg)
        P.master.copy_(torch.cat(parts))

    def reload_master(self) -> None:
        """Nothing to refresh: this path updates the shard of the full-size master buffer in place."""

    def optimizer_shard(self) -> tuple:
        """(m, v): Adam moments of this rank's flat shard (views of the full-size buffers)."""
        P = self.t.engine.params
        return P.m[self.t.shard], P.v[self.t.shard]

    def close(self) -> None:
        pass


def make_zero_comm(trainer, kind: str = "auto"):
    """"fused" / "auto" on a CUDA device: the peer-memory kernels, and an error if they cannot be set up (there is no
    quiet switch to the library path: a run that asked for the fused kernels either uses them or stops).  "nccl", or
    CPU ranks: library collectives."""
    if kind in ("auto", "fused") and trainer.device.type == "cuda":
        from .fused_zero import FusedZeroComm
        return FusedZeroComm(trainer)
    if kind == "fused":
        raise ValueError("the fused ZeRO kernels need CUDA devices")
    return NcclZeroComm(trainer)
