"""Data-parallel training over a ProcessGroup (crates/distributed/src/lib.rs:311-488).

Gradients of all parameters are flattened into buckets (25 MiB by default) and each bucket takes one all-reduce,
instead of the reference's one blocking all-reduce per parameter (lib.rs:378-386)."""
from __future__ import annotations

import torch

from .process_group import ProcessGroup


def bucketize(tensors, bucket_bytes: int = 25 << 20) -> list:
    buckets, cur, size = [], [], 0
    for t in tensors:
        n = t.numel() * t.element_size()
        if cur and size + n > bucket_bytes:
            buckets.append(cur)
            cur, size = [], 0
        cur.append(t)
        size += n
    if cur:
        buckets.append(cur)
    return buckets


def all_reduce_gradients(pg: ProcessGroup, grads, average: bool = True, bucket_bytes: int = 25 << 20) -> None:
    """In-place bucketed all-reduce of a list of gradient tensors."""
    if pg.world_size == 1:
        return
    for bucket in bucketize([g for g in grads if g is not None], bucket_bytes):
        flat = torch.cat([g.reshape(-1).float() for g in bucket])
        pg.all_reduce_sum(flat, "grad_bucket")
        if average:
            flat.div_(pg.world_size)
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g).to(g.dtype))
            off += n


class DataParallelTrainer:
    def __init__(self, process_group: ProcessGroup, optimizer, bucket_bytes: int = 25 << 20):
        self.pg, self.optimizer, self.bucket_bytes = process_group, optimizer, bucket_bytes

    def split_batch(self, batch) -> list:
        """Round-robin: sample i goes to rank i % world (lib.rs:415)."""
        return [s for i, s in enumerate(batch) if i % self.pg.world_size == self.pg.rank]

    def step(self, params, batch, loss_fn, ctx=None) -> float:
        """loss_fn(local_batch, ctx) -> scalar loss tensor (mean over the local batch) with autograd attached to
        `params`.  Returns the global mean loss."""
        local = self.split_batch(batch)
        for p in params:
            p.zero_grad()
        loss = loss_fn(local, ctx)
        loss.backward()
        grads = [p.tensor.grad for p in params]
        all_reduce_gradients(self.pg, grads, True, self.bucket_bytes)
        self.optimizer.step(params)
        l = loss.detach().float().reshape(1).clone()
        self.pg.all_reduce_mean(l, "loss")
        return float(l)


class GradientAccumulator:
    """Accumulates gradients over micro-steps; `all_reduce` averages over world x steps."""

    def __init__(self, process_group: ProcessGroup | None = None):
        self.pg = process_group
        self.acc: dict = {}
        self.steps = 0

    def accumulate(self, named_grads: dict) -> None:
        for k, g in named_grads.items():
            if k in self.acc:
                self.acc[k] += g.float()
            else:
                self.acc[k] = g.detach().float().clone()
        self.steps += 1

    def all_reduce(self) -> dict:
        world = self.pg.world_size if self.pg else 1
        keys = sorted(self.acc)
        if self.pg and world > 1:
            all_reduce_gradients(self.pg, [self.acc[k] for k in keys], average=False)
        for k in keys:
            self.acc[k].div_(world * max(1, self.steps))
        return self.acc

    def reset(self) -> None:
        self.acc.clear()
        self.steps = 0
