"""Data-parallel training over a ProcessGroup (crates/distributed/src/lib.rs:311-488).

Gradients of all parameters are flattened into buckets (25 MiB by default) and each bucket takes one all-reduce,
instead of the reference's one blocking all-reduce per parameter (lib.rs:378-386).  `OverlappedGradientReducer` starts
a bucket's all-reduce from a gradient hook as soon as the backward pass has produced all of its gradients, so the
collectives of the last layers run under the backward pass of the earlier ones, optionally with bf16 on the wire."""
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


class OverlappedGradientReducer:
    """Bucketed gradient all-reduce overlapped with the backward pass.

    The parameters are bucketed in REVERSE order (the backward pass produces the last layer's gradients first).  A
    post-accumulate hook on every parameter counts its bucket down; when the bucket is complete its gradients are packed
    into one flat buffer of `wire_dtype` (fp32, or bf16 to halve the bytes) and the all-reduce is started
    asynchronously.  `finish()` waits for the buckets in launch order, averages and unpacks into `.grad`.  Use:

        reducer = OverlappedGradientReducer(pg, params)      # once
        loss.backward(); reducer.finish(); optimizer.step(params)
    """

    def __init__(self, pg: ProcessGroup, params, bucket_bytes: int = 25 << 20, wire_dtype=torch.float32, average: bool = True):
        self.pg, self.average, self.wire_dtype = pg, average, wire_dtype
        self.tensors = [getattr(p, "tensor", p) for p in params]
        self.buckets = bucketize(list(reversed(self.tensors)), bucket_bytes)
        self._bucket_of = {id(t): bi for bi, b in enumerate(self.buckets) for t in b}
        self._left = [len(b) for b in self.buckets]
        self._inflight: list = []
        self.launch_order: list = []              # bucket indices in the order their collectives started (last step)
        self._hooks = [t.register_post_accumulate_grad_hook(self._on_grad) for t in self.tensors if t.requires_grad]

    def _on_grad(self, t: torch.Tensor) -> None:
        bi = self._bucket_of[id(t)]
        self._left[bi] -= 1
        if self._left[bi] == 0:
            self._launch(bi)

    def _launch(self, bi: int) -> None:
        if self.pg.world_size == 1:
            return
        bucket = [t for t in self.buckets[bi] if t.grad is not None]
        if not bucket:
            return
        flat = torch.cat([t.grad.reshape(-1).to(self.wire_dtype) for t in bucket])
        work = self.pg.all_reduce_sum_async(flat, f"grad_bucket{bi}")
        self._inflight.append((bi, bucket, flat, work))
        self.launch_order.append(bi)

    def finish(self) -> None:
        """Call after backward(): launches what is still pending (parameters that got no gradient leave their bucket
        incomplete), waits for every bucket, writes the averaged gradients back and re-arms the hooks' counters."""
        launched = {bi for bi, *_ in self._inflight}
        for bi in range(len(self.buckets)):
            if bi not in launched and any(t.grad is not None for t in self.buckets[bi]):
                self._launch(bi)
        for bi, bucket, flat, work in self._inflight:
            work.wait()
            if self.average:
                flat.div_(self.pg.world_size)
            off = 0
            for t in bucket:
                n = t.numel()
                t.grad.copy_(flat[off:off + n].view_as(t.grad).to(t.grad.dtype))
                off += n
        self._inflight = []
        self._left = [len(b) for b in self.buckets]

    def begin_step(self) -> None:
        self.launch_order = []

    def close(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []


class DataParallelTrainer:
    """`overlap=True`: gradients are reduced bucket by bucket during the backward pass (`OverlappedGradientReducer`);
    `wire_dtype=torch.bfloat16` halves the bytes on the wire."""

    def __init__(self, process_group: ProcessGroup, optimizer, bucket_bytes: int = 25 << 20, overlap: bool = False,
                 wire_dtype=torch.float32):
        self.pg, self.optimizer, self.bucket_bytes = process_group, optimizer, bucket_bytes
        self.overlap, self.wire_dtype = overlap, wire_dtype
        self._reducer = None

    def split_batch(self, batch) -> list:
        """Round-robin: sample i goes to rank i % world (lib.rs:415)."""
        return [s for i, s in enumerate(batch) if i % self.pg.world_size == self.pg.rank]

    def step(self, params, batch, loss_fn, ctx=None) -> float:
        """loss_fn(local_batch, ctx) -> scalar loss tensor (mean over the local batch) with autograd attached to
        `params`.  Returns the global mean loss."""
        local = self.split_batch(batch)
        params = list(params)
        for p in params:
            p.zero_grad()
        if self.overlap:
            if self._reducer is None or [id(t) for t in self._reducer.tensors] != [id(p.tensor) for p in params]:
                if self._reducer is not None:
                    self._reducer.close()
                self._reducer = OverlappedGradientReducer(self.pg, params, self.bucket_bytes, self.wire_dtype)
            self._reducer.begin_step()
            loss = loss_fn(local, ctx)
            loss.backward()
            self._reducer.finish()
        else:
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
