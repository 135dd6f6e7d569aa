"""ProcessGroup: the collective verbs of the framework over torch.distributed (NCCL on GPUs, gloo on CPU ranks)
(crates/distributed/src/lib.rs:73-297).

Backends: `SingleProcess` (world of one, every verb is the identity), `Threaded` (ranks are threads of one process
sharing ONE rendezvous object, so sums really are sums: the reference's threaded groups each own a private map,
lib.rs:132-144) and `Torch` (a torch.distributed group).  On top of the reference's verbs (all_reduce_sum / mean,
all_gather, broadcast, barrier) this adds reduce_scatter, all_to_all, send and recv.
"""
from __future__ import annotations

import enum
import threading

import torch
import torch.distributed as dist

from ..core.errors import CoreError


class DistributedError(CoreError):
    pass


class RankMismatch(DistributedError):
    pass


class CommunicationError(DistributedError):
    pass


class _ThreadedRendezvous:
    """Shared state of a threaded group: a reusable barrier plus per-tag slots."""

    def __init__(self, world: int):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.lock = threading.Lock()
        self.slots: dict = {}
        self.mail: dict = {}
        self.mail_cv = threading.Condition()

    def exchange(self, tag: str, rank: int, value):
        """Every rank deposits `value`; all get the list of all values in rank order."""
        with self.lock:
            self.slots.setdefault(tag, [None] * self.world)[rank] = value
        self.barrier.wait()
        vals = list(self.slots[tag])
        self.barrier.wait()
        if rank == 0:
            with self.lock:
                self.slots.pop(tag, None)
        self.barrier.wait()
        return vals


class CommunicationBackend(enum.Enum):
    """The transports a `ProcessGroup` can sit on (crates/distributed/src/lib.rs:107-125: SingleProcess, Threaded, Mpi;
    here: one process, threads of one process sharing a rendezvous, or a torch.distributed group over gloo / NCCL).
    `ProcessGroup.backend` holds the member's value; `ProcessGroup.communication_backend` the member itself."""
    SINGLE_PROCESS = "single"
    THREADED = "threaded"
    TORCH = "torch"


class ProcessGroup:
    def __init__(self, rank: int, world_size: int, backend: str, group=None, rendezvous=None, timeout_s: float = 60.0):
        if not (0 <= rank < world_size):
            raise RankMismatch(f"rank {rank} outside world of {world_size}")
        self.rank, self.world_size, self.backend = rank, world_size, backend
        self.group = group
        self._rdv = rendezvous
        self._seq = 0
        self.timeout_s = timeout_s

    # ---- constructors --------------------------------------------------------------------------------------
    @classmethod
    def new_single_process(cls) -> "ProcessGroup":
        return cls(0, 1, "single")

    @classmethod
    def new_threaded(cls, world_size: int) -> list:
        """All ranks of a threaded group at once (they share one rendezvous)."""
        rdv = _ThreadedRendezvous(world_size)
        return [cls(r, world_size, "threaded", rendezvous=rdv) for r in range(world_size)]

    @classmethod
    def from_torch(cls, group=None) -> "ProcessGroup":
        if not dist.is_initialized():
            raise DistributedError("torch.distributed is not initialised")
        return cls(dist.get_rank(group), dist.get_world_size(group), "torch", group=group)

    @classmethod
    def new_torch_subgroup(cls, ranks) -> "ProcessGroup | None":
        """Collective over the default group: every rank must call it with the same `ranks`."""
        g = dist.new_group(list(ranks))
        me = dist.get_rank()
        if me not in ranks:
            return None
        return cls(list(ranks).index(me), len(ranks), "torch", group=g)

    def is_primary(self) -> bool:
        return self.rank == 0

    @property
    def communication_backend(self) -> "CommunicationBackend":
        return CommunicationBackend(self.backend) if self.backend in ("single", "threaded", "torch") else CommunicationBackend.TORCH

    def _tag(self, name: str) -> str:
        self._seq += 1
        return f"{name}#{self._seq}"

    # ---- collectives ------------------------------------------------------------------------------------------
    def all_reduce_sum(self, t: torch.Tensor, name: str = "") -> torch.Tensor:
        """In place."""
        if self.backend == "single":
            return t
        if self.backend == "threaded":
            vals = self._rdv.exchange(self._tag("ar:" + name), self.rank, t.detach().clone())
            acc = vals[0].clone()
            for v in vals[1:]:
                acc += v
            t.copy_(acc)
            return t
        try:
            dist.all_reduce(t, group=self.group)
        except RuntimeError as e:
            raise CommunicationError(str(e)) from e
        return t

    def all_reduce_sum_async(self, t: torch.Tensor, name: str = ""):
        """Starts an in-place sum; returns a handle with `wait()`.  Over torch.distributed the collective runs on the
        backend's own stream / thread while the caller goes on (the handle's `wait` orders the current stream behind it);
        the threaded and single-process groups complete at once."""
        if self.backend in ("single", "threaded"):
            self.all_reduce_sum(t, name)

            class _Done:
                def wait(self_inner):
                    return True
            return _Done()
        try:
            return dist.all_reduce(t, group=self.group, async_op=True)
        except RuntimeError as e:
            raise CommunicationError(str(e)) from e

    def all_reduce_mean(self, t: torch.Tensor, name: str = "") -> torch.Tensor:
        self.all_reduce_sum(t, name)
        t.div_(self.world_size)
        return t

    all_reduce_mean_f32 = all_reduce_mean

    def barrier(self) -> None:
        if self.backend == "single":
            return
        if self.backend == "threaded":
            self._rdv.barrier.wait(self.timeout_s)
            return
        dist.barrier(group=self.group)

    def all_gather(self, t: torch.Tensor) -> list:
        if self.backend == "single":
            return [t]
        if self.backend == "threaded":
            return self._rdv.exchange(self._tag("ag"), self.rank, t.detach().clone())
        outs = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(outs, t.contiguous(), group=self.group)
        return outs

    def all_gather_into(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return torch.cat(self.all_gather(t), dim)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self.backend == "single":
            return t
        if self.backend == "threaded":
            vals = self._rdv.exchange(self._tag("bc"), self.rank, t.detach().clone() if self.rank == root else None)
            t.copy_(vals[root])
            return t
        dist.broadcast(t, src=dist.get_global_rank(self.group, root) if self.group is not None else root, group=self.group)
        return t

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sums `t` (length divisible by world) over ranks; returns this rank's contiguous shard."""
        n = t.shape[0]
        if n % self.world_size:
            raise DistributedError("reduce_scatter: leading dimension must be divisible by the world size")
        per = n // self.world_size
        if self.backend == "single":
            return t.clone()
        if self.backend == "torch" and t.is_cuda:
            out = torch.empty((per, *t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
            return out
        full = self.all_reduce_sum(t.clone())
        return full[self.rank * per:(self.rank + 1) * per].clone()

    def all_to_all(self, chunks: list) -> list:
        """chunks[r] goes to rank r; returns what every rank sent to this one (in rank order)."""
        if len(chunks) != self.world_size:
            raise DistributedError("all_to_all needs one chunk per rank")
        if self.backend == "single":
            return [chunks[0]]
        if self.backend == "threaded":
            table = self._rdv.exchange(self._tag("a2a"), self.rank, [c.detach().clone() for c in chunks])
            return [table[src][self.rank] for src in range(self.world_size)]
        if chunks[0].is_cuda:
            sizes = torch.tensor([c.shape[0] for c in chunks], device=chunks[0].device)
            all_sizes = [torch.empty_like(sizes) for _ in range(self.world_size)]
            dist.all_gather(all_sizes, sizes, group=self.group)
            outs = [torch.empty((int(all_sizes[src][self.rank]), *chunks[0].shape[1:]), dtype=chunks[0].dtype,
                                device=chunks[0].device) for src in range(self.world_size)]
            dist.all_to_all(outs, [c.contiguous() for c in chunks], group=self.group)
            return outs
        gathered = [None] * self.world_size          # gloo: object exchange
        dist.all_gather_object(gathered, [c.cpu() for c in chunks], group=self.group)
        return [gathered[src][self.rank] for src in range(self.world_size)]

    def send(self, t: torch.Tensor, dst: int, tag: int = 0) -> None:
        if self.backend == "threaded":
            with self._rdv.mail_cv:
                self._rdv.mail.setdefault((self.rank, dst, tag), []).append(t.detach().clone())
                self._rdv.mail_cv.notify_all()
            return
        if self.backend == "single":
            raise DistributedError("send in a world of one")
        dist.send(t.contiguous(), dist.get_global_rank(self.group, dst) if self.group is not None else dst, group=self.group, tag=tag)

    def recv(self, t: torch.Tensor, src: int, tag: int = 0) -> torch.Tensor:
        if self.backend == "threaded":
            key = (src, self.rank, tag)
            with self._rdv.mail_cv:
                ok = self._rdv.mail_cv.wait_for(lambda: self._rdv.mail.get(key), timeout=self.timeout_s)
                if not ok:
                    raise CommunicationError(f"recv from {src} timed out")
                t.copy_(self._rdv.mail[key].pop(0))
            return t
        if self.backend == "single":
            raise DistributedError("recv in a world of one")
        dist.recv(t, dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group, tag=tag)
        return t
