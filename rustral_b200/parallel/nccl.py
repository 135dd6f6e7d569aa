"""NCCL communicator facade (crates/distributed/src/nccl.rs:159-487: NcclCommunicator, NcclProcessGroup,
NcclCompressedCommunicator).

The reference declares the NCCL C API itself and hands it host pointers on a null stream (nccl.rs:240-249), which a
real NCCL rejects.  Here the communicator is torch.distributed's NCCL backend (device tensors, the current stream),
and it is the baseline transport: the fused peer-memory kernels of this package are measured against it.  On CPU
tensors (gloo) the same calls work, which is how the host-side logic is tested.
"""
from __future__ import annotations

import enum
import torch
import torch.distributed as dist

from .compression import CompressedCommunicator, CompressionType
from .process_group import DistributedError, ProcessGroup

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT}


class NcclDataType(enum.IntEnum):
    """NCCL's element types with NCCL's own numbering (crates/distributed/src/nccl.rs:35-46)."""
    INT8 = 0
    UINT8 = 1
    INT32 = 2
    UINT32 = 3
    INT64 = 4
    UINT64 = 5
    FLOAT16 = 6
    FLOAT32 = 7
    FLOAT64 = 8
    BFLOAT16 = 9

    @classmethod
    def of(cls, dtype: torch.dtype) -> "NcclDataType":
        table = {torch.int8: cls.INT8, torch.uint8: cls.UINT8, torch.int32: cls.INT32, torch.int64: cls.INT64,
                 torch.float16: cls.FLOAT16, torch.float32: cls.FLOAT32, torch.float64: cls.FLOAT64, torch.bfloat16: cls.BFLOAT16}
        if dtype not in table:
            raise DistributedError(f"no NCCL element type for {dtype}")
        return table[dtype]

    def size_bytes(self) -> int:
        return {0: 1, 1: 1, 2: 4, 3: 4, 4: 8, 5: 8, 6: 2, 7: 4, 8: 8, 9: 2}[int(self)]


class NcclRedOp(enum.IntEnum):
    """crates/distributed/src/nccl.rs:63-69.  `NcclCommunicator.all_reduce` takes a member or its lower-case name."""
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3
    AVG = 4

    @property
    def op_name(self) -> str:
        return self.name.lower()


class NcclUniqueId:
    """The 128-byte token that rank 0 creates and every rank needs to join a communicator (nccl.rs:154-156).  With
    torch.distributed the exchange is the store's job; this object is the explicit form: `NcclUniqueId.create(store)` on
    rank 0 publishes random bytes under a key, `NcclUniqueId.fetch(store)` reads them elsewhere, and two ranks hold the
    same communicator exactly when their ids are equal."""

    KEY = "rustral_nccl_unique_id"

    def __init__(self, internal: bytes):
        if len(internal) != 128:
            raise DistributedError("an NCCL unique id is 128 bytes")
        self.internal = bytes(internal)

    @classmethod
    def create(cls, store=None) -> "NcclUniqueId":
        import os
        uid = cls(os.urandom(128))
        if store is not None:
            store.set(cls.KEY, uid.internal.hex())
        return uid

    @classmethod
    def fetch(cls, store) -> "NcclUniqueId":
        raw = store.get(cls.KEY)
        raw = raw.decode() if isinstance(raw, (bytes, bytearray)) else raw
        return cls(bytes.fromhex(raw))

    def __eq__(self, other):
        return isinstance(other, NcclUniqueId) and self.internal == other.internal

    def __hash__(self):
        return hash(self.internal)


class NcclComm:
    """Opaque handle of one communicator (nccl.rs:93-95): here the torch process group it wraps; `None` is the world."""

    def __init__(self, group=None):
        self.group = group


class NcclCommunicator:
    def __init__(self, group=None):
        if not dist.is_initialized():
            raise DistributedError("torch.distributed is not initialised")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    @staticmethod
    def version() -> str:
        try:
            return ".".join(str(v) for v in torch.cuda.nccl.version())
        except (RuntimeError, AttributeError, AssertionError):     # a torch build without NCCL, or no CUDA runtime
            return "unavailable"

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """In place.  "avg" divides once after the sum (the reference divides a second time on the host,
        nccl.rs:257-262)."""
        if isinstance(op, NcclRedOp):
            op = op.op_name
        if op == "avg":
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            return t.div_(self.world_size)
        dist.all_reduce(t, op=_OPS[op], group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if t.shape[0] % self.world_size:
            raise DistributedError("reduce_scatter: dim 0 must be divisible by the world size")
        out = torch.empty((t.shape[0] // self.world_size,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t.contiguous(), op=_OPS[op], group=self.group)
        return out

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        src = dist.get_global_rank(self.group, root) if self.group is not None else root
        dist.broadcast(t, src=src, group=self.group)
        return t

    def barrier(self) -> None:
        dist.barrier(group=self.group)


class NcclProcessGroup(ProcessGroup):
    """A ProcessGroup over an NCCL (or gloo) torch group that also exposes the raw communicator."""

    def __init__(self, group=None):
        super().__init__(dist.get_rank(group), dist.get_world_size(group), "torch", group=group)
        self.comm = NcclCommunicator(group)


class NcclCompressedCommunicator:
    """All-reduce with a compressed wire format (bf16 / fp16 cast, or the codecs of parallel/compression.py) around
    the NCCL collective (nccl.rs:426-487)."""

    def __init__(self, comm: NcclCommunicator, compression: CompressionType = CompressionType.BF16):
        self.comm = comm
        self.compression = compression
        # the other codecs (fp8, 1-bit, 4-bit with error feedback) go through the generic compressed communicator
        self._codec = CompressedCommunicator(ProcessGroup.from_torch(comm.group), compression)

    def all_reduce_mean(self, t: torch.Tensor) -> torch.Tensor:
        if self.compression in (CompressionType.BF16, CompressionType.FP16):
            wire = t.to(torch.bfloat16 if self.compression is CompressionType.BF16 else torch.float16)
            self.comm.all_reduce(wire, "sum")
            return t.copy_(wire.to(t.dtype)).div_(self.comm.world_size)
        if self.compression is CompressionType.NONE:
            return self.comm.all_reduce(t, "avg")
        self._codec.all_reduce_sum(t)
        return t.div_(self.comm.world_size)
