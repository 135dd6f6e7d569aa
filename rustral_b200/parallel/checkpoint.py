"""Distributed checkpoints (crates/distributed/src/checkpoint.rs:20-363).

Directory layout: <dir>/epoch_<E>/{rank_<R>.safetensors, optimizer_rank_<R>.json, metadata.json}; the primary
rank writes metadata.json {epoch, step, world_size, timestamp, version}; keep-last-N rotation.  Optimizer state is
keyed by parameter name.  Loading on a different world size re-shards flat ZeRO state (`reshard_flat`); the
reference refuses any world-size change (checkpoint.rs:157-163).
"""
from __future__ import annotations

import json
import os
import shutil
import time
from dataclasses import dataclass

import torch

from ..core.errors import SerializationError
from ..io import safetensors_io as st
from .process_group import ProcessGroup, RankMismatch


@dataclass
class CheckpointMetadata:
    epoch: int
    step: int
    world_size: int
    timestamp: float
    version: str = "1.0"


class DistributedCheckpointManager:
    def __init__(self, process_group: ProcessGroup, checkpoint_dir: str, keep_last_n: int = 3):
        self.pg, self.dir, self.keep_last_n = process_group, checkpoint_dir, keep_last_n
        os.makedirs(checkpoint_dir, exist_ok=True)

    def _epoch_dir(self, epoch: int) -> str:
        return os.path.join(self.dir, f"epoch_{epoch}")

    def save(self, epoch: int, step: int, named_tensors, optimizer_state: dict | None = None) -> str:
        """named_tensors: iterable of (name, Parameter | Tensor) holding THIS rank's state."""
        d = self._epoch_dir(epoch)
        os.makedirs(d, exist_ok=True)
        self.pg.barrier()
        tensors = {n: (p.tensor if hasattr(p, "tensor") else p).detach().cpu() for n, p in named_tensors}
        st.save_file(tensors, os.path.join(d, f"rank_{self.pg.rank}.safetensors"))
        if optimizer_state is not None:
            tmp = os.path.join(d, f"optimizer_rank_{self.pg.rank}.json.partial")
            with open(tmp, "w") as f:
                json.dump(optimizer_state, f)
            os.replace(tmp, os.path.join(d, f"optimizer_rank_{self.pg.rank}.json"))
        self.pg.barrier()
        if self.pg.is_primary():
            meta = CheckpointMetadata(epoch, step, self.pg.world_size, time.time())
            tmp = os.path.join(d, "metadata.json.partial")
            with open(tmp, "w") as f:
                json.dump(meta.__dict__, f)
            os.replace(tmp, os.path.join(d, "metadata.json"))
            self._rotate()
        self.pg.barrier()
        return d

    def save_async(self, epoch: int, step: int, named_tensors, writer: "AsyncCheckpointWriter",
                   optimizer_state: dict | None = None) -> str:
        """Snapshots THIS rank's state into host memory and queues its files on `writer`; returns without waiting for
        the disk, so training continues while the files are written.  The checkpoint only counts once
        `finish_async(epoch, step, writer)` has run: it flushes the writer, and after a barrier the primary rank writes
        metadata.json, the file whose presence marks an epoch directory as complete."""
        d = self._epoch_dir(epoch)
        os.makedirs(d, exist_ok=True)
        tensors = {n: (p.tensor if hasattr(p, "tensor") else p).detach().to("cpu", copy=True) for n, p in named_tensors}
        writer.write(os.path.join(d, f"rank_{self.pg.rank}.safetensors"), st.save_state_dict_typed(tensors, {}))
        if optimizer_state is not None:
            writer.write(os.path.join(d, f"optimizer_rank_{self.pg.rank}.json"), json.dumps(optimizer_state).encode())
        return d

    def finish_async(self, epoch: int, step: int, writer: "AsyncCheckpointWriter") -> str:
        """Collective: waits for this rank's queued files, then publishes the checkpoint (metadata + rotation)."""
        d = self._epoch_dir(epoch)
        writer.flush()
        self.pg.barrier()
        if self.pg.is_primary():
            meta = CheckpointMetadata(epoch, step, self.pg.world_size, time.time())
            tmp = os.path.join(d, "metadata.json.partial")
            with open(tmp, "w") as f:
                json.dump(meta.__dict__, f)
            os.replace(tmp, os.path.join(d, "metadata.json"))
            self._rotate()
        self.pg.barrier()
        return d

    def load_shard(self, epoch: int) -> "ShardData":
        """This rank's tensors and optimizer state of `epoch` as one record."""
        _, tensors, opt = self.load(epoch)
        return ShardData(tensors, opt)

    def _rotate(self) -> None:
        eps = self.list_checkpoints()
        for e in eps[:-self.keep_last_n] if self.keep_last_n > 0 else []:
            shutil.rmtree(self._epoch_dir(e), ignore_errors=True)

    def list_checkpoints(self) -> list:
        out = []
        for name in os.listdir(self.dir):
            if name.startswith("epoch_") and os.path.exists(os.path.join(self.dir, name, "metadata.json")):
                try:
                    out.append(int(name[6:]))
                except ValueError:
                    pass
        return sorted(out)

    def latest_checkpoint(self):
        eps = self.list_checkpoints()
        return eps[-1] if eps else None

    def read_metadata(self, epoch: int) -> CheckpointMetadata:
        path = os.path.join(self._epoch_dir(epoch), "metadata.json")
        try:
            with open(path) as f:
                return CheckpointMetadata(**json.load(f))
        except (OSError, json.JSONDecodeError, TypeError) as e:
            raise SerializationError(f"cannot read {path}: {e}") from e

    def load(self, epoch: int, named_tensors=None, allow_reshard: bool = False):
        """Returns (step, tensors of this rank, optimizer state | None).  With `named_tensors` the loaded values are
        copied into them after a strict key / element-count check."""
        meta = self.read_metadata(epoch)
        if meta.world_size != self.pg.world_size and not allow_reshard:
            raise RankMismatch(f"checkpoint was written by {meta.world_size} ranks, this job has {self.pg.world_size}")
        d = self._epoch_dir(epoch)
        if meta.world_size == self.pg.world_size:
            tensors, _ = st.load_file(os.path.join(d, f"rank_{self.pg.rank}.safetensors"))
        else:
            shards = [st.load_file(os.path.join(d, f"rank_{r}.safetensors"))[0] for r in range(meta.world_size)]
            tensors = {k: reshard_flat([s[k] for s in shards], self.pg.world_size, self.pg.rank) for k in shards[0]}
        opt = None
        op = os.path.join(d, f"optimizer_rank_{self.pg.rank}.json")
        if os.path.exists(op) and meta.world_size == self.pg.world_size:
            with open(op) as f:
                opt = json.load(f)
        if named_tensors is not None:
            named = list(named_tensors)
            missing = [n for n, _ in named if n not in tensors]
            if missing:
                raise SerializationError(f"checkpoint is missing keys: {missing}")
            for n, p in named:
                dst = p.tensor if hasattr(p, "tensor") else p
                if dst.numel() != tensors[n].numel():
                    raise SerializationError(f"{n}: element count {tensors[n].numel()} != {dst.numel()}")
            with torch.no_grad():
                for n, p in named:
                    dst = p.tensor if hasattr(p, "tensor") else p
                    dst.copy_(tensors[n].reshape(dst.shape).to(dst.dtype))
        return meta.step, tensors, opt


def reshard_flat(old_shards: list, new_world: int, new_rank: int) -> torch.Tensor:
    """Equal contiguous shards of one flat buffer written by len(old_shards) ranks, re-cut for `new_world` ranks."""
    full = torch.cat([s.reshape(-1) for s in old_shards])
    per = (full.numel() + new_world - 1) // new_world
    padded = torch.zeros(per * new_world, dtype=full.dtype)
    padded[:full.numel()] = full
    return padded[new_rank * per:(new_rank + 1) * per].clone()


class AsyncCheckpointWriter:
    """Background checkpoint writer: `write(path, bytes)` returns at once; `flush()` waits; errors surface on flush
    (crates/distributed/src/checkpoint.rs:271-308).  The work is done by the C++ writer pool of the runtime library
    (csrc/runtime/async_writer.cpp): worker threads write "<path>.partial", fsync and rename, outside the
    interpreter lock.  `write_tensor` hands over a host tensor without copying it (pinned memory that a device-to-host
    copy has filled, for instance) and returns a ticket; the tensor is kept alive until the ticket has been waited on."""

    def __init__(self, num_threads: int = 2):
        from .. import _native as N
        self._lib = N.runtime()
        self._h = self._lib.rb_aw_create(int(num_threads))
        if not self._h:
            raise SerializationError("cannot start the asynchronous checkpoint writer")
        self._borrowed: dict = {}

    def write(self, path: str, blob) -> int:
        blob = bytes(blob)
        t = self._lib.rb_aw_submit_copy(self._h, os.fsencode(path), blob, len(blob))
        if t <= 0:
            raise SerializationError(f"asynchronous checkpoint writer refused {path}")
        return int(t)

    def write_tensor(self, path: str, tensor) -> int:
        """Queues the raw bytes of a contiguous host tensor; nothing is copied.  Do not modify the tensor until
        `wait(ticket)` or `flush()` has returned."""
        if tensor.is_cuda or not tensor.is_contiguous():
            raise SerializationError("write_tensor takes a contiguous host tensor")
        n = tensor.numel() * tensor.element_size()
        t = self._lib.rb_aw_submit_borrowed(self._h, os.fsencode(path), tensor.data_ptr(), n)
        if t <= 0:
            raise SerializationError(f"asynchronous checkpoint writer refused {path}")
        self._borrowed[int(t)] = tensor
        return int(t)

    def wait(self, ticket: int, timeout_s: float | None = None) -> bool:
        """True when the job has finished (successfully or not; `flush` reports failures)."""
        rc = self._lib.rb_aw_wait(self._h, int(ticket), -1 if timeout_s is None else int(timeout_s * 1000))
        if rc == 0:
            self._borrowed.pop(int(ticket), None)
        return rc == 0

    def pending(self) -> int:
        return int(self._lib.rb_aw_pending(self._h))

    def bytes_written(self) -> int:
        return int(self._lib.rb_aw_bytes_written(self._h))

    def flush(self) -> None:
        failed = self._lib.rb_aw_flush(self._h, -1)
        self._borrowed.clear()
        if failed > 0:
            import ctypes
            buf = ctypes.create_string_buffer(512)
            self._lib.rb_aw_take_error(self._h, buf, 512)
            raise SerializationError(f"asynchronous checkpoint write failed ({failed} job(s)): {buf.value.decode(errors='replace')}")

    def close(self) -> None:
        if self._h:
            try:
                self.flush()
            finally:
                self._lib.rb_aw_destroy(self._h)
                self._h = None

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.rb_aw_destroy(self._h)
                self._h = None
        except Exception:       # noqa: BLE001 - interpreter shutdown
            pass


@dataclass
class ShardData:
    """One rank's part of a sharded checkpoint: its named parameter shards and, optionally, its optimizer state
    (crates/distributed/src/checkpoint.rs:327-333).  `DistributedCheckpointManager.load_shard(epoch)` returns it."""
    params: dict
    optimizer: dict | None = None


class ShardedCheckpoint:
    """Gather per-rank shards into one full tensor on every rank, or cut a full tensor into this rank's shard."""

    def __init__(self, process_group: ProcessGroup):
        self.pg = process_group

    def gather(self, shard: torch.Tensor) -> torch.Tensor:
        return torch.cat(self.pg.all_gather(shard))

    def scatter(self, full: torch.Tensor) -> torch.Tensor:
        per = (full.shape[0] + self.pg.world_size - 1) // self.pg.world_size
        return full[self.pg.rank * per:(self.pg.rank + 1) * per].clone()
