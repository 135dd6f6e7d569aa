"""Dataset abstractions and the batching loader (crates/data/src/lib.rs)."""
from __future__ import annotations

import ctypes as C
import mmap
import os
import queue
import random
import threading
from dataclasses import dataclass

import numpy as np
import torch

from .. import _native as N


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def get(self, i: int):
        raise NotImplementedError

    def get_batch(self, indices) -> list:
        return [self.get(i) for i in indices]

    def __getitem__(self, i):
        return self.get(i)


class InMemoryDataset(Dataset):
    def __init__(self, items):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def get(self, i):
        return self.items[i]


class StreamingDataset(Dataset):
    """One record per line of a text file.  Line offsets are indexed once, so `get` is a seek, not a rescan
    (the reference re-opens the file and scans to line N on every get)."""

    def __init__(self, path: str, parse=lambda line: line):
        self.path, self.parse = path, parse
        self._offsets = [0]
        with open(path, "rb") as f:
            for line in f:
                self._offsets.append(self._offsets[-1] + len(line))
        self._offsets.pop()
        self._local = threading.local()

    def __len__(self):
        return len(self._offsets)

    def get(self, i):
        f = getattr(self._local, "f", None)
        if f is None:
            f = self._local.f = open(self.path, "rb")
        f.seek(self._offsets[i])
        return self.parse(f.readline().decode("utf-8").rstrip("\n"))


class MmapDataset(Dataset):
    """Fixed-size binary records in a memory-mapped file; `get_f32_slice` views a record as float32."""

    def __init__(self, path: str, element_size: int):
        self.path, self.element_size = path, element_size
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) % element_size:
            raise ValueError("file size is not a multiple of the element size")

    def __len__(self):
        return len(self._mm) // self.element_size

    def get(self, i) -> bytes:
        if not (0 <= i < len(self)):
            raise IndexError(i)
        return self._mm[i * self.element_size:(i + 1) * self.element_size]

    def get_f32_slice(self, i) -> np.ndarray:
        return np.frombuffer(self.get(i), dtype=np.float32)

    def close(self):
        self._mm.close()
        self._f.close()


class TokenFileDataset:
    """Flat file of token ids (uint16 or int32) served by the C++ memory-mapped reader (csrc/runtime/token_file.cpp):
    `batch(step)` returns int64 [batch, seq_len + 1] windows at seeded uniform offsets, in pinned memory on request."""

    def __init__(self, path: str, seq_len: int, bytes_per_token: int = 2, seed: int = 0):
        self._lib = N.runtime()
        self._h = self._lib.rb_tokens_open(path.encode(), bytes_per_token)
        if not self._h:
            raise OSError(f"cannot open token file {path}")
        self.seq_len, self.seed = seq_len, seed
        self.num_tokens = int(self._lib.rb_tokens_len(self._h))

    def batch(self, step: int, batch_size: int, pin: bool = False) -> torch.Tensor:
        n = self.seq_len + 1
        offs = (C.c_int64 * batch_size)()
        self._lib.rb_tokens_sample_offsets(self._h, self.seed, step, batch_size, n, offs)
        out = torch.empty((batch_size, n), dtype=torch.int64, pin_memory=pin and torch.cuda.is_available())
        rc = self._lib.rb_tokens_gather(self._h, offs, batch_size, n, out.data_ptr())
        if rc != 0:
            raise IndexError("token window out of range")
        return out

    def prefetcher(self, batch_size: int, depth: int = 3, first_step: int = 0, pin: bool | None = None) -> "TokenBatchPrefetcher":
        """Batches of consecutive steps gathered by a native worker thread into `depth` (pinned) buffers, ahead of the
        consumer; the data of step s equals `batch(s, batch_size)`."""
        return TokenBatchPrefetcher(self, batch_size, depth, first_step, pin)

    def close(self):
        if self._h:
            self._lib.rb_tokens_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001 - interpreter shutdown: the library or its handle may already be gone
            pass


@dataclass
class DataLoaderConfig:
    batch_size: int = 32
    shuffle: bool = False
    seed: int = 0
    num_workers: int = 0
    drop_last: bool = False


class DataLoader:
    """Batches of items; reshuffles (seed + epoch) on `reset`."""

    def __init__(self, dataset: Dataset, config: DataLoaderConfig):
        self.dataset, self.config = dataset, config
        self.epoch = 0
        self._order = []
        self._pos = 0
        self.reset(first=True)

    def reset(self, first: bool = False) -> None:
        if not first:
            self.epoch += 1
        self._order = list(range(len(self.dataset)))
        if self.config.shuffle:
            random.Random(self.config.seed + self.epoch).shuffle(self._order)
        self._pos = 0

    def num_batches(self) -> int:
        n, b = len(self.dataset), self.config.batch_size
        return n // b if self.config.drop_last else (n + b - 1) // b

    def next_batch(self):
        b = self.config.batch_size
        if self._pos >= len(self._order):
            return None
        idx = self._order[self._pos:self._pos + b]
        if self.config.drop_last and len(idx) < b:
            return None
        self._pos += b
        return self.dataset.get_batch(idx)

    def __iter__(self):
        self.reset(first=(self._pos == 0 and self.epoch == 0))
        while True:
            batch = self.next_batch()
            if batch is None:
                return
            yield batch


def simple_loader(items, batch_size: int) -> DataLoader:
    return DataLoader(InMemoryDataset(items), DataLoaderConfig(batch_size))


def shuffled_loader(items, batch_size: int, seed: int = 0) -> DataLoader:
    return DataLoader(InMemoryDataset(items), DataLoaderConfig(batch_size, True, seed))


class TokenBatchPrefetcher:
    """Handle on the native prefetcher (csrc/runtime/prefetch.cpp).  `next()` returns (tokens, step): a view of one of
    the ring's buffers, valid until `release(tokens)` (or the next `next()`, which releases the previous batch unless
    `hold=True` was passed).  Typical loop: `t, _ = pf.next(); dev = t.to("cuda", non_blocking=True); ...` and release
    after the copy has been ordered before the next use of the stream."""

    def __init__(self, dataset: "TokenFileDataset", batch_size: int, depth: int = 3, first_step: int = 0, pin: bool | None = None):
        self._ds, self._lib = dataset, dataset._lib
        n = dataset.seq_len + 1
        pin = torch.cuda.is_available() if pin is None else (pin and torch.cuda.is_available())
        self._bufs = [torch.empty((batch_size, n), dtype=torch.int64, pin_memory=pin) for _ in range(depth)]
        ptrs = (C.c_void_p * depth)(*[b.data_ptr() for b in self._bufs])
        self._h = self._lib.rb_prefetch_create(dataset._h, dataset.seed, first_step, batch_size, n, depth, ptrs)
        if not self._h:
            raise ValueError("TokenBatchPrefetcher: bad sizes (file shorter than one window, depth outside 1..64, ...)")
        self._held: list = []
        self._auto = None

    def next(self, timeout_s: float | None = None, hold: bool = False):
        if self._auto is not None:
            self.release(self._auto)
            self._auto = None
        step = C.c_uint64()
        idx = self._lib.rb_prefetch_next(self._h, -1 if timeout_s is None else int(timeout_s * 1000), C.byref(step))
        if idx == -2:
            raise TimeoutError("no batch became ready in time (are all buffers held?)")
        if idx < 0:
            raise IndexError("token window out of range")
        self._held.append(idx)
        if not hold:
            self._auto = idx
        return self._bufs[idx], int(step.value)

    def release(self, batch) -> None:
        idx = batch if isinstance(batch, int) else next(i for i, b in enumerate(self._bufs) if b.data_ptr() == batch.data_ptr())
        if idx in self._held:
            self._held.remove(idx)
            self._lib.rb_prefetch_release(self._h, idx)

    def close(self) -> None:
        if self._h:
            self._lib.rb_prefetch_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001 - interpreter shutdown: the library or its handle may already be gone
            pass


class PinnedBatchPrefetcher:
    """Produces batches on a background thread into pinned host buffers, `depth` ahead, so the host-to-device copy
    of step i+1 overlaps the compute of step i."""

    def __init__(self, make_batch, depth: int = 2):
        self._make = make_batch
        self._q: "queue.Queue" = queue.Queue(maxsize=depth)
        self._stop = False
        self._step = 0
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        while not self._stop:
            b = self._make(self._step)
            self._step += 1
            if torch.cuda.is_available() and not b.is_pinned():
                b = b.pin_memory()
            while not self._stop:
                try:
                    self._q.put(b, timeout=0.1)
                    break
                except queue.Full:
                    continue

    def next(self) -> torch.Tensor:
        return self._q.get()

    def close(self):
        self._stop = True
        self._t.join(timeout=2)
