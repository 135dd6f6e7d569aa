"""KV caches (crates/nn/src/kv_cache.rs:40-682): dense, sliding-window, paged and batched.

`KVCache.append` really stores the new keys and values (the reference validates and then rewrites the cache
unchanged, kv_cache.rs:197-210).  `PagedCache` owns tensor storage as well as the block tables; the tables live in
the C++ allocator (csrc/runtime/block_allocator.cpp) and a second `allocate` for a sequence extends its table.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import torch

from .. import _native as N
from ..core.errors import InvalidArgument


class CacheQuantization(enum.Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"
    INT8 = "int8"

    @property
    def bytes_per_element(self) -> int:
        return {"fp32": 4, "fp16": 2, "bf16": 2, "fp8": 1, "int8": 1}[self.value]

    def torch_dtype(self):
        return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn,
                "int8": torch.int8}[self.value]

    @property
    def scaled(self) -> bool:
        """8-bit formats are stored with one scale per tensor (absmax / 127 for int8, absmax / 448 for e4m3)."""
        return self in (CacheQuantization.FP8, CacheQuantization.INT8)


@dataclass
class CacheConfig:
    num_heads: int
    head_dim: int
    max_seq_len: int
    batch_size: int = 1
    quantization: CacheQuantization = CacheQuantization.BF16
    use_mqa: bool = False
    num_kv_heads: int = 0
    num_layers: int = 1

    def __post_init__(self):
        if self.num_kv_heads == 0:
            self.num_kv_heads = 1 if self.use_mqa else self.num_heads

    def with_mqa(self):
        self.use_mqa, self.num_kv_heads = True, 1
        return self

    def with_gqa(self, num_kv_heads: int):
        if self.num_heads % num_kv_heads:
            raise InvalidArgument("num_heads must be divisible by num_kv_heads")
        self.num_kv_heads = num_kv_heads
        return self

    def memory_bytes(self) -> int:
        per = self.batch_size * self.num_kv_heads * self.max_seq_len * self.head_dim
        return int(2 * per * self.num_layers * self.quantization.bytes_per_element)


@dataclass
class CacheMemoryStats:
    allocated_bytes: int
    used_bytes: int
    utilization: float


class KVCache:
    """Dense cache [batch, kv_heads, max_seq_len, head_dim] for K and V of one layer."""

    def __init__(self, config: CacheConfig, device="cpu"):
        self.config = config
        dt = config.quantization.torch_dtype()
        shape = (config.batch_size, config.num_kv_heads, config.max_seq_len, config.head_dim)
        self.k = torch.zeros(shape, dtype=dt, device=device)
        self.v = torch.zeros(shape, dtype=dt, device=device)
        self.k_scale = self.v_scale = 1.0
        self.len = 0

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """k_new / v_new: [batch, kv_heads, n, head_dim]."""
        n = k_new.shape[2]
        if self.len + n > self.config.max_seq_len:
            raise InvalidArgument(f"KV cache overflow: {self.len} + {n} > {self.config.max_seq_len}")
        self.k[:, :, self.len:self.len + n] = self._encode(k_new, "k")
        self.v[:, :, self.len:self.len + n] = self._encode(v_new, "v")
        self.len += n

    def _encode(self, t: torch.Tensor, which: str) -> torch.Tensor:
        """Values in the storage format.  8-bit formats use one scale per tensor, fixed by the first append after a
        reset (absmax over that append; later values beyond it saturate)."""
        q = self.config.quantization
        if not q.scaled:
            return t.to(self.k.dtype)
        top = 127.0 if q is CacheQuantization.INT8 else 448.0
        name = which + "_scale"
        if self._empty():
            amax = float(t.abs().max())
            setattr(self, name, amax / top if amax > 0 else 1.0)
        x = (t.float() / getattr(self, name)).clamp(-top, top)
        return torch.round(x).to(torch.int8) if q is CacheQuantization.INT8 else x.to(torch.float8_e4m3fn)

    def _decode(self, t: torch.Tensor, which: str) -> torch.Tensor:
        if not self.config.quantization.scaled:
            return t
        return t.float() * getattr(self, which + "_scale")

    def _empty(self) -> bool:
        return self.len == 0

    def get(self):
        return self.get_range(0, self.len)

    def get_range(self, start: int, end: int):
        return self._decode(self.k[:, :, start:end], "k"), self._decode(self.v[:, :, start:end], "v")

    def reset(self) -> None:
        self.len = 0

    def memory_stats(self) -> CacheMemoryStats:
        alloc = 2 * self.k.numel() * self.k.element_size()
        used = int(alloc * self.len / max(1, self.config.max_seq_len))
        return CacheMemoryStats(alloc, used, self.len / max(1, self.config.max_seq_len))


class SlidingWindowCache(KVCache):
    """Keeps the last `window` positions; older entries are overwritten ring-buffer style."""

    def __init__(self, config: CacheConfig, window: int, device="cpu"):
        cfg = CacheConfig(**{**config.__dict__, "max_seq_len": window})
        super().__init__(cfg, device)
        self.window = window
        self.total = 0

    def append(self, k_new, v_new) -> None:
        n = k_new.shape[2]
        kq, vq = self._encode(k_new, "k"), self._encode(v_new, "v")
        for i in range(n):
            pos = self.total % self.window
            self.k[:, :, pos] = kq[:, :, i]
            self.v[:, :, pos] = vq[:, :, i]
            self.total += 1
        self.len = min(self.total, self.window)

    def _empty(self) -> bool:
        return self.total == 0

    def reset(self) -> None:
        self.len = self.total = 0

    def get(self):
        """Entries in chronological order."""
        if self.total <= self.window:
            return self._decode(self.k[:, :, :self.len], "k"), self._decode(self.v[:, :, :self.len], "v")
        start = self.total % self.window
        idx = (torch.arange(self.window, device=self.k.device) + start) % self.window
        return self._decode(self.k[:, :, idx], "k"), self._decode(self.v[:, :, idx], "v")


class PagedCache:
    """Paged KV storage for all layers plus per-sequence block tables."""

    def __init__(self, num_blocks: int, block_size: int = 16, num_layers: int = 1, num_kv_heads: int = 1, head_dim: int = 64,
                 dtype=torch.bfloat16, device="cpu", allocate_storage: bool = True):
        self.block_size, self.num_blocks = block_size, num_blocks
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self._lib = N.runtime()
        self._h = self._lib.rb_ba_create(num_blocks, block_size)
        if not self._h:
            raise InvalidArgument("PagedCache: num_blocks and block_size must be positive")
        self.k = self.v = None
        if allocate_storage:
            shape = (num_layers, num_blocks, block_size, num_kv_heads, head_dim)
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rb_ba_destroy(h)

    @property
    def free_blocks(self) -> int:
        return self._lib.rb_ba_num_free(self._h)

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def can_allocate(self, seq_id: int, num_tokens: int) -> bool:
        return bool(self._lib.rb_ba_can_reserve(self._h, seq_id, num_tokens))

    def allocate(self, seq_id: int, num_tokens: int) -> bool:
        """Ensures `seq_id` can hold `num_tokens` tokens in total.  False (nothing changed) when out of blocks."""
        return self._lib.rb_ba_reserve(self._h, seq_id, num_tokens) >= 0

    def free(self, seq_id: int) -> int:
        return self._lib.rb_ba_free(self._h, seq_id)

    def block_table(self, seq_id: int) -> list:
        n = self._lib.rb_ba_table_len(self._h, seq_id)
        if n < 0:
            return []
        buf = (C.c_int32 * max(n, 1))()
        self._lib.rb_ba_table(self._h, seq_id, buf, n)
        return list(buf[:n])

    def slot(self, seq_id: int, token_index: int) -> int:
        return int(self._lib.rb_ba_slot(self._h, seq_id, token_index))

    def num_sequences(self) -> int:
        return self._lib.rb_ba_num_sequences(self._h)

    def memory_bytes(self) -> int:
        return 0 if self.k is None else 2 * self.k.numel() * self.k.element_size()


class BatchedCache:
    """One dense KVCache per layer, appended in lock step."""

    def __init__(self, num_layers: int, config: CacheConfig, device="cpu"):
        self.layers = [KVCache(config, device) for _ in range(num_layers)]

    def append(self, layer: int, k_new, v_new) -> None:
        self.layers[layer].append(k_new, v_new)

    def get(self, layer: int):
        return self.layers[layer].get()

    @property
    def len(self) -> int:
        return self.layers[0].len

    def reset(self) -> None:
        for l in self.layers:
            l.reset()
