"""Symmetric memory between the ranks of one node.

Every rank allocates the same sequence of device buffers; each buffer is exported through CUDA IPC and mapped
into every peer, so a kernel on rank r can load from and store to rank q's copy directly over NVLink.  A signal
pad (one per rank, peer-writable) carries the flags the kernels synchronise on; all waits on it are bounded and
report through the device status word.

The reference's process group moves host slices through a mutex map or MPI (crates/distributed/src/lib.rs:99-297)
and its NCCL FFI hands host pointers to NCCL (crates/distributed/src/nccl.rs:225-265); this layer is the
device-side substrate those interfaces lack.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native as N

N.optional_sig("rb_symm_alloc", [N.c_ll], N.c_void_p)
N.optional_sig("rb_symm_free", [N.c_void_p])
N.optional_sig("rb_ipc_export", [N.c_void_p, C.c_char_p])
N.optional_sig("rb_ipc_import", [C.c_char_p], N.c_void_p)
N.optional_sig("rb_ipc_close", [N.c_void_p])
N.optional_sig("rb_signal_all", [N.c_void_p, N.c_int, N.c_int, N.c_int, C.c_uint, N.c_void_p])
N.optional_sig("rb_wait_all", [N.c_void_p, N.c_int, N.c_int, C.c_uint, N.c_int, N.c_void_p])

SIGNAL_PAD_BYTES = 65536               # 16384 flag words: 2048 channels at 8 ranks
GUARD_BYTES = 256                      # canary region before and after every symmetric buffer
_CANARY = 0x5AA5C33C


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class SymmetricBuffer:
    """One symmetric allocation: `local` is this rank's tensor (uint8), `peer_ptrs[r]` the address of rank r's copy
    as mapped into this process, `ptrs_dev` the same table as an int64 device tensor for kernels."""

    def __init__(self, nbytes: int, group, device):
        lib = N.kernels()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = nbytes
        self.device = torch.device(device)
        # the usable range sits between two guard regions filled with a canary pattern: a kernel of any rank that
        # writes past either end of a buffer is caught by `check_canaries()` on the host instead of silently
        # corrupting a neighbouring allocation
        padded = (nbytes + 15) // 16 * 16
        base = lib.rb_symm_alloc(padded + 2 * GUARD_BYTES)
        if not base:
            raise N.NativeError(f"symmetric allocation of {nbytes} bytes failed")
        self._base_ptr = int(base)
        self.local_ptr = self._base_ptr + GUARD_BYTES
        whole = tensor_from_ptr(self._base_ptr, padded + 2 * GUARD_BYTES, self.device)
        self._guards = (whole[:GUARD_BYTES].view(torch.int32), whole[GUARD_BYTES + padded:].view(torch.int32))
        for g in self._guards:
            g.fill_(_CANARY)
        handle = C.create_string_buffer(64)
        N.check(lib.rb_ipc_export(self._base_ptr, handle), "rb_ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.peer_ptrs = []
        self._imported = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            p = lib.rb_ipc_import(C.create_string_buffer(h, 64))
            if not p:
                raise N.NativeError(f"rank {self.rank}: cannot map the symmetric buffer of rank {r} (no peer access?)")
            self.peer_ptrs.append(int(p) + GUARD_BYTES)
            self._imported.append(int(p))
        self.local = tensor_from_ptr(self.local_ptr, nbytes, self.device)
        self.ptrs_dev = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)
        dist.barrier(group=group)

    def view(self, dtype, numel: int | None = None, byte_offset: int = 0) -> torch.Tensor:
        t = self.local[byte_offset:]
        t = t.view(dtype)
        return t if numel is None else t[:numel]

    def check_canaries(self) -> bool:
        """True when the guard words before and after this rank's buffer are intact (synchronises the device)."""
        return all(bool((g == _CANARY).all()) for g in self._guards)

    def close(self) -> None:
        """Unmaps the peers and frees the local allocation.  Collective: call on every rank, with no kernel in flight."""
        lib = N.kernels()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._imported:
            lib.rb_ipc_close(p)
        self._imported = []
        dist.barrier(group=self.group)
        if self.local_ptr:
            self.local = None
            self._guards = ()
            lib.rb_symm_free(self._base_ptr)
            self.local_ptr = self._base_ptr = 0


class SignalPad(SymmetricBuffer):
    """Peer-writable u32 flags: slot (channel, src_rank) of every rank's pad."""

    def __init__(self, group, device):
        super().__init__(SIGNAL_PAD_BYTES, group, device)

    def signal_all(self, channel: int, value: int) -> None:
        N.check(N.kernels().rb_signal_all(self.ptrs_dev.data_ptr(), self.world, self.rank, channel, value & 0xFFFFFFFF,
                                          N.stream_ptr()), "rb_signal_all")

    def wait_all(self, channel: int, value: int, limit_ms: int = 2000) -> None:
        N.check(N.kernels().rb_wait_all(self.local_ptr, self.world, channel, value & 0xFFFFFFFF, limit_ms,
                                        N.stream_ptr()), "rb_wait_all")
