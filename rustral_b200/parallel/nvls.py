"""NVLink multicast (NVLS) buffers and their data-plane calls.

A `MulticastBuffer` is one allocation per rank, all bound to one multicast object of the NVSwitch: besides the peers'
unicast addresses (plain peer loads / stores, copy engines) it has a multicast address through which
`multimem.ld_reduce` returns the sum of an element over all ranks, computed inside the switch, and `multimem.st` writes
an element to all ranks at once (`csrc/comm/nvls.cu`).  A reduce-scatter then moves 1 / world of the bytes a rank would
pull with peer loads, and an all-reduce is one read and one write of a rank's own slice.

The allocation, the exchange of handles and the binding are torch.distributed's symmetric memory; the kernels are this
library's.  Ordering between ranks is the caller's (flag kernels with bounded waits, or host barriers): nothing here
waits.  The reference only stubs these collectives (crates/distributed/src/nccl.rs:240-262,283-346).

Not for tests in which a rank exits early: a process that dies while its memory is bound to a multicast object can
raise NVLink errors on the other GPUs; elastic / failure paths run on the plain peer-memory planes.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _native as N

_P, _LL, _I = N.c_void_p, N.c_ll, N.c_int
N.optional_sig("rb_mc_reduce_f32", [_P, _LL, _P, _LL, _I, _I, _P])
N.optional_sig("rb_mc_allreduce", [_P, _LL, _LL, _I, _I, _P])
N.optional_sig("rb_mc_broadcast", [_P, _P, _LL, _LL, _I, _P])


class MulticastUnavailable(RuntimeError):
    pass


class MulticastBuffer:
    def __init__(self, nbytes: int, group=None, device=None):
        try:
            import torch.distributed._symmetric_memory as symm_mem
        except ImportError as e:                                  # pragma: no cover
            raise MulticastUnavailable(f"torch.distributed symmetric memory is not available: {e}") from e
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.nbytes = (nbytes + 15) // 16 * 16
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.mc_ptr = int(self.handle.multicast_ptr or 0)
        if not self.mc_ptr:
            raise MulticastUnavailable("this system exposes no NVLink multicast address (no NVSwitch, or NVLS is disabled)")
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.local_ptr = self.peer_ptrs[self.rank]
        self.ptrs_dev = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)

    def view(self, dtype, numel: int | None = None, byte_offset: int = 0) -> torch.Tensor:
        t = self.local[byte_offset:].view(dtype)
        return t if numel is None else t[:numel]

    def peer_view(self, rank: int, dtype, numel: int) -> torch.Tensor:
        return self.handle.get_buffer(rank, (numel,), dtype)

    # ---- data plane -----------------------------------------------------------------------------------------------
    def reduce_into(self, dst: torch.Tensor, elem_offset: int, accumulate: bool = False, max_ctas: int = 0) -> torch.Tensor:
        """dst (fp32, contiguous) (+)= sum over ranks of this buffer's fp32 elements [elem_offset, elem_offset + dst.numel())."""
        assert dst.dtype == torch.float32 and dst.is_contiguous()
        N.check(N.kernels().rb_mc_reduce_f32(self.mc_ptr, elem_offset, dst.data_ptr(), dst.numel(), int(accumulate), max_ctas,
                                             N.stream_ptr()), "rb_mc_reduce_f32")
        return dst

    def all_reduce_slice_(self, dtype, byte_offset: int | None = None, nbytes: int | None = None, max_ctas: int = 0) -> None:
        """Sums this rank's slice (default: the rank-th 1 / world of the buffer) over all ranks, in place on every rank.
        When every rank has run it (and the caller has ordered the ranks) the whole buffer holds the all-reduce."""
        if byte_offset is None:
            per = self.nbytes // self.world // 16 * 16
            byte_offset = self.rank * per
            nbytes = per if self.rank < self.world - 1 else self.nbytes - byte_offset
        N.check(N.kernels().rb_mc_allreduce(self.mc_ptr, byte_offset, nbytes, int(dtype == torch.bfloat16), max_ctas, N.stream_ptr()),
                "rb_mc_allreduce")

    def broadcast_from(self, src: torch.Tensor, byte_offset: int = 0, max_ctas: int = 0) -> None:
        """Writes `src` (contiguous, a multiple of 16 bytes) at `byte_offset` of every rank's buffer."""
        nbytes = src.numel() * src.element_size()
        N.check(N.kernels().rb_mc_broadcast(src.data_ptr(), self.mc_ptr, byte_offset, nbytes, max_ctas, N.stream_ptr()),
                "rb_mc_broadcast")

    def check_canaries(self) -> bool:
        return True

    def close(self) -> None:
        """Collective: no kernel of any rank may still use the buffer."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.handle = None
        self.local = None


def multicast_available(group=None, device=None) -> bool:
    """True when a small multicast buffer can be created on this system (collective call)."""
    try:
        MulticastBuffer(4096, group, device).close()
        return True
    except Exception:      # noqa: BLE001 - any failure of the plumbing means "not available"
        return False
