"""Tensor-parallel communication for inference: one-shot all-reduce and all-gather of small activations over NVLink
peer memory (decode steps are latency-bound: one kernel, one flag exchange, every rank sums the peers' contributions
itself in rank order, so all ranks hold bit-identical results and sample the same token).

The producing GEMM writes straight into this rank's symmetric staging buffer (`staging(rows, cols)` is its `out=`),
so there is no copy before the exchange.  The reference's tensor-parallel layers all-reduce host slices
(crates/distributed/src/tensor_parallel.rs:151-173).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _native as N
from .symm import SignalPad, SymmetricBuffer

P, I = N.c_void_p, N.c_int
N.optional_sig("rb_tp_allreduce", [P, P, P, I, I, I, N.C.c_uint, P, I, P, P, I, I, I, P])
N.optional_sig("rb_tp_allreduce_mc", [P, P, P, I, I, I, P, I, P, P, I, I, P])


class TPInferenceComm:
    """`transport` (`RUSTRAL_TP_ALLREDUCE` overrides the default "auto": "nvls" from four ranks up where the system has
    NVLink multicast, else "peer").  "peer": every rank sums the peers' staged tensors with plain peer loads in rank
    order.  "nvls": the staging buffers are bound to an NVLink multicast object and the sum is
    formed inside the NVSwitch (`multimem.ld_reduce`, `csrc/comm/nvls.cu`): one load per 16 bytes instead of one per rank;
    the all-gather keeps the peer loads."""

    def __init__(self, group, device, max_elems: int, limit_ms: int = 5000, transport: str | None = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.max_elems = max_elems
        self.limit_ms = limit_ms
        import os
        self.transport = transport or os.environ.get("RUSTRAL_TP_ALLREDUCE", "auto")
        if self.transport not in ("peer", "nvls", "auto"):
            raise ValueError(f"TPInferenceComm: unknown transport {self.transport!r}")
        self.pad = SignalPad(group, self.device)
        from .nvls import MulticastBuffer, MulticastUnavailable
        if self.transport == "auto":
            # measured on 8 x B200 (Llama-8B, 16 requests/s): p50 inter-token latency 5.31 ms with peer loads, 4.60 ms through
            # the switch; no difference at two ranks, where a peer-load all-reduce reads a single remote copy
            self.transport = "nvls" if self.world >= 4 else "peer"
            if self.transport == "nvls":
                try:
                    self.stage = [MulticastBuffer(max_elems * 2, group, self.device) for _ in range(2)]
                except MulticastUnavailable:
                    self.transport = "peer"
        elif self.transport == "nvls":
            self.stage = [MulticastBuffer(max_elems * 2, group, self.device) for _ in range(2)]
        if self.transport == "peer":
            self.stage = [SymmetricBuffer(max_elems * 2, group, self.device) for _ in range(2)]
        self.calls = 0                   # host count of collective calls: selects the staging buffer
        # The epoch the flags carry lives on the device and is advanced by a kernel before every collective, so a
        # decode step captured in a CUDA graph uses fresh epochs at every replay.
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._pad_out = torch.zeros((1, 8), dtype=torch.bfloat16, device=self.device)

    def staging(self, rows: int, cols: int) -> torch.Tensor:
        """The buffer the NEXT collective call reads this rank's contribution from."""
        if rows * cols > self.max_elems:
            raise ValueError(f"TPInferenceComm: {rows}x{cols} exceeds the staging capacity of {self.max_elems} elements")
        return self.stage[(self.calls + 1) & 1].view(torch.bfloat16, rows * cols).view(rows, cols)

    def _run(self, rows, cols, residual, out, gather):
        self.calls += 1
        st = self.stage[self.calls & 1]
        self.epoch_dev.add_(1)
        if self.transport == "nvls" and not gather:
            N.check(N.kernels().rb_tp_allreduce_mc(st.mc_ptr, self.pad.ptrs_dev.data_ptr(), self.pad.local_ptr, self.world, self.rank,
                                                   0, self.epoch_dev.data_ptr(), self.limit_ms, N.ptr(residual), out.data_ptr(),
                                                   rows, cols, N.stream_ptr()), "rb_tp_allreduce_mc")
            return out
        N.check(N.kernels().rb_tp_allreduce(st.ptrs_dev.data_ptr(), self.pad.ptrs_dev.data_ptr(), self.pad.local_ptr,
                                            self.world, self.rank, 0, 0, self.epoch_dev.data_ptr(), self.limit_ms,
                                            N.ptr(residual), out.data_ptr(), rows, cols, gather, N.stream_ptr()),
                "rb_tp_allreduce")
        return out

    def end_step(self) -> None:
        """Call after the last collective of a model step: pads the step to an even number of collectives, so that
        every step starts on the same staging buffer (a step replayed from a CUDA graph has its buffers baked in)."""
        if self.calls & 1:
            self.staging(1, 8).zero_()
            self._run(1, 8, None, self._pad_out, 0)

    def all_reduce(self, rows: int, cols: int, residual=None, out=None) -> torch.Tensor:
        """Sum of every rank's staged [rows, cols] (+ residual)."""
        if out is None:
            out = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        return self._run(rows, cols, residual, out, 0)

    def all_gather_cols(self, rows: int, cols: int, out=None) -> torch.Tensor:
        """[rows, world * cols]: every rank's staged [rows, cols] side by side in rank order."""
        if out is None:
            out = torch.empty((rows, self.world * cols), dtype=torch.bfloat16, device=self.device)
        return self._run(rows, cols, None, out, 1)

    def broadcast_scalar(self, value: float, src: int = 0) -> float:
        """Rank `src`'s value on every rank (keeps the serving loops of the ranks in lockstep)."""
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.broadcast(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
        return float(t)

    def close(self) -> None:
        for s in self.stage:
            s.close()
        self.pad.close()
