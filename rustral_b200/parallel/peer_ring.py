"""Ring / context-parallel attention over NVLink peer memory.

Every rank publishes its K / V block in a symmetric buffer.  A rank then works through the blocks it needs, nearest
source first: block i + 2 is pulled from its owner's buffer on a side stream (a bounded-grid copy kernel issuing plain
peer loads, or a copy engine) while the tensor cores attend block i, partial results are folded into an fp32
accumulator with their log-sum-exp by one kernel, and causally invisible blocks are neither pulled nor computed.
Through NVSwitch every owner is one hop away, so nothing is relayed around a ring: the "ring" is only the order of
the pulls, which spreads the load over the owners.  In the backward pass K / V are published again (the buffers have
been reused by other layers since), the key / value gradient of every block is stored into the owner's receive slot
of this rank (peer stores on the side stream), and each owner folds its slots in rank order, so the result is
bit-reproducible.

All cross-rank ordering goes through bounded flag waits (`SignalPad`); an expired wait sets the device status word.
The host-relayed variant (NCCL send / recv) stays in `sequence_parallel.py`; the reference's ring never moves a
block and merges outputs as if they were logits (crates/distributed/src/sequence_parallel.rs:327-369,
crates/distributed/src/context_parallel.rs:232-344).
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from .. import _native as N
from . import sequence_parallel as sp
from .symm import SignalPad, SymmetricBuffer

N.optional_sig("rb_peer_copy", [N.c_void_p, N.c_void_p, N.c_ll, N.c_int, N.c_void_p])
N.optional_sig("rb_attn_merge", [N.c_void_p, N.c_void_p, N.c_void_p, N.c_void_p, N.c_int, N.c_int, N.c_int, N.c_int,
                                 N.c_int, N.c_void_p])
N.optional_sig("rb_ring_fold", [N.c_void_p, N.c_int, C.c_uint, N.c_ll, N.c_void_p, N.c_void_p])

CH_KV, CH_GRAD, CH_GRAD_DONE = 0, 1, 2          # signal channels: K/V published, gradients deposited, slots folded


class PeerRing:
    """Symmetric buffers, flags and streams for peer-memory ring attention among the ranks of `group`.

    max_kv_elems: the largest K (= V) block of one rank in elements (batch * local sequence * kv heads * head dim).
    copy_ctas: grid bound of the pull / push kernels; negative = copy engine.
    """

    def __init__(self, group, device, max_kv_elems: int, copy_ctas: int = 64, limit_ms: int = 2000):
        if max_kv_elems <= 0 or max_kv_elems % 8:
            raise ValueError("max_kv_elems must be a positive multiple of 8")
        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap = max_kv_elems
        self.copy_ctas, self.limit_ms = copy_ctas, limit_ms
        self.kv = [SymmetricBuffer(4 * max_kv_elems, group, device) for _ in range(2)]        # K then V, bf16
        self.slots = SymmetricBuffer(self.world * 4 * max_kv_elems, group, device)            # [world][dK, dV] bf16
        self.pad = SignalPad(group, device)
        self.land = [torch.empty(2 * max_kv_elems, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.stage = [torch.empty(2 * max_kv_elems, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.side = torch.cuda.Stream(device)
        self.kv_epoch = 0
        self.grad_epoch = 0

    # ---- building blocks ------------------------------------------------------------------------------------------
    def _copy(self, dst_ptr: int, src_ptr: int, nbytes: int) -> None:
        N.check(N.kernels().rb_peer_copy(dst_ptr, src_ptr, nbytes, self.copy_ctas, N.stream_ptr()), "rb_peer_copy")

    def _publish(self, k, v) -> int:
        """Copies this rank's K / V into the symmetric buffer of the new epoch and waits until every rank has done so.
        Returns the buffer parity.  The buffer of parity p was last read by peers two epochs ago; every one of them has
        raised the flag of the epoch in between after those reads, and this rank has waited for that flag."""
        n = k.numel()
        if n != v.numel() or n > self.cap or n % 8:
            raise ValueError(f"K / V block of {n} elements does not fit the ring's buffers ({self.cap})")
        self.kv_epoch += 1
        p = self.kv_epoch & 1
        buf = self.kv[p].view(torch.bfloat16)
        buf[:n].view(k.shape).copy_(k)
        buf[n:2 * n].view(v.shape).copy_(v)
        self.pad.signal_all(CH_KV, self.kv_epoch)
        self.pad.wait_all(CH_KV, self.kv_epoch, self.limit_ms)
        return p

    def _sources(self, causal: bool, striped: bool) -> list:
        """(source rank, block mode) of the remote blocks this rank needs, nearest first."""
        out = []
        for s in range(1, self.world):
            src = (self.rank - s) % self.world
            mode = sp._block_mode(self.rank, src, causal, striped)
            if mode != "skip":
                out.append((src, mode))
        return out

    def _contributors(self, causal: bool, striped: bool) -> int:
        """Bit mask of the ranks that deposit a key / value gradient for THIS rank's block."""
        mask = 0
        for q in range(self.world):
            if sp._block_mode(q, self.rank, causal, striped) != "skip":
                mask |= 1 << q
        return mask

    def _pull(self, i: int, src: int, parity: int, n: int, free_after) -> torch.cuda.Event:
        """Side stream: once the landing buffer is free, copy K and V of rank `src` into it."""
        with torch.cuda.stream(self.side):
            if free_after is not None:
                self.side.wait_event(free_after)
            self._copy(self.land[i & 1].data_ptr(), self.kv[parity].peer_ptrs[src], 4 * n)
            ev = torch.cuda.Event()
            ev.record(self.side)
        return ev

    def _blocks(self, k, v, causal, striped):
        """Generator over (source rank, mode, K block, V block, done) with the pulls running two blocks ahead on the
        side stream; the consumer records `done` (an event) on the main stream when it has finished with the block."""
        n = k.numel()
        parity = self._publish(k, v)
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        self.side.wait_event(ready)
        srcs = self._sources(causal, striped)
        fetched = {}
        done = [torch.cuda.Event() for _ in srcs]
        for i in range(min(2, len(srcs))):
            fetched[i] = self._pull(i, srcs[i][0], parity, n, None)
        yield self.rank, sp._block_mode(self.rank, self.rank, causal, striped), k, v, None
        for i, (src, mode) in enumerate(srcs):
            main.wait_event(fetched[i])
            land = self.land[i & 1]
            yield src, mode, land[:n].view(k.shape), land[n:2 * n].view(v.shape), done[i]
            if i + 2 < len(srcs):
                fetched[i + 2] = self._pull(i + 2, srcs[i + 2][0], parity, n, done[i])

    # ---- forward / backward ---------------------------------------------------------------------------------------
    def forward(self, q, k, v, causal: bool, striped: bool, scale: float):
        B, S, H, D = q.shape
        lib = N.kernels()
        o_acc = torch.empty((B, S, H, D), dtype=torch.float32, device=q.device)
        lse_acc = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        first = True
        main = torch.cuda.current_stream(self.device)
        for _, mode, kb, vb, done in self._blocks(k, v, causal, striped):
            r = sp._block_forward(q, kb, vb, mode, scale)
            if done is not None:
                done.record(main)
            if r is None:
                continue
            o_b, lse_b = r
            N.check(lib.rb_attn_merge(o_acc.data_ptr(), lse_acc.data_ptr(), o_b.contiguous().data_ptr(),
                                      lse_b.contiguous().data_ptr(), B, S, H, D, 1 if first else 0, N.stream_ptr()),
                    "rb_attn_merge")
            first = False
        if first:
            raise RuntimeError("ring attention: no visible block (the local block is always visible)")
        return o_acc.to(q.dtype), lse_acc

    def backward(self, do, q, k, v, o, lse, causal: bool, striped: bool, scale: float):
        n = k.numel()
        W, r = self.world, self.rank
        main = torch.cuda.current_stream(self.device)
        self.grad_epoch += 1
        g = self.grad_epoch
        # the owners have folded the slots of the previous backward before anything new is stored into them
        self.pad.wait_all(CH_GRAD_DONE, g - 1, self.limit_ms)
        slots_may_be_written = torch.cuda.Event()
        slots_may_be_written.record(main)
        self.side.wait_event(slots_may_be_written)
        dq = None
        my_slots = self.slots.view(torch.bfloat16)
        pushed, stage_free = [], [None, None]
        j = 0
        for src, mode, kb, vb, done in self._blocks(k, v, causal, striped):
            grads = sp._block_backward(do, q, kb, vb, o, lse, mode, scale)
            if done is not None:
                done.record(main)
            if grads is None:        # visible by rank order but empty (a strict-causal block of one token): deposit zeros
                grads = (None, torch.zeros_like(k), torch.zeros_like(v))
            if grads[0] is not None:
                dq = grads[0].float() if dq is None else dq.add_(grads[0])
            if src == r:
                own = my_slots[r * 2 * self.cap:r * 2 * self.cap + 2 * n]
                own[:n].view(k.shape).copy_(grads[1])
                own[n:].view(v.shape).copy_(grads[2])
                continue
            st = self.stage[j & 1]
            if stage_free[j & 1] is not None:
                main.wait_event(stage_free[j & 1])
            st[:n].view(k.shape).copy_(grads[1])
            st[n:2 * n].view(v.shape).copy_(grads[2])
            staged = torch.cuda.Event()
            staged.record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(staged)
                self._copy(self.slots.peer_ptrs[src] + (r * 2 * self.cap) * 2, st.data_ptr(), 4 * n)
                ev = torch.cuda.Event()
                ev.record(self.side)
            stage_free[j & 1] = ev
            pushed.append(ev)
            j += 1
        for ev in pushed:
            main.wait_event(ev)
        self.pad.signal_all(CH_GRAD, g)
        self.pad.wait_all(CH_GRAD, g, self.limit_ms)
        dkv = torch.empty(2 * n, dtype=torch.bfloat16, device=q.device)
        mask = self._contributors(causal, striped)
        if n == self.cap:
            N.check(N.kernels().rb_ring_fold(my_slots.data_ptr(), W, mask, 2 * n, dkv.data_ptr(), N.stream_ptr()), "rb_ring_fold")
        else:                        # a block smaller than the buffers: the slots are cap apart, fold a strided view
            sl = my_slots.view(W, 2 * self.cap)[:, :2 * n]
            acc = torch.zeros(2 * n, dtype=torch.float32, device=q.device)
            for rr in range(W):
                if (mask >> rr) & 1:
                    acc += sl[rr]
            dkv.copy_(acc)
        self.pad.signal_all(CH_GRAD_DONE, g)
        if dq is None:
            dq = torch.zeros_like(q, dtype=torch.float32)
        return dq.to(q.dtype), dkv[:n].view(k.shape).clone(), dkv[n:].view(v.shape).clone()

    def attention(self, q, k, v, causal: bool = True, striped: bool = False, scale: float | None = None):
        """Differentiable attention of this rank's queries [B, S_local, H, D] over the sequence sharded across the
        group (K, V: [B, S_local, Hkv, D]); bf16 CUDA tensors."""
        scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
        return _PeerRingFn.apply(q, k, v, self, causal, striped, scale)

    def check_canaries(self) -> bool:
        return all(b.check_canaries() for b in (*self.kv, self.slots, self.pad))

    def close(self) -> None:
        """Collective; no kernel of any rank may still be using the buffers."""
        torch.cuda.synchronize(self.device)
        for b in (*self.kv, self.slots, self.pad):
            b.close()


class _PeerRingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ring, causal, striped, scale):
        for t in (q, k, v):
            if not t.is_cuda or t.dtype != torch.bfloat16:
                raise TypeError("peer-memory ring attention takes bf16 CUDA tensors")
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = ring.forward(q, k, v, causal, striped, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (ring, causal, striped, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        ring, causal, striped, scale = ctx.meta
        dq, dk, dv = ring.backward(do.contiguous(), q, k, v, o, lse, causal, striped, scale)
        return dq, dk, dv, None, None, None, None
