"""ZeRO stage 3 for the hand-scheduled training engine: parameters, gradients and optimizer state are sharded over
the data-parallel ranks; full-size storage exists only for the buckets in flight.

Layout.  The parameters are cut into buckets: bucket 0 holds the embeddings, the final norm and an untied head,
bucket 1 + l holds transformer block l.  Inside a bucket the decayed parameters come first, every parameter starts on
a 128-element boundary, and the bucket is padded to a multiple of world x 128 elements.  Rank r owns elements
[r * n / W, (r + 1) * n / W) of every bucket: its fp32 master weights, Adam moments and gradient accumulator hold
exactly those slices, back to back ("the shard"), and so does its bf16 parameter shard, which lives in symmetric
memory so that peers can read it.

A micro-batch then runs like this (all of it inside the engine's CUDA graph):

* before a block computes, its bucket is gathered into one of two landing buffers on a side stream (every rank pulls
  the peers' slices over NVLink), one block ahead of the tensor cores, in the forward and again in the backward pass;
* weight gradients of a block are written (fp32) into one of two symmetric gradient buffers; when the block's backward
  is done a reduce kernel on a second side stream pulls this rank's slice out of every peer's buffer, sums in rank
  order and adds the sum to the gradient shard, while the main stream goes on with the next block;
* a gradient buffer is reused two blocks later, once every peer has flagged that it is done reading it.

After the last micro-batch the ranks exchange their partial squared norms and loss sums, clip, apply AdamW to their
slices and write the new bf16 slices into their shard buffers; the next step's gathers wait for the "parameters
ready" flag of every peer.  No full-size parameter, gradient or optimizer tensor exists on any rank.

The same bookkeeping runs over library collectives (`transport="collective"`: gloo on CPU ranks, NCCL on GPUs) as the
comparison arm and for tests without GPUs.

Reference behaviour being replaced: crates/distributed/src/fsdp.rs:199-210 (shard geometry), :238-249 (gather before
compute, free after), :323-338 (reduce-scatter after backward), :362-386 (train_step).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import _native as N
from .. import ops
from ..runtime.fused_gpt import ALIGN, ParamSpec, flat_to_state, param_specs, state_to_flat

CH_PARAMS, CH_NORM, CH_BASE = 4, 5, 8


class RbZero3Gather(C.Structure):
    _fields_ = [("lowp_ptrs_dev", N.c_void_p), ("local_pad", N.c_void_p), ("epoch_dev", N.c_void_p), ("channel", N.c_int),
                ("shard_off", N.c_ll), ("n_per_rank", N.c_ll), ("dst", N.c_void_p),
                ("world", N.c_int), ("rank", N.c_int), ("limit_ms", N.c_int), ("max_ctas", N.c_int), ("threads", N.c_int)]


class RbZero3Reduce(C.Structure):
    _fields_ = [("grad_ptrs_dev", N.c_void_p), ("pad_ptrs_dev", N.c_void_p), ("local_pad", N.c_void_p),
                ("epoch_dev", N.c_void_p), ("ready_channel", N.c_int), ("consumed_channel", N.c_int),
                ("n_per_rank", N.c_ll), ("shard_dst", N.c_void_p), ("accumulate", N.c_int), ("counter", N.c_void_p),
                ("world", N.c_int), ("rank", N.c_int), ("limit_ms", N.c_int), ("max_ctas", N.c_int), ("threads", N.c_int)]


class RbZero3Sum(C.Structure):
    _fields_ = [("src", N.c_void_p * 16), ("dst", N.c_void_p), ("n", N.c_ll), ("num_src", N.c_int), ("accumulate", N.c_int)]


class RbZero3Step(C.Structure):
    _fields_ = [("pad_ptrs_dev", N.c_void_p), ("local_pad", N.c_void_p), ("slots_ptrs_dev", N.c_void_p),
                ("local_slots", N.c_void_p), ("sumsq_local", N.c_void_p), ("loss_local", N.c_void_p),
                ("loss_out", N.c_void_p), ("loss_scale", N.c_float), ("norm_channel", N.c_int), ("params_channel", N.c_int),
                ("step", C.c_uint), ("step_epoch_dev", N.c_void_p),
                ("master", N.c_void_p), ("m", N.c_void_p), ("v", N.c_void_p), ("grad", N.c_void_p), ("lowp_shard", N.c_void_p),
                ("shard_len", N.c_ll), ("bucket_shard_start", N.c_void_p), ("bucket_decay_count", N.c_void_p),
                ("num_buckets", N.c_int),
                ("lr", N.c_float), ("beta1", N.c_float), ("beta2", N.c_float), ("eps", N.c_float), ("weight_decay", N.c_float),
                ("bc1", N.c_float), ("bc2", N.c_float), ("max_grad_norm", N.c_float),
                ("counter", N.c_void_p), ("world", N.c_int), ("rank", N.c_int), ("limit_ms", N.c_int)]


N.optional_sig("rb_epoch_advance", [N.c_void_p, N.c_void_p])
N.optional_sig("rb_zero3_gather", [C.POINTER(RbZero3Gather), N.c_void_p])
N.optional_sig("rb_zero3_reduce", [C.POINTER(RbZero3Reduce), N.c_void_p])
N.optional_sig("rb_zero3_wait", [N.c_void_p, N.c_int, N.c_int, N.c_void_p, N.c_int, N.c_int, N.c_void_p])
N.optional_sig("rb_zero3_signal", [N.c_void_p, N.c_int, N.c_int, N.c_int, N.c_void_p, N.c_void_p])
N.optional_sig("rb_zero3_sum", [C.POINTER(RbZero3Sum), N.c_void_p])
N.optional_sig("rb_zero3_publish", [C.POINTER(RbZero3Step), N.c_void_p])
N.optional_sig("rb_zero3_adam", [C.POINTER(RbZero3Step), N.c_void_p])


@dataclass
class Bucket:
    index: int
    specs: list = field(default_factory=list)      # (ParamSpec of the flat layout, offset inside the bucket)
    length: int = 0                                # padded to a multiple of world * ALIGN
    decay_end: int = 0                             # offsets below this take weight decay
    shard_start: int = 0                           # first element of this bucket's slice inside a rank's shard
    n_per_rank: int = 0


def bucket_of(name: str) -> int:
    if name.startswith("layers."):
        return 1 + int(name.split(".")[1])
    return 0


def build_buckets(cfg, world: int) -> tuple:
    """(buckets, placement) where placement maps a parameter name to (bucket index, offset inside the bucket)."""
    specs = param_specs(cfg)
    buckets = [Bucket(i) for i in range(cfg.n_layer + 1)]
    placement = {}
    for decay in (True, False):
        for s in specs:
            if s.decay != decay:
                continue
            b = buckets[bucket_of(s.name)]
            placement[s.name] = (b.index, b.length)
            b.specs.append((s, b.length))
            b.length += (s.numel + ALIGN - 1) // ALIGN * ALIGN
        for b in buckets:
            if decay:
                b.decay_end = b.length
    unit = world * ALIGN
    off = 0
    for b in buckets:
        b.length = (b.length + unit - 1) // unit * unit
        b.n_per_rank = b.length // world
        b.shard_start = off
        off += b.n_per_rank
    layer_layouts = {tuple((s.name.split(".", 2)[2], o, s.numel) for s, o in b.specs) for b in buckets[1:]}
    if len(layer_layouts) > 1:
        raise ValueError("ZeRO-3 buckets need identical parameter layouts in every transformer block")
    return buckets, placement


class _CollectiveTransport:
    """Gather / reduce-scatter through torch.distributed on the current stream (gloo on CPU, NCCL on GPUs)."""
    overlapped = False

    def __init__(self, sp: "ShardedParams"):
        self.sp = sp

    def alloc_shard_lowp(self, n, dtype):
        return torch.zeros(n, dtype=dtype, device=self.sp.device)

    def alloc_grad_buffer(self, n):
        return torch.zeros(n, dtype=torch.float32, device=self.sp.device)

    def begin_micro(self):
        pass

    def gather(self, b: Bucket, dst: torch.Tensor):
        sp = self.sp
        src = sp.lowp_shard[b.shard_start:b.shard_start + b.n_per_rank]
        if dst.is_cuda:
            dist.all_gather_into_tensor(dst[:b.length], src.contiguous(), group=sp.group)
        else:
            parts = [torch.empty_like(src) for _ in range(sp.world)]
            dist.all_gather(parts, src.contiguous(), group=sp.group)
            dst[:b.length].copy_(torch.cat(parts))

    def wait_gather(self, b):
        pass

    def before_grad_write(self, b: Bucket, slot):
        pass

    def reduce(self, b: Bucket, buf: torch.Tensor, slot, accumulate: bool):
        sp = self.sp
        out = sp.gshard[b.shard_start:b.shard_start + b.n_per_rank]
        if buf.is_cuda:
            tmp = torch.empty_like(out)
            dist.reduce_scatter_tensor(tmp, buf[:b.length], op=dist.ReduceOp.SUM, group=sp.group)
        else:
            full = buf[:b.length].clone()
            dist.all_reduce(full, group=sp.group)
            tmp = full[sp.rank * b.n_per_rank:(sp.rank + 1) * b.n_per_rank]
        if accumulate:
            out.add_(tmp)
        else:
            out.copy_(tmp)

    def end_micro(self):
        pass

    def step(self, sp, loss_local, loss_scale, hp) -> torch.Tensor:
        """Norm / loss exchange, clip and AdamW on the shard with tensor ops and two small collectives."""
        sq = ops.sumsq(sp.gshard).reshape(1).clone()
        pair = torch.cat([sq, loss_local.reshape(1).float()])
        dist.all_reduce(pair, group=sp.group)
        norm = pair[0].sqrt()
        for b in sp.buckets:
            lo = b.shard_start
            my0 = sp.rank * b.n_per_rank
            nd = min(max(b.decay_end - my0, 0), b.n_per_rank)
            for a, e, wd in ((lo, lo + nd, hp["weight_decay"]), (lo + nd, lo + b.n_per_rank, 0.0)):
                if e <= a:
                    continue
                ops.adam_step(sp.master_shard[a:e], sp.m[a:e], sp.v[a:e], sp.gshard[a:e], lr=hp["lr"], beta1=hp["beta1"],
                              beta2=hp["beta2"], eps=hp["eps"], weight_decay=wd, step=hp["step"], decoupled=True,
                              p_lowp=sp.lowp_shard[a:e] if sp.lowp_shard.dtype != torch.float32 else None,
                              max_grad_norm=hp["max_grad_norm"], grad_norm=norm)
        if sp.lowp_shard.dtype == torch.float32:
            sp.lowp_shard.copy_(sp.master_shard)
        return (pair[1] * loss_scale).reshape(())

    def close(self):
        pass


class _PeerTransport:
    """Peer memory over NVLink on two side streams.  Two data planes:

    "dma" (default): the bulk bytes are moved by the copy engines (stream-ordered device-to-device copies from the
    peers' mapped buffers), so no SM is taken from the GEMMs, whose persistent CTAs fill every SM's shared memory and
    leave no room for a second kernel to run beside them.  Kernels only carry the flags (one tiny CTA each: "my
    gradients of bucket b are written", bounded waits, "I am done reading your buffer") and the local part of the
    reduce-scatter (`rb_zero3_sum` on the main stream: own slice + the pulled slices, rank order, into the shard).
    "kernel": `rb_zero3_gather` / `rb_zero3_reduce` pull with peer loads from inside the kernels.
    "nvls" (reduce only, `RUSTRAL_Z3_REDUCE=nvls`): the gradient staging buffers are bound to an NVLink multicast object
    and a rank's slice is reduced inside the switch by one `multimem.ld_reduce` pass (`parallel/nvls.py`).
    """
    overlapped = True

    def __init__(self, sp: "ShardedParams", limit_ms: int = 5000, gather_ctas: int = 48, reduce_ctas: int = 64):
        import os
        from .symm import SignalPad, SymmetricBuffer, tensor_from_ptr
        self.sp = sp
        self._SymmetricBuffer, self._tensor_from_ptr = SymmetricBuffer, tensor_from_ptr
        # Tuning knobs (environment): CTAs and threads per CTA of the gather / reduce kernels, "dma" to move the
        # parameter slices with the copy engines instead of a kernel, "serial" to issue everything on the main stream.
        self.gather_ctas = int(os.environ.get("RUSTRAL_Z3_GATHER_CTAS", gather_ctas))
        self.reduce_ctas = int(os.environ.get("RUSTRAL_Z3_REDUCE_CTAS", reduce_ctas))
        self.threads = int(os.environ.get("RUSTRAL_Z3_THREADS", 256))
        self.gather_mode = os.environ.get("RUSTRAL_Z3_GATHER", "dma")
        self.reduce_mode = os.environ.get("RUSTRAL_Z3_REDUCE", "dma")
        self.serial = os.environ.get("RUSTRAL_Z3_SERIAL", "0") == "1"
        if self.serial:
            self.reduce_mode = "kernel"
        self._stage, self._peer_grad, self._pending_sums = {}, {}, []
        self.limit_ms = limit_ms
        dev = sp.device
        self.pad = SignalPad(sp.group, dev)
        self.slots = SymmetricBuffer(max(256, 8 * sp.world), sp.group, dev)
        self._symm = [self.pad, self.slots]
        if self.serial:
            self.gs = self.rs = None
        else:
            self.gs, self.rs = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self._params_waited = False
        self.micro_epoch = torch.zeros(1, dtype=torch.int32, device=dev)      # advanced once per micro-batch
        self.step_epoch = torch.zeros(1, dtype=torch.int32, device=dev)       # optimizer steps completed by this rank
        self.counters = torch.zeros(8, dtype=torch.int32, device=dev)
        self.sumsq = torch.zeros((), dtype=torch.float32, device=dev)
        self.loss_out = torch.zeros((), dtype=torch.float32, device=dev)
        self._gather_ev, self._grad_bufs = {}, {}
        self._pending_reduce = False
        self._pending_gather = False
        nb = len(sp.buckets)
        if (CH_BASE + 2 * nb) * sp.world > 16384:
            raise ValueError("too many buckets for the signal pad")
        self._tables = None

    # -- allocation ------------------------------------------------------------------------------------------
    def alloc_shard_lowp(self, n, dtype):
        buf = self._SymmetricBuffer(n * 2, self.sp.group, self.sp.device)
        self._symm.append(buf)
        self.lowp_buf = buf
        self._peer_lowp = [self._tensor_from_ptr(p, n * 2, self.sp.device).view(torch.bfloat16) for p in buf.peer_ptrs]
        return buf.view(torch.bfloat16, n)

    def alloc_grad_buffer(self, n):
        if self.reduce_mode == "nvls":
            # bound to an NVLink multicast object: the reduce-scatter is one multimem.ld_reduce pass over the own slice
            from .nvls import MulticastBuffer
            buf = MulticastBuffer(n * 4, self.sp.group, self.sp.device)
            self._symm.append(buf)
            t = buf.view(torch.float32, n)
            self._grad_bufs[t.data_ptr()] = buf
            return t
        buf = self._SymmetricBuffer(n * 4, self.sp.group, self.sp.device)
        self._symm.append(buf)
        t = buf.view(torch.float32, n)
        self._grad_bufs[t.data_ptr()] = buf
        sp = self.sp
        self._peer_grad[t.data_ptr()] = [self._tensor_from_ptr(p, n * 4, sp.device).view(torch.float32) for p in buf.peer_ptrs]
        if self.reduce_mode == "dma":
            # landing area for the peers' copies of this rank's slice: (world - 1) slices of the largest bucket it serves
            self._stage[t.data_ptr()] = torch.empty((sp.world - 1) * (n // sp.world), dtype=torch.float32, device=sp.device)
        return t

    # -- one micro-batch -------------------------------------------------------------------------------------
    def begin_micro(self):
        N.check(N.kernels().rb_epoch_advance(self.micro_epoch.data_ptr(), N.stream_ptr()), "rb_epoch_advance")
        self._params_waited = False

    def _gather_on(self, b: Bucket, dst: torch.Tensor):
        sp = self.sp
        if self.gather_mode == "dma":
            # copy engines move the slices; one bounded wait per micro-batch makes sure every peer has published the
            # parameters of the last step (the flag is per step, not per bucket)
            if not self._params_waited:
                N.check(N.kernels().rb_zero3_wait(self.pad.local_ptr, sp.world, CH_PARAMS, self.step_epoch.data_ptr(), 0,
                                                  self.limit_ms, N.stream_ptr()), "rb_zero3_wait")
                self._params_waited = True
            n, off = b.n_per_rank, b.shard_start
            for j in range(sp.world):
                r = (sp.rank + 1 + j) % sp.world
                dst[r * n:(r + 1) * n].copy_(self._peer_lowp[r][off:off + n], non_blocking=True)
            return
        a = RbZero3Gather()
        a.lowp_ptrs_dev, a.local_pad = self.lowp_buf.ptrs_dev.data_ptr(), self.pad.local_ptr
        a.epoch_dev, a.channel = self.step_epoch.data_ptr(), CH_PARAMS
        a.shard_off, a.n_per_rank, a.dst = b.shard_start, b.n_per_rank, dst.data_ptr()
        a.world, a.rank, a.limit_ms, a.max_ctas = sp.world, sp.rank, self.limit_ms, self.gather_ctas
        a.threads = self.threads
        N.check(N.kernels().rb_zero3_gather(a, N.stream_ptr()), "rb_zero3_gather")

    def gather(self, b: Bucket, dst: torch.Tensor):
        if self.serial:
            self._gather_on(b, dst)
            return
        main = torch.cuda.current_stream(self.sp.device)
        self.gs.wait_stream(main)          # the landing buffer's previous occupant has been consumed by kernels issued so far
        with torch.cuda.stream(self.gs):
            self._gather_on(b, dst)
            ev = torch.cuda.Event()
            ev.record(self.gs)
        self._gather_ev[b.index] = ev
        self._pending_gather = True

    def wait_gather(self, b: Bucket):
        ev = self._gather_ev.pop(b.index, None)
        if ev is not None:
            torch.cuda.current_stream(self.sp.device).wait_event(ev)

    def before_grad_write(self, b: Bucket, prev):
        """`prev`: (bucket index, epoch delta) of the reduce that last read the buffer this bucket is about to
        overwrite, on every peer; None when the buffer has never been reduced."""
        if prev is None:
            return
        N.check(N.kernels().rb_zero3_wait(self.pad.local_ptr, self.sp.world, CH_BASE + len(self.sp.buckets) + prev[0],
                                          self.micro_epoch.data_ptr(), prev[1], self.limit_ms, N.stream_ptr()), "rb_zero3_wait")

    def _reduce_dma(self, b: Bucket, buf: torch.Tensor, accumulate: bool):
        sp, lib = self.sp, N.kernels()
        W, rank, npr = sp.world, sp.rank, b.n_per_rank
        main = torch.cuda.current_stream(sp.device)
        ready, consumed = CH_BASE + b.index, CH_BASE + len(sp.buckets) + b.index
        N.check(lib.rb_zero3_signal(self.pad.ptrs_dev.data_ptr(), W, rank, ready, self.micro_epoch.data_ptr(), N.stream_ptr()),
                "rb_zero3_signal")
        # the fork also orders these copies behind the sum that last read this staging area (issued on the main stream)
        self.rs.wait_stream(main)
        stage, peers = self._stage[buf.data_ptr()], self._peer_grad[buf.data_ptr()]
        src = [None] * W
        with torch.cuda.stream(self.rs):
            N.check(lib.rb_zero3_wait(self.pad.local_ptr, W, ready, self.micro_epoch.data_ptr(), 0, self.limit_ms,
                                      N.stream_ptr()), "rb_zero3_wait")
            for k in range(W - 1):
                r = (rank + 1 + k) % W
                dst = stage[k * npr:(k + 1) * npr]
                dst.copy_(peers[r][rank * npr:(rank + 1) * npr], non_blocking=True)
                src[r] = dst
            N.check(lib.rb_zero3_signal(self.pad.ptrs_dev.data_ptr(), W, rank, consumed, self.micro_epoch.data_ptr(),
                                        N.stream_ptr()), "rb_zero3_signal")
            ev = torch.cuda.Event()
            ev.record(self.rs)
        src[rank] = buf[rank * npr:(rank + 1) * npr]
        self._pending_sums.append((b, src, accumulate, ev))
        self._pending_reduce = True
        self._flush_sums(keep=1)

    def _flush_sums(self, keep: int):
        """Adds the pulled slices of all but the `keep` most recent buckets into the gradient shard (main stream)."""
        sp = self.sp
        main = torch.cuda.current_stream(sp.device)
        while len(self._pending_sums) > keep:
            b, src, accumulate, ev = self._pending_sums.pop(0)
            main.wait_event(ev)
            a = RbZero3Sum()
            for i, t in enumerate(src):                                  # rank order: the sum does not depend on timing
                a.src[i] = t.data_ptr()
            a.dst = sp.gshard[b.shard_start:b.shard_start + b.n_per_rank].data_ptr()
            a.n, a.num_src, a.accumulate = b.n_per_rank, sp.world, int(accumulate)
            N.check(N.kernels().rb_zero3_sum(a, N.stream_ptr()), "rb_zero3_sum")

    def _reduce_nvls(self, b: Bucket, buf: torch.Tensor, accumulate: bool):
        """Reduce-scatter through the switch: flag "my gradients are written", (side stream) wait for everybody's flag,
        one `multimem.ld_reduce` pass over this rank's slice straight into the gradient shard, flag "done reading"."""
        sp, lib = self.sp, N.kernels()
        W, rank, npr = sp.world, sp.rank, b.n_per_rank
        ready, consumed = CH_BASE + b.index, CH_BASE + len(sp.buckets) + b.index
        N.check(lib.rb_zero3_signal(self.pad.ptrs_dev.data_ptr(), W, rank, ready, self.micro_epoch.data_ptr(), N.stream_ptr()),
                "rb_zero3_signal")
        main = torch.cuda.current_stream(sp.device)
        self.rs.wait_stream(main)
        mc = self._grad_bufs[buf.data_ptr()]
        with torch.cuda.stream(self.rs):
            N.check(lib.rb_zero3_wait(self.pad.local_ptr, W, ready, self.micro_epoch.data_ptr(), 0, self.limit_ms, N.stream_ptr()),
                    "rb_zero3_wait")
            mc.reduce_into(sp.gshard[b.shard_start:b.shard_start + npr], rank * npr, accumulate, self.reduce_ctas)
            N.check(lib.rb_zero3_signal(self.pad.ptrs_dev.data_ptr(), W, rank, consumed, self.micro_epoch.data_ptr(), N.stream_ptr()),
                    "rb_zero3_signal")
        self._pending_reduce = True

    def reduce(self, b: Bucket, buf: torch.Tensor, slot, accumulate: bool):
        sp = self.sp
        if self.reduce_mode == "dma":
            self._reduce_dma(b, buf, accumulate)
            return
        if self.reduce_mode == "nvls":
            self._reduce_nvls(b, buf, accumulate)
            return
        main = torch.cuda.current_stream(sp.device)
        if not self.serial:
            self.rs.wait_stream(main)
        symm = self._grad_bufs[buf.data_ptr()]
        a = RbZero3Reduce()
        a.grad_ptrs_dev, a.pad_ptrs_dev, a.local_pad = symm.ptrs_dev.data_ptr(), self.pad.ptrs_dev.data_ptr(), self.pad.local_ptr
        a.epoch_dev = self.micro_epoch.data_ptr()
        a.ready_channel, a.consumed_channel = CH_BASE + b.index, CH_BASE + len(sp.buckets) + b.index
        a.n_per_rank = b.n_per_rank
        a.shard_dst = sp.gshard[b.shard_start:b.shard_start + b.n_per_rank].data_ptr()
        a.accumulate, a.counter = int(accumulate), self.counters[0:1].data_ptr()
        a.world, a.rank, a.limit_ms, a.max_ctas = sp.world, sp.rank, self.limit_ms, self.reduce_ctas
        a.threads = self.threads
        if self.serial:
            N.check(N.kernels().rb_zero3_reduce(a, N.stream_ptr()), "rb_zero3_reduce")
            return
        with torch.cuda.stream(self.rs):
            N.check(N.kernels().rb_zero3_reduce(a, N.stream_ptr()), "rb_zero3_reduce")
        self._pending_reduce = True

    def end_micro(self):
        if self.serial:
            return
        main = torch.cuda.current_stream(self.sp.device)
        self._flush_sums(keep=0)
        # only streams that took work in this micro-batch are joined: inside a graph capture, waiting for a stream
        # that was never forked from the capturing stream would make the capture depend on work outside it
        if self._pending_gather:
            main.wait_stream(self.gs)
            self._pending_gather = False
        if self._pending_reduce:
            main.wait_stream(self.rs)
            self._pending_reduce = False

    # -- optimizer step ------------------------------------------------------------------------------------------
    def step(self, sp, loss_local, loss_scale, hp) -> torch.Tensor:
        lib = N.kernels()
        if self._tables is None:
            starts = torch.tensor([b.shard_start for b in sp.buckets], dtype=torch.int64, device=sp.device)
            decay = torch.tensor([min(max(b.decay_end - sp.rank * b.n_per_rank, 0), b.n_per_rank) for b in sp.buckets],
                                 dtype=torch.int64, device=sp.device)
            self._tables = (starts, decay)
        ops.sumsq(sp.gshard, out=self.sumsq)
        a = RbZero3Step()
        a.pad_ptrs_dev, a.local_pad = self.pad.ptrs_dev.data_ptr(), self.pad.local_ptr
        a.slots_ptrs_dev, a.local_slots = self.slots.ptrs_dev.data_ptr(), self.slots.local_ptr
        a.sumsq_local, a.loss_local, a.loss_out = self.sumsq.data_ptr(), loss_local.data_ptr(), self.loss_out.data_ptr()
        a.loss_scale, a.norm_channel, a.params_channel = loss_scale, CH_NORM, CH_PARAMS
        a.step, a.step_epoch_dev = hp["step"], self.step_epoch.data_ptr()
        a.master, a.m, a.v, a.grad = (t.data_ptr() for t in (sp.master_shard, sp.m, sp.v, sp.gshard))
        a.lowp_shard, a.shard_len = sp.lowp_shard.data_ptr(), sp.shard_len
        a.bucket_shard_start, a.bucket_decay_count = self._tables[0].data_ptr(), self._tables[1].data_ptr()
        a.num_buckets = len(sp.buckets)
        a.lr, a.beta1, a.beta2, a.eps, a.weight_decay = hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["weight_decay"]
        a.bc1, a.bc2 = 1.0 - hp["beta1"] ** hp["step"], 1.0 - hp["beta2"] ** hp["step"]
        a.max_grad_norm = hp["max_grad_norm"]
        a.counter = self.counters[1:2].data_ptr()
        a.world, a.rank, a.limit_ms = sp.world, sp.rank, self.limit_ms
        N.check(lib.rb_zero3_publish(a, N.stream_ptr()), "rb_zero3_publish")
        N.check(lib.rb_zero3_adam(a, N.stream_ptr()), "rb_zero3_adam")
        self._params_waited = False
        return self.loss_out

    def close(self):
        torch.cuda.synchronize(self.sp.device)
        for b in self._symm:
            b.close()
        self._symm = []


class ShardedParams:
    """Parameter store of the training engine under ZeRO-3.  Same access interface as `FlatParams` (`w(name)`,
    `g(name)`, `specs`, `state_dict`, `load_state_dict`) plus the hooks the engine calls around each block."""
    per_micro_reduce = True

    def __init__(self, cfg, device, seed: int = 0, group=None, transport: str = "peer"):
        self.cfg, self.device, self.group = cfg, torch.device(device), group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.specs = param_specs(cfg)
        self.by_name = {s.name: s for s in self.specs}
        self.flat_total = self.specs[-1].offset + (self.specs[-1].numel + ALIGN - 1) // ALIGN * ALIGN
        self.buckets, self.placement = build_buckets(cfg, self.world)
        self.total = sum(b.length for b in self.buckets)
        self.shard_len = self.total // self.world
        cuda = self.device.type == "cuda"
        lowp_dtype = torch.bfloat16 if cuda else torch.float32
        if transport == "peer" and not cuda:
            raise ValueError("the peer-memory transport needs CUDA devices")
        self.transport = _PeerTransport(self) if transport == "peer" else _CollectiveTransport(self)
        f32 = lambda n: torch.zeros(n, dtype=torch.float32, device=self.device)
        self.master_shard, self.m, self.v, self.gshard = f32(self.shard_len), f32(self.shard_len), f32(self.shard_len), f32(self.shard_len)
        self.lowp_shard = self.transport.alloc_shard_lowp(self.shard_len, lowp_dtype)
        layer_len = max((b.length for b in self.buckets[1:]), default=0)
        # landing buffers for gathered parameters (local) and for gradients of the block in flight (peer-readable)
        self.pbuf = [torch.zeros(layer_len, dtype=lowp_dtype, device=self.device) for _ in range(2)] if layer_len else []
        self.pbuf0 = torch.zeros(self.buckets[0].length, dtype=lowp_dtype, device=self.device)
        self.gbuf = [self.transport.alloc_grad_buffer(layer_len) for _ in range(2)] if layer_len else []
        self.gbuf0 = self.transport.alloc_grad_buffer(self.buckets[0].length)
        self._resident = {}              # landing-buffer key -> bucket index currently in it
        self._last_reduced = {}          # gradient-buffer key -> (bucket index, micro-batch number) of its last reduce
        self._micro = 0
        self._init(seed)
        if cuda:
            torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # ---- geometry --------------------------------------------------------------------------------------------
    def _slot(self, bi: int):
        return "e" if bi == 0 else bi % 2

    def _pbuf(self, bi: int) -> torch.Tensor:
        return self.pbuf0 if bi == 0 else self.pbuf[bi % 2]

    def _gbuf(self, bi: int) -> torch.Tensor:
        return self.gbuf0 if bi == 0 else self.gbuf[bi % 2]

    def _view(self, buf: torch.Tensor, name: str) -> torch.Tensor:
        s = self.by_name[name]
        _, off = self.placement[name]
        return buf[off:off + s.numel].view(s.shape)

    def w(self, name: str) -> torch.Tensor:
        return self._view(self._pbuf(self.placement[name][0]), name)

    def g(self, name: str) -> torch.Tensor:
        return self._view(self._gbuf(self.placement[name][0]), name)

    # ---- initialisation and checkpoints: through a host image in the flat (unsharded) layout --------------------
    def _init(self, seed: int) -> None:
        from ..runtime.fused_gpt import init_flat_host
        self._load_flat_host(init_flat_host(self.cfg, self.specs, self.flat_total, seed))

    def _load_flat_host(self, host: torch.Tensor) -> None:
        shard = torch.zeros(self.shard_len, dtype=torch.float32)
        for b in self.buckets:
            full = torch.zeros(b.length, dtype=torch.float32)
            for s, off in b.specs:
                full[off:off + s.numel] = host[s.offset:s.offset + s.numel]
            shard[b.shard_start:b.shard_start + b.n_per_rank] = full[self.rank * b.n_per_rank:(self.rank + 1) * b.n_per_rank]
        self.master_shard.copy_(shard)
        self.sync_lowp()
        self.invalidate()

    def sync_lowp(self) -> None:
        if self.lowp_shard.dtype == torch.float32:
            self.lowp_shard.copy_(self.master_shard)
        else:
            ops.cast_f32_to_bf16(self.master_shard, self.lowp_shard)

    def _gather_flat_host(self, shard: torch.Tensor) -> torch.Tensor:
        """Collects every rank's slices of a sharded fp32 tensor into a host image in the flat layout (collective)."""
        host = torch.zeros(self.flat_total, dtype=torch.float32)
        for b in self.buckets:
            mine = shard[b.shard_start:b.shard_start + b.n_per_rank].contiguous()
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            full = torch.cat(parts).cpu()
            for s, off in b.specs:
                host[s.offset:s.offset + s.numel] = full[off:off + s.numel]
        return host

    def state_dict(self) -> dict:
        return flat_to_state(self.cfg, self.specs, self._gather_flat_host(self.master_shard))

    def load_state_dict(self, state: dict) -> None:
        host = self._gather_flat_host(self.master_shard)
        state_to_flat(self.cfg, self.specs, state, host)      # strict; raises before anything is written
        self._load_flat_host(host)

    # ---- hooks called by the engine ---------------------------------------------------------------------------
    def state_key(self):
        return tuple(sorted((str(k), v) for k, v in self._resident.items()))

    def get_state(self):
        return dict(self._resident), dict(self._last_reduced), self._micro

    def set_state(self, st) -> None:
        self._resident, self._last_reduced, self._micro = dict(st[0]), dict(st[1]), st[2]

    def invalidate(self) -> None:
        """The parameter shards changed (optimizer step, checkpoint load): nothing gathered earlier may be reused."""
        self._resident = {}

    def begin_micro(self, first_micro: bool) -> None:
        self._micro += 1
        self._first = bool(first_micro)
        self.transport.begin_micro()

    def _gather(self, bi: int) -> None:
        key = self._slot(bi)
        if self._resident.get(key) == bi:
            return
        self.transport.gather(self.buckets[bi], self._pbuf(bi))
        self._resident[key] = bi

    def acquire(self, bi: int, prefetch: int | None = None) -> None:
        """Makes bucket `bi` usable by the kernels issued next; starts the gather of `prefetch` behind it."""
        self._gather(bi)
        self.transport.wait_gather(self.buckets[bi])
        if prefetch is not None and 0 <= prefetch < len(self.buckets):
            self._gather(prefetch)

    def begin_grads(self, bi: int) -> None:
        """Call before the first kernel that writes a gradient of bucket `bi` in this micro-batch."""
        last = self._last_reduced.get(self._slot(bi))
        self.transport.before_grad_write(self.buckets[bi], None if last is None else (last[0], last[1] - self._micro))

    def grads_done(self, bi: int) -> None:
        """Every gradient of bucket `bi` has been written for this micro-batch: reduce-scatter it into the shard."""
        self.transport.reduce(self.buckets[bi], self._gbuf(bi), self._slot(bi), accumulate=not self._first)
        self._last_reduced[self._slot(bi)] = (bi, self._micro)

    def end_micro(self) -> None:
        self.transport.end_micro()

    # ---- memory accounting --------------------------------------------------------------------------------------
    def state_bytes(self) -> dict:
        lp = self.lowp_shard.element_size()
        return {"param_shard": self.shard_len * lp, "optimizer_shard": 3 * self.shard_len * 4, "grad_shard": self.shard_len * 4,
                "param_landing": sum(t.numel() for t in self.pbuf + [self.pbuf0]) * lp,
                "grad_landing": sum(t.numel() for t in self.gbuf + [self.gbuf0]) * 4,
                "grad_staging": sum(t.numel() for t in getattr(self.transport, "_stage", {}).values()) * 4}

    def close(self) -> None:
        self.transport.close()


class Zero3Comm:
    """Step tail of the trainer under ZeRO-3 (same interface as the stage-2 communicators)."""

    def __init__(self, trainer):
        self.t = trainer
        self.sp: ShardedParams = trainer.engine.params
        self._loss_in = torch.zeros((), dtype=torch.float32, device=trainer.device)

    def reduce_and_step(self, loss_sum: torch.Tensor, lr):
        """`loss_sum`: this rank's summed token loss (device scalar).  Returns the global mean loss (device scalar)."""
        eng, sp = self.t.engine, self.sp
        eng.step_count += 1
        hp = dict(lr=eng.lr if lr is None else lr, beta1=eng.betas[0], beta2=eng.betas[1], eps=eng.eps,
                  weight_decay=eng.weight_decay, max_grad_norm=eng.max_grad_norm, step=eng.step_count)
        out = sp.transport.step(sp, loss_sum, 1.0 / self.t.tokens_per_step, hp)
        sp.invalidate()
        return out

    def gather_master(self) -> None:
        pass                                   # state_dict() of the sharded store gathers by itself

    def reload_master(self) -> None:
        pass

    def optimizer_shard(self) -> tuple:
        return self.sp.m, self.sp.v

    def close(self) -> None:
        self.sp.close()
