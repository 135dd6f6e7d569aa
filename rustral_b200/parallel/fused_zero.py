"""ZeRO gradient reduction + sharded AdamW + parameter gather as two peer-memory kernels (csrc/comm/symm.cu).

Each rank's fp32 gradient buffer and bf16 parameter buffer live in symmetric memory.  After the last backward of a
step a rank raises its "gradients ready" flag on every peer; `rb_zero_reduce` waits for all flags, pulls this
rank's shard of every peer's gradients over NVLink and sums it in a fixed order, and publishes the shard's squared
norm; `rb_zero_adam_push` waits for all partial norms, clips, applies AdamW to the fp32 master shard and stores the
updated bf16 parameters straight into every rank's working copy, then raises "parameters pushed".  The next step
waits for that flag from all peers before its first kernel reads a parameter.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from .. import ops
from .symm import SignalPad, SymmetricBuffer


class RbZeroArgs(C.Structure):
    _fields_ = [
        ("grad_ptrs_dev", N.c_void_p), ("lowp_ptrs_dev", N.c_void_p), ("pad_ptrs_dev", N.c_void_p),
        ("local_pad", N.c_void_p), ("norm_slots", N.c_void_p), ("norm_ptrs_dev", N.c_void_p),
        ("grad_shard", N.c_void_p), ("master", N.c_void_p), ("m", N.c_void_p), ("v", N.c_void_p),
        ("partials", N.c_void_p),
        ("shard_off", N.c_ll), ("shard_len", N.c_ll), ("decay_end", N.c_ll),
        ("world", N.c_int), ("rank", N.c_int), ("epoch", C.c_uint),
        ("lr", N.c_float), ("beta1", N.c_float), ("beta2", N.c_float), ("eps", N.c_float), ("weight_decay", N.c_float),
        ("bc1", N.c_float), ("bc2", N.c_float), ("max_grad_norm", N.c_float),
        ("limit_ms", N.c_int),
    ]


N.optional_sig("rb_zero_reduce", [C.POINTER(RbZeroArgs), N.c_void_p])
N.optional_sig("rb_zero_adam_push", [C.POINTER(RbZeroArgs), N.c_void_p])


class FusedZeroComm:
    def __init__(self, trainer, limit_ms: int = 5000):
        t = trainer
        self.t = t
        P = t.engine.params
        pg, dev = t.pg, t.device
        self.world, self.rank = t.world, t.rank
        self.limit_ms = limit_ms
        # move the gradient and working-copy buffers into symmetric memory (same contents, new storage)
        self.grad_buf = SymmetricBuffer(P.total * 4, pg, dev)
        self.lowp_buf = SymmetricBuffer(P.total * 2, pg, dev)
        self.norm_buf = SymmetricBuffer(256, pg, dev)
        self.pad = SignalPad(pg, dev)
        new_grad = self.grad_buf.view(torch.float32, P.total)
        new_lowp = self.lowp_buf.view(torch.bfloat16, P.total)
        new_lowp.copy_(P.lowp)
        P.grad, P.lowp = new_grad, new_lowp
        # optimizer state only for the owned shard
        sl = t.shard
        self.master = P.master[sl].clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros(t.shard_len, dtype=torch.float32, device=dev)
        self.partials = torch.zeros(2048, dtype=torch.float32, device=dev)
        self.epoch = 0
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        torch.cuda.synchronize(dev)
        torch.distributed.barrier(group=pg)

    def _args(self, lr) -> RbZeroArgs:
        t = self.t
        eng = t.engine
        eng.step_count += 1
        a = RbZeroArgs()
        a.grad_ptrs_dev = self.grad_buf.ptrs_dev.data_ptr()
        a.lowp_ptrs_dev = self.lowp_buf.ptrs_dev.data_ptr()
        a.pad_ptrs_dev = self.pad.ptrs_dev.data_ptr()
        a.local_pad = self.pad.local_ptr
        a.norm_slots = self.norm_buf.local_ptr
        a.norm_ptrs_dev = self.norm_buf.ptrs_dev.data_ptr()
        a.grad_shard, a.master, a.m, a.v = (x.data_ptr() for x in (self.grad_shard, self.master, self.m, self.v))
        a.partials = self.partials.data_ptr()
        a.shard_off, a.shard_len, a.decay_end = t.shard.start, t.shard_len, eng.params.decay_end
        a.world, a.rank, a.epoch = self.world, self.rank, self.epoch
        a.lr = eng.lr if lr is None else lr
        a.beta1, a.beta2, a.eps, a.weight_decay = eng.betas[0], eng.betas[1], eng.eps, eng.weight_decay
        a.bc1 = 1.0 - eng.betas[0] ** eng.step_count
        a.bc2 = 1.0 - eng.betas[1] ** eng.step_count
        a.max_grad_norm = eng.max_grad_norm
        a.limit_ms = self.limit_ms
        return a

    def reduce_and_step(self, loss: torch.Tensor, lr):
        self.epoch += 1
        lib = N.kernels()
        a = self._args(lr)
        self.pad.signal_all(0, self.epoch)                     # my gradients are complete
        N.check(lib.rb_zero_reduce(a, N.stream_ptr()), "rb_zero_reduce")
        N.check(lib.rb_zero_adam_push(a, N.stream_ptr()), "rb_zero_adam_push")
        self.pad.wait_all(2, self.epoch, self.limit_ms)        # every peer's parameters have landed here
        # the loss is a scalar: one library all-reduce (a metric, not on the parameter path)
        self.loss_buf.copy_(loss.reshape(1))
        torch.distributed.all_reduce(self.loss_buf, group=self.t.pg)
        return self.loss_buf.view(())

    def gather_master(self) -> None:
        """Collects every rank's fp32 master shard into the full-size buffer (for checkpoints)."""
        P = self.t.engine.params
        torch.distributed.all_gather_into_tensor(P.master, self.master, group=self.t.pg)

    def reload_master(self) -> None:
        """After a checkpoint has been loaded into the full-size master buffer: refresh this rank's shard copy."""
        self.master.copy_(self.t.engine.params.master[self.t.shard])

    def optimizer_shard(self) -> tuple:
        """(m, v): Adam moments of this rank's flat shard."""
        return self.m, self.v

    def close(self):
        for b in (self.grad_buf, self.lowp_buf, self.norm_buf, self.pad):
            b.close()
