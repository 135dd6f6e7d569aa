"""Sequence / context parallelism: ring attention with contiguous or striped shards
(crates/distributed/src/sequence_parallel.rs:28-400, crates/distributed/src/context_parallel.rs:32-436).

Every rank holds a slice of the sequence.  Attention over the full sequence is computed block by block: at ring
step s a rank attends its queries against the K/V block that started on rank (r - s) mod W, then passes that block
on.  Partial results are merged with their log-sum-exp (o = sum_i o_i * exp(lse_i - lse)); the backward pass walks
the ring again using the FINAL (o, lse), so each block's gradient is exact.  The reference merges block outputs as if
they were logits, never rotates anything and applies no causal mask (sequence_parallel.rs:327-369).

Striped sharding (token t on rank t mod W) balances causal work: every (query block, key block) pair is roughly
half masked, instead of whole pairs being empty or full.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import attention as attn_ops
from .process_group import DistributedError, ProcessGroup


@dataclass
class SequenceParallelConfig:
    num_devices: int
    block_size: int = 1024
    use_ring_attention: bool = True
    striped: bool = False
    causal: bool = True


def shard_sequence(t: torch.Tensor, num_shards: int, shard_id: int, striped: bool = False, dim: int = 1) -> torch.Tensor:
    S = t.shape[dim]
    if S % num_shards:
        raise DistributedError("sequence length must be divisible by the number of shards")
    if striped:
        idx = torch.arange(shard_id, S, num_shards, device=t.device)
        return t.index_select(dim, idx).contiguous()
    per = S // num_shards
    return t.narrow(dim, shard_id * per, per).contiguous()


def gather_sequence(shards: list, striped: bool = False, dim: int = 1) -> torch.Tensor:
    if not striped:
        return torch.cat(shards, dim)
    W = len(shards)
    per = shards[0].shape[dim]
    shape = list(shards[0].shape)
    shape[dim] = per * W
    out = torch.empty(shape, dtype=shards[0].dtype, device=shards[0].device)
    for r, s in enumerate(shards):
        out.index_copy_(dim, torch.arange(r, per * W, W, device=s.device), s)
    return out


def compute_sequence_sharding(seq_len: int, num_devices: int) -> list:
    per = seq_len // num_devices
    return [(r * per, (r + 1) * per) for r in range(num_devices)]


def _block_forward(q, k, v, mode: str, scale: float):
    """One (query shard, key block) attention.  mode: "full", "causal" (diagonal included), "causal_strict"
    (diagonal excluded), "skip".  Returns (o [B,S,H,D] fp32-mergeable, lse [B,H,S]) or None."""
    if mode == "skip":
        return None
    if mode == "causal_strict":
        if q.shape[1] < 2:
            return None
        r = _block_forward(q[:, 1:], k[:, :-1], v[:, :-1], "causal", scale)
        o = torch.zeros_like(q)
        lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
        o[:, 1:] = r[0]
        lse[:, :, 1:] = r[1]
        return o, lse
    causal = mode == "causal"
    if q.is_cuda:
        o, lse = attn_ops.attention_forward(q, k, v, causal, scale)
        return o, lse
    B, Sq, H, D = q.shape
    qf = q.float().permute(0, 2, 1, 3)
    rep = H // k.shape[2]
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        Sk = k.shape[1]
        i = torch.arange(Sq)[:, None] + (Sk - Sq)
        s = s.masked_fill(torch.arange(Sk)[None, :] > i, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def _merge(acc, new):
    if new is None:
        return acc
    if acc is None:
        return new[0].float(), new[1]
    o_a, l_a = acc
    o_b, l_b = new
    lse = torch.logaddexp(l_a, l_b)
    wa = torch.exp(l_a - lse).permute(0, 2, 1).unsqueeze(-1)      # [B,S,H,1]
    wb = torch.exp(l_b - lse).permute(0, 2, 1).unsqueeze(-1)
    wa = torch.nan_to_num(wa, nan=0.0)
    wb = torch.nan_to_num(wb, nan=0.0)
    return o_a * wa + o_b.float() * wb, lse


def _block_mode(q_rank: int, kv_rank: int, causal: bool, striped: bool) -> str:
    if not causal:
        return "full"
    if striped:
        return "causal" if kv_rank <= q_rank else "causal_strict"
    if kv_rank < q_rank:
        return "full"
    return "causal" if kv_rank == q_rank else "skip"


def _ring_shift(pg: ProcessGroup, tensors: list, step_tag: int) -> list:
    """Sends every tensor to rank + 1 and receives the corresponding one from rank - 1."""
    W, r = pg.world_size, pg.rank
    out = [torch.empty_like(t) for t in tensors]
    if pg.backend == "torch" and tensors[0].is_cuda:
        import torch.distributed as dist
        ops_ = []
        for t, o in zip(tensors, out):
            dst = dist.get_global_rank(pg.group, (r + 1) % W) if pg.group is not None else (r + 1) % W
            src = dist.get_global_rank(pg.group, (r - 1) % W) if pg.group is not None else (r - 1) % W
            ops_.append(dist.P2POp(dist.isend, t.contiguous(), dst, pg.group))
            ops_.append(dist.P2POp(dist.irecv, o, src, pg.group))
        for req in dist.batch_isend_irecv(ops_):
            req.wait()
        return out
    for i, t in enumerate(tensors):         # even ranks send first, odd ranks receive first: no deadlock on blocking p2p
        tag = step_tag * 16 + i
        if r % 2 == 0:
            pg.send(t, (r + 1) % W, tag)
            pg.recv(out[i], (r - 1) % W, tag)
        else:
            pg.recv(out[i], (r - 1) % W, tag)
            pg.send(t, (r + 1) % W, tag)
    return out


class _RingAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pg, causal, striped, scale):
        W, r = pg.world_size, pg.rank
        acc = None
        kb, vb = k, v
        for s in range(W):
            src = (r - s) % W
            acc = _merge(acc, _block_forward(q, kb, vb, _block_mode(r, src, causal, striped), scale))
            if s + 1 < W:
                kb, vb = _ring_shift(pg, [kb, vb], s)
        o, lse = acc
        o = o.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (pg, causal, striped, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        pg, causal, striped, scale = ctx.meta
        W, r = pg.world_size, pg.rank
        dq = torch.zeros_like(q, dtype=torch.float32)
        kb, vb = k, v
        dkb = torch.zeros_like(k, dtype=torch.float32)
        dvb = torch.zeros_like(v, dtype=torch.float32)
        do = do.contiguous()
        for s in range(W):
            src = (r - s) % W
            mode = _block_mode(r, src, causal, striped)
            g = _block_backward(do, q, kb, vb, o, lse, mode, scale)
            if g is not None:
                dq += g[0].float()
                dkb += g[1].float()
                dvb += g[2].float()
            if s + 1 < W:
                kb, vb, dkb, dvb = _ring_shift(pg, [kb, vb, dkb, dvb], 100 + s)
        # after W - 1 shifts the gradient buffers sit one hop before their owner
        if W > 1:
            dkb, dvb = _ring_shift(pg, [dkb, dvb], 200)
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None, None


def _block_backward(do, q, k, v, o, lse, mode: str, scale: float):
    """Gradients of one block given the FINAL output and log-sum-exp of the whole ring."""
    if mode == "skip":
        return None
    if mode == "causal_strict":
        if q.shape[1] < 2:
            return None
        g = _block_backward(do[:, 1:], q[:, 1:], k[:, :-1], v[:, :-1], o[:, 1:], lse[:, :, 1:], "causal", scale)
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        dq[:, 1:], dk[:, :-1], dv[:, :-1] = g
        return dq, dk, dv
    causal = mode == "causal"
    if q.is_cuda:
        return attn_ops.attention_backward(do.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), o.contiguous(),
                                           lse.contiguous(), causal, scale)
    B, Sq, H, D = q.shape
    rep = H // k.shape[2]
    qf, dof, of = (t.float().permute(0, 2, 1, 3) for t in (q, do, o))
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        Sk = k.shape[1]
        i = torch.arange(Sq)[:, None] + (Sk - Sq)
        s = s.masked_fill(torch.arange(Sk)[None, :] > i, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    delta = (dof * of).sum(-1, keepdim=True)
    dv = p.transpose(-1, -2) @ dof
    ds = p * (dof @ vf.transpose(-1, -2) - delta)
    dq = ds @ kf * scale
    dk = ds.transpose(-1, -2) @ qf * scale
    Hk = k.shape[2]
    dk = dk.view(B, Hk, rep, -1, D).sum(2)
    dv = dv.view(B, Hk, rep, -1, D).sum(2)
    return dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)


class RingAttention:
    """Differentiable attention over a sequence sharded across `process_group` ([B, S_local, H, D] per rank)."""

    def __init__(self, process_group: ProcessGroup, config: SequenceParallelConfig | None = None):
        self.pg = process_group
        self.config = config or SequenceParallelConfig(process_group.world_size)
        self._peer = None

    def use_peer_memory(self, ring) -> "RingAttention":
        """Routes CUDA bf16 calls through `ring` (a `peer_ring.PeerRing` over the same ranks): K / V blocks are pulled
        from the owners' symmetric buffers over NVLink under the attention of the previous block instead of being
        relayed by send / recv.  Pass None to go back to the relayed path."""
        if ring is not None and ring.world != self.pg.world_size:
            raise DistributedError("the peer ring spans a different number of ranks")
        self._peer = ring
        return self

    def compute(self, q, k, v, scale: float | None = None):
        scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
        if self._peer is not None and q.is_cuda and q.dtype == torch.bfloat16:
            return self._peer.attention(q, k, v, self.config.causal, self.config.striped, scale)
        return _RingAttentionFn.apply(q, k, v, self.pg, self.config.causal, self.config.striped, scale)

    __call__ = compute


class _SeqToHeads(torch.autograd.Function):
    """[B, S/W, H, D] sharded by sequence -> [B, S, H/W, D] sharded by heads (one all-to-all); the backward pass is the
    inverse exchange."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _seq_to_heads(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g.contiguous(), ctx.pg), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _heads_to_seq(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g.contiguous(), ctx.pg), None


def _seq_to_heads(x, pg: ProcessGroup):
    W = pg.world_size
    B, Sl, H, D = x.shape
    if H % W:
        raise DistributedError("the number of heads must be divisible by the sequence-parallel size")
    # chunk r: this rank's tokens of head group r, leading dimension = local sequence for the exchange
    chunks = [x[:, :, r * (H // W):(r + 1) * (H // W)].permute(1, 0, 2, 3).contiguous() for r in range(W)]
    got = pg.all_to_all(chunks)                               # got[src]: [Sl, B, H/W, D], rank src's tokens
    return torch.cat(got, 0).permute(1, 0, 2, 3).contiguous()


def _heads_to_seq(x, pg: ProcessGroup):
    W = pg.world_size
    B, S, Hl, D = x.shape
    if S % W:
        raise DistributedError("the sequence length must be divisible by the sequence-parallel size")
    Sl = S // W
    chunks = [x[:, r * Sl:(r + 1) * Sl].permute(2, 0, 1, 3).contiguous() for r in range(W)]     # [Hl, B, Sl, D]
    got = pg.all_to_all(chunks)                               # got[src]: head group src of this rank's tokens
    return torch.cat(got, 0).permute(1, 2, 0, 3).contiguous()


class UlyssesAttention:
    """Sequence parallelism by head exchange: the sequence-sharded q / k / v ([B, S/W, H, D], contiguous shards) are
    all-to-all'ed into head shards over the FULL sequence ([B, S, H/W, D]), attention runs locally with the ordinary
    flash kernel (causal masks need no special handling), and one more all-to-all returns the output to sequence
    shards.  Four all-to-alls per layer move 4/W of the activations each; against ring attention this trades the
    W - 1 K/V block pulls for a bound of W <= number of KV heads.  The reference has no such path (its only
    all-to-all mention is a configuration flag, crates/nn/src/expert_choice.rs:49)."""

    def __init__(self, process_group: ProcessGroup, causal: bool = True):
        self.pg, self.causal = process_group, causal

    def compute(self, q, k, v, scale: float | None = None):
        W = self.pg.world_size
        if k.shape[2] % W or q.shape[2] % W:
            raise DistributedError("query and KV head counts must be divisible by the sequence-parallel size")
        if W == 1:
            return attn_ops.flash_attention(q, k, v, self.causal, scale)
        qh, kh, vh = (_SeqToHeads.apply(t, self.pg) for t in (q, k, v))
        o = attn_ops.flash_attention(qh, kh, vh, self.causal, scale)
        return _HeadsToSeq.apply(o, self.pg)

    __call__ = compute


@dataclass
class ContextParallelConfig:
    num_devices: int
    sequence_length: int = 131072
    block_size: int = 4096
    striped: bool = True
    use_ring_attention: bool = True
    all_gather_output: bool = False
    causal: bool = True

    def validate(self) -> None:
        if self.sequence_length % self.num_devices:
            raise DistributedError("sequence_length must be divisible by num_devices")
        if (self.sequence_length // self.num_devices) % self.block_size and self.sequence_length // self.num_devices > self.block_size:
            raise DistributedError("tokens per device must be a multiple of block_size")

    def tokens_per_device(self) -> int:
        return self.sequence_length // self.num_devices


@dataclass
class CommunicationStats:
    kv_bytes_per_step: int
    total_bytes: int
    steps: int


class ContextParallel:
    """Striped (load-balanced causal) ring attention with input sharding helpers."""

    def __init__(self, process_group: ProcessGroup, config: ContextParallelConfig):
        if process_group.world_size != config.num_devices:
            raise DistributedError("world size differs from config.num_devices")
        self.pg, self.config = process_group, config
        self.ring = RingAttention(process_group, SequenceParallelConfig(config.num_devices, config.block_size, True,
                                                                        config.striped, config.causal))

    def shard_input(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        return shard_sequence(x, self.pg.world_size, self.pg.rank, self.config.striped, dim)

    def forward(self, q, k, v, scale=None):
        o = self.ring.compute(q, k, v, scale)
        if self.config.all_gather_output:
            return gather_sequence(self.pg.all_gather(o), self.config.striped, 1)
        return o

    def communication_stats(self, kv_heads: int, head_dim: int, batch: int = 1, elem_bytes: int = 2) -> CommunicationStats:
        per = self.config.tokens_per_device() * batch * kv_heads * head_dim * 2 * elem_bytes
        steps = self.pg.world_size - 1
        return CommunicationStats(per, per * steps, steps)


class DynamicLoadBalancer:
    """Flags ranks whose measured step time exceeds `threshold` x the mean."""

    def __init__(self, world_size: int, threshold: float = 1.2):
        self.world_size, self.threshold = world_size, threshold
        self.times = [0.0] * world_size

    def report(self, rank: int, seconds: float) -> None:
        self.times[rank] = seconds

    def overloaded(self) -> list:
        mean = sum(self.times) / max(1, self.world_size)
        return [r for r, t in enumerate(self.times) if mean > 0 and t > self.threshold * mean]
