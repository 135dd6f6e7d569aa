"""Plain-PyTorch arm of the headline benchmark: the same GPT-2-small-shaped decoder, batch, optimizer and metric as
`bench.py`, built only from stock PyTorch pieces: `nn.Linear` (cuBLAS), `F.scaled_dot_product_attention`,
`F.cross_entropy`, bf16 autocast over fp32 parameters, the fused `torch.optim.AdamW`, global-norm clipping, and
`torch.distributed.fsdp.FullyShardedDataParallel` (full sharding, one unit per transformer block) when there is more
than one rank.  Nothing of this framework is imported here: this is the library baseline the framework's number is
divided by (the reference's own PyTorch twins, benchmarks/pytorch/*.py, are the precedent for such an arm).

`run(...)` is called by `bench.py --impl torch` and, for the `vs_baseline` field, at the end of the framework's own run
on the same GPUs.
"""
from __future__ import annotations

import math
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d: int, heads: int, ffn: int, n_layer: int):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, ffn), nn.Linear(ffn, d)
        for lin in (self.qkv, self.fc1):
            nn.init.normal_(lin.weight, std=0.02)
        for lin in (self.proj, self.fc2):
            nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * n_layer))
        for lin in (self.qkv, self.proj, self.fc1, self.fc2):
            nn.init.zeros_(lin.bias)

    def forward(self, x):
        B, S, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, vocab: int, seq_len: int, n_layer: int, heads: int, d: int, ffn: int):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, d), nn.Embedding(seq_len, d)
        self.blocks = nn.ModuleList(Block(d, heads, ffn, n_layer) for _ in range(n_layer))
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.head.weight = self.tok.weight          # tied input / output embedding
        nn.init.normal_(self.tok.weight, std=0.02)
        nn.init.normal_(self.pos.weight, std=0.02)

    def forward(self, ids, targets, loss_scale: float):
        S = ids.shape[1]
        x = self.tok(ids) + self.pos(torch.arange(S, device=ids.device))
        for b in self.blocks:
            x = b(x)
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1), reduction="sum") * loss_scale


def run(*, vocab: int, seq_len: int, n_layer: int, heads: int, d_model: int, ffn: int, global_batch: int,
        micro_batch: int, steps: int, warmup: int, device, rank: int = 0, world: int = 1, lr: float = 3e-4,
        weight_decay: float = 0.1, max_grad_norm: float = 1.0, seed: int = 0) -> dict:
    """Trains `warmup` + `steps` optimizer steps twice (device-timed with tokens already on the GPU, then end to end
    from pinned host batches with the loss read back every step) and returns the timings.  Timings are the maximum
    over ranks."""
    import torch.distributed as dist
    torch.manual_seed(seed)
    model = GPT2(vocab, seq_len, n_layer, heads, d_model, ffn).to(device)
    if world > 1:
        import functools
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, MixedPrecision, ShardingStrategy
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy
        model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({Block}), sharding_strategy=ShardingStrategy.FULL_SHARD,
                     mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                                    buffer_dtype=torch.bfloat16),
                     device_id=device, use_orig_params=True, limit_all_gathers=True)
    decay = [p for n, p in model.named_parameters() if p.dim() >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=lr, betas=(0.9, 0.95), eps=1e-8, fused=True)
    local_b = global_batch // world
    mb = min(micro_batch, local_b)
    total_tokens = global_batch * seq_len
    loss_acc = torch.zeros((), device=device)

    def step(tokens_dev):
        loss_acc.zero_()
        n_micro = local_b // mb
        for i in range(n_micro):
            chunk = tokens_dev[i * mb:(i + 1) * mb]
            last = i == n_micro - 1
            # FSDP averages gradients over the ranks; the loss is scaled so that the result is the gradient of the
            # mean loss over the global batch.  Micro-batches before the last accumulate unsharded gradients locally.
            ctx = model.no_sync() if (world > 1 and not last) else _null()
            with ctx:
                with torch.autocast("cuda", dtype=torch.bfloat16, enabled=(world == 1)):
                    loss = model(chunk[:, :-1], chunk[:, 1:], float(world) / total_tokens)
                loss.backward()
            loss_acc.add_(loss.detach(), alpha=1.0 / world)
        if world > 1:
            model.clip_grad_norm_(max_grad_norm)
        else:
            torch.nn.utils.clip_grad_norm_(model.parameters(), max_grad_norm)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss_acc

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gen = torch.Generator().manual_seed(4321 + rank)
    host = [torch.randint(0, min(vocab, 50257), (local_b, seq_len + 1), generator=gen).pin_memory()
            for _ in range(2 * (warmup + steps))]
    dev = [h.to(device, non_blocking=True) for h in host[:warmup + steps]]
    torch.cuda.synchronize()
    for i in range(warmup):
        step(dev[i])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(dev[warmup + i])
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    del dev
    it = iter(host[warmup + steps:])
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
    stage = torch.empty((local_b, seq_len + 1), dtype=torch.int64, device=device)
    for _ in range(warmup):
        stage.copy_(next(it), non_blocking=True)
        step(stage)
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        stage.copy_(next(it), non_blocking=True)
        loss_host.copy_(step(stage), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    barrier()
    final = torch.tensor([float(loss_host)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
        dist.all_reduce(final)
    peak = torch.cuda.max_memory_allocated(device)
    del model, opt
    torch.cuda.empty_cache()
    return {"ms_per_step": float(ms) / steps, "e2e_ms_per_step": float(e2e) * 1e3 / steps, "tokens_per_step": total_tokens,
            "final_loss": float(final), "peak_mem_bytes": int(peak), "micro_batch": mb,
            "h2d_bytes_per_step": local_b * (seq_len + 1) * 8, "d2h_bytes_per_step": 4}


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
