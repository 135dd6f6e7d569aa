"""Device-timed micro-benchmarks of the peer-memory communication kernels against their library baselines.

One rank per GPU (torch.distributed.run); every number is CUDA-event time, maximum over ranks; rank 0 prints one JSON
line.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29650 \
        -m rustral_b200.bench.comm_kernels tp --iters 20
    ... -m rustral_b200.bench.comm_kernels ep --iters 10
    ... -m rustral_b200.bench.comm_kernels ring --iters 5 --seq-local 8192

* tp    all-gather -> GEMM, GEMM -> reduce-scatter and the sharded-weight gather -> GEMM fused over peer memory
        (`parallel.fused_tp.FusedTP`) against NCCL collective + the same GEMM kernel, and the GEMM alone;
* ep    one expert-parallel MoE layer forward (peer-memory dispatch / combine + grouped GEMM);
* nvls  in-switch reduce-scatter and all-reduce (`parallel.nvls.MulticastBuffer`: multimem.ld_reduce / multimem.st) against
        NCCL's reduce_scatter_tensor / all_reduce on the same sizes;
* ring  ring / striped context-parallel attention forward + backward: send / recv relay against K / V pulled from peer
        memory by a kernel or by the copy engines.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def bench_tp(tp, rank, world, dev, iters):
    from rustral_b200.ops.matmul import gemm
    res = []
    # (rows per rank, K, N of the all-gather GEMM) and the mirrored reduce-scatter GEMM, Llama-8B-like TP shapes
    shapes = [(8192 // world, 4096, 3 * 4096 // world), (8192 // world, 4096, 2 * 14336 // world)]
    for rows, K, Nn in shapes:
        M = rows * world
        x_local = torch.randn(rows, K, device=dev).bfloat16()
        w = torch.randn(Nn, K, device=dev).bfloat16() * 0.02
        gathered = torch.empty(M, K, dtype=torch.bfloat16, device=dev)

        def fused_ag():
            tp.ag_gemm(x_local, w)

        def nccl_ag():
            dist.all_gather_into_tensor(gathered, x_local)
            gemm(gathered, w)

        def gemm_only():
            gemm(gathered, w)

        x2 = torch.randn(M, Nn, device=dev).bfloat16()        # row layer: [M, k_local = Nn] x [K, Nn]^T
        w2 = torch.randn(K, Nn, device=dev).bfloat16() * 0.02
        part = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        red = torch.empty(rows, K, dtype=torch.bfloat16, device=dev)

        def fused_rs():
            tp.gemm_rs(x2, w2)

        def nccl_rs():
            gemm(x2, w2, out=part)
            dist.reduce_scatter_tensor(red, part)

        def gemm_only2():
            gemm(x2, w2, out=part)

        # FSDP: weight [Nn * world, K] row-sharded, tokens local
        wsh = tp.shard_weight(w)
        w_gathered = torch.empty(Nn * world, K, dtype=torch.bfloat16, device=dev)
        xt = torch.randn(M, K, device=dev).bfloat16()

        def fused_fsdp():
            tp.fsdp_gemm(xt, wsh)

        def nccl_fsdp():
            dist.all_gather_into_tensor(w_gathered, w)
            gemm(xt, w_gathered)

        def gemm_only3():
            gemm(xt, w_gathered)

        row = {"rows_per_rank": rows, "K": K, "N": Nn}
        for name, fn in (("fused_fsdp_gemm", fused_fsdp), ("nccl_allgather_w_then_gemm", nccl_fsdp), ("gemm_alone_fsdp_shape", gemm_only3),
                         ("fused_ag_gemm", fused_ag), ("nccl_ag_then_gemm", nccl_ag), ("gemm_alone", gemm_only),
                         ("fused_gemm_rs", fused_rs), ("gemm_then_nccl_rs", nccl_rs), ("gemm_alone_rs_shape", gemm_only2)):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            row[name + "_us"] = round(float(ms) * 1e3, 1)
        flops = 2.0 * M * K * Nn
        row["fused_ag_tflops"] = round(flops / (row["fused_ag_gemm_us"] * 1e-6) / 1e12, 1)
        row["fused_rs_tflops"] = round(flops / (row["fused_gemm_rs_us"] * 1e-6) / 1e12, 1)
        # bytes each GPU must pull (ag) or push (rs) over NVLink
        row["nvlink_bytes_ag"] = (world - 1) * rows * K * 2
        row["nvlink_bytes_rs"] = (world - 1) * rows * K * 2
        res.append(row)
    return res



def bench_ep(rank, world, dev, iters):
    from rustral_b200.parallel.expert_parallel import FusedEP, ep_moe_mlp
    out = {}
    # config-4-like layer: d 2048, FFN 8192 SwiGLU, 8 experts, top-2, 8192 local tokens
    E, d, F, T, k = 8, 2048, 8192, 8192, 2
    El = E // world
    ep = FusedEP(None, dev, E, d, max_tokens=T, k=k)
    x = torch.randn(T, d, device=dev).bfloat16()
    router_w = (torch.randn(E, d, device=dev) * 0.02).bfloat16()
    w1 = (torch.randn(El, 2 * F, d, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(El, d, F, device=dev) * 0.02).bfloat16()

    def fwd():
        with torch.no_grad():
            ep_moe_mlp(x, router_w, w1, w2, ep, k=k)

    for _ in range(3):
        fwd()
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fwd()
    e1.record(); torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    flops = 2.0 * T * k * d * (3 * F)          # per rank on average (uniform routing)
    out["ep_layer_fwd_ms"] = round(float(ms), 3)
    out["expert_tflops_per_gpu"] = round(flops / (float(ms) * 1e-3) / 1e12, 1)
    ep.close()
    return out


def bench_ring(rank, world, dev, group, a):
    from rustral_b200.parallel.peer_ring import PeerRing
    from rustral_b200.parallel.process_group import ProcessGroup
    from rustral_b200.parallel.sequence_parallel import RingAttention, SequenceParallelConfig
    B, Sl, H, Hkv, D = a.batch, a.seq_local, a.heads, a.kv_heads, a.head_dim
    gen = torch.Generator().manual_seed(rank)
    mk = lambda h: torch.randn(B, Sl, h, D, generator=gen).bfloat16().to(dev).requires_grad_()
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    do = torch.randn(B, Sl, H, D, generator=gen).bfloat16().to(dev)
    pg = ProcessGroup.from_torch(group)
    out = {"shape": [B, Sl, H, Hkv, D], "world": world}
    for striped in (False, True):
        variants = {"relay": None, "peer_kernel": PeerRing(group, dev, k.numel(), 64), "peer_engine": PeerRing(group, dev, k.numel(), -1)}
        for name, ring in variants.items():
            ra = RingAttention(pg, SequenceParallelConfig(world, striped=striped, causal=True)).use_peer_memory(ring)

            def step():
                for t in (q, k, v):
                    t.grad = None
                ra(q, k, v).backward(do)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            dist.barrier(group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                step()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out[f"{'striped' if striped else 'contig'}_{name}_ms"] = float(t)
        for ring in variants.values():
            if ring is not None:
                ring.close()
    return out



def bench_nvls(rank, world, dev, iters):
    """In-switch collectives (multimem.ld_reduce / multimem.st over an NVLink multicast buffer) against NCCL on the same
    sizes.  The kernels alone, back to back; ranks are aligned by a barrier before each timed loop."""
    from rustral_b200.parallel.nvls import MulticastBuffer

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e3                                    # microseconds, slowest rank

    rows = []
    for mb in (28, 256):                                         # one GPT-2-small layer's fp32 gradients; a large bucket
        n = mb * (1 << 20) // 4 // (world * 128) * (world * 128)
        buf = MulticastBuffer(n * 4, None, dev)
        buf.view(torch.float32, n).normal_()
        per = n // world
        shard = torch.empty(per, device=dev)
        src = torch.randn(n, device=dev)
        t_mc = timed(lambda: buf.reduce_into(shard, rank * per))
        t_nccl = timed(lambda: dist.reduce_scatter_tensor(shard, src))
        # bytes that reach this rank: its slice once through the switch; over peer loads it would be (world - 1) slices
        rows.append({"op": "reduce_scatter_f32", "mbytes": mb, "multimem_us": round(t_mc, 1), "nccl_us": round(t_nccl, 1),
                     "multimem_gbs_in": round(per * 4 / t_mc / 1e3, 1), "nccl_over_multimem": round(t_nccl / t_mc, 2)})
        torch.cuda.synchronize()
        dist.barrier()
        buf.close()
    for rows_, cols in ((64, 4096), (2048, 4096)):               # decode batch / prefill chunk activations, bf16
        n = rows_ * cols
        buf = MulticastBuffer(n * 2, None, dev)
        buf.view(torch.bfloat16, n).normal_()
        x = torch.randn(n, device=dev).bfloat16()
        t_mc = timed(lambda: buf.all_reduce_slice_(torch.bfloat16))
        t_nccl = timed(lambda: dist.all_reduce(x))
        rows.append({"op": "all_reduce_bf16", "shape": [rows_, cols], "multimem_us": round(t_mc, 1), "nccl_us": round(t_nccl, 1),
                     "nccl_over_multimem": round(t_nccl / t_mc, 2)})
        torch.cuda.synchronize()
        dist.barrier()
        buf.close()
    return {"bench": rows}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["tp", "ep", "ring", "nvls"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq-local", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native
    out = {"world": world, "what": a.what}
    if a.what == "tp":
        from rustral_b200.parallel.fused_tp import FusedTP
        tp = FusedTP(None, dev)
        out["bench"] = bench_tp(tp, rank, world, dev, a.iters)
        torch.cuda.synchronize()
        dist.barrier()
        tp.close()
    elif a.what == "ep":
        out.update(bench_ep(rank, world, dev, a.iters))
    elif a.what == "nvls":
        out.update(bench_nvls(rank, world, dev, a.iters))
    else:
        out.update(bench_ring(rank, world, dev, dist.group.WORLD, a))
    torch.cuda.synchronize()
    st = torch.tensor([_native.read_status()[0]], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status_max"] = int(st)
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
