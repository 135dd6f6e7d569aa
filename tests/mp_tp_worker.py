"""Worker for the fused tensor-parallel GEMM tests and micro-benchmark: one rank per GPU under torch.distributed.run.

--mode check : ag_gemm and gemm_rs against all_gather / reduce_scatter + fp32 matmul, twice (bit-reproducibility and
               workspace parity), then a sequence-parallel column->row MLP, fused against the collective path,
               forward and backward.
--mode bench : device time of the fused primitives against NCCL collective + the same GEMM kernel, max over ranks.
Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel_err(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def check(tp, rank, world, dev):
    from rustral_b200.ops.matmul import gemm
    out = {}
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    rows, K, Nn = 256, 320, 192
    w = torch.randn(Nn, K, generator=torch.Generator().manual_seed(5)).mul(0.05).bfloat16().to(dev)
    errs, same = [], True
    prev = None
    for it in range(3):
        x_local = torch.randn(rows, K, generator=g).bfloat16().to(dev)
        y, x_full = tp.ag_gemm(x_local, w)
        gathered = [torch.empty_like(x_local) for _ in range(world)]
        dist.all_gather(gathered, x_local)
        xf = torch.cat(gathered, 0)
        ref = xf.float() @ w.float().t()
        errs.append(rel_err(y, ref))
        assert torch.equal(x_full, xf), "gathered operand differs from all_gather"
        y2, _ = tp.ag_gemm(x_local, w)
        same = same and torch.equal(y, y2)
    out["ag_gemm_err"] = max(errs)
    out["ag_gemm_repeatable"] = same

    M, Kl = rows * world, 256
    w2 = torch.randn(Nn, Kl, generator=g).mul(0.05).bfloat16().to(dev)
    errs, same = [], True
    for it in range(3):
        x = torch.randn(M, Kl, generator=g).bfloat16().to(dev)
        res = torch.randn(rows, Nn, generator=g).bfloat16().to(dev)
        y = tp.gemm_rs(x, w2, residual=res)
        partial = (x.float() @ w2.float().t())
        red = torch.empty(rows, Nn, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(red, partial.contiguous())
        errs.append(rel_err(y, red + res.float()))
        y2 = tp.gemm_rs(x, w2, residual=res)
        same = same and torch.equal(y, y2)
    out["gemm_rs_err"] = max(errs)
    out["gemm_rs_repeatable"] = same

    # FSDP / ZeRO-3: row-sharded weight gathered inside the consuming GEMM, gradient reduce-scattered inside the wgrad GEMM
    from rustral_b200.parallel.fused_tp import FSDPLinearFn
    n_r, Kf, Mf = 256, 192, 384
    w_full = torch.randn(n_r * world, Kf, generator=torch.Generator().manual_seed(9)).mul(0.05).bfloat16().to(dev)
    wsh = tp.shard_weight(w_full[rank * n_r:(rank + 1) * n_r])
    errs, same = [], True
    for it in range(2):
        xf = torch.randn(Mf, Kf, generator=g).bfloat16().to(dev)
        y, wf = tp.fsdp_gemm(xf, wsh)
        assert torch.equal(wf, w_full), "gathered weight differs"
        errs.append(rel_err(y, xf.float() @ w_full.float().t()))
        y2, _ = tp.fsdp_gemm(xf, wsh)
        same = same and torch.equal(y, y2)
    out["fsdp_gemm_err"] = max(errs)
    out["fsdp_gemm_repeatable"] = same
    xf = torch.randn(Mf, Kf, generator=g).bfloat16().to(dev).requires_grad_()
    wparam = wsh.tensor.detach().clone().requires_grad_()
    bias = torch.zeros(n_r * world, dtype=torch.bfloat16, device=dev, requires_grad=True)
    yf = FSDPLinearFn.apply(xf, wparam, bias, "gelu", tp, wsh)
    gyf = torch.randn(Mf, n_r * world, generator=g).bfloat16().to(dev)
    yf.backward(gyf)
    xr = xf.detach().float().requires_grad_()
    wr = w_full.float().requires_grad_()
    yr = torch.nn.functional.gelu(xr @ wr.t(), approximate="tanh")
    yr.backward(gyf.float())
    dw_sum = wr.grad.clone()
    dist.all_reduce(dw_sum)
    out["fsdp_layer_err"] = {"y": rel_err(yf, yr), "dx": rel_err(xf.grad, xr.grad),
                             "dw_shard": rel_err(wparam.grad, dw_sum[rank * n_r:(rank + 1) * n_r])}

    # sequence-parallel MLP: column (gelu) -> row, fused vs collectives
    from rustral_b200.core import B200Backend
    from rustral_b200.parallel.process_group import ProcessGroup
    from rustral_b200.parallel.tensor_parallel import TensorParallelLinear
    pg = ProcessGroup.from_torch()
    be = B200Backend(dev)
    d, hid, s_local = 256, 1024, 128
    grads = {}
    for fused in (False, True):
        col = TensorParallelLinear.column_parallel(be, d, hid, pg, bias=True, seed=3, sequence_parallel=True, activation="gelu")
        row = TensorParallelLinear.row_parallel(be, hid, d, pg, bias=False, seed=4, sequence_parallel=True)
        if fused:
            col.use_fused(tp)
            row.use_fused(tp)
        x = torch.randn(s_local, d, generator=torch.Generator().manual_seed(50 + rank)).bfloat16().to(dev).requires_grad_()
        col.weight.tensor.requires_grad_(); row.weight.tensor.requires_grad_(); col.bias.tensor.requires_grad_()
        y = row(col(x), residual=x)
        gy = torch.randn(s_local, d, generator=torch.Generator().manual_seed(70 + rank)).bfloat16().to(dev)
        y.backward(gy)
        grads[fused] = (y.detach(), x.grad, col.weight.tensor.grad, row.weight.tensor.grad, col.bias.tensor.grad)
    names = ["y", "dx", "dw_col", "dw_row", "db_col"]
    out["layer_err"] = {n: rel_err(a, b) for n, a, b in zip(names, grads[True], grads[False])}
    return out


def bench(tp, rank, world, dev, iters):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="check")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native
    from rustral_b200.parallel.fused_tp import FusedTP
    tp = FusedTP(None, dev)
    out = {"world": world}
    if a.mode == "check":
        out.update(check(tp, rank, world, dev))
    else:
        out["bench"] = bench(tp, rank, world, dev, a.iters)
    torch.cuda.synchronize()
    bufs = [tp.pad] + [b for ws in tp._ws.values() for b in (getattr(ws, "shard", None) or getattr(ws, "slots", None) or [ws.buf])]
    out["canaries_ok"] = all(b.check_canaries() for b in bufs)
    out["status"] = _native.read_status()[0]
    st = torch.tensor([out["status"]], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status_max"] = int(st)
    dist.barrier()
    tp.close()
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
