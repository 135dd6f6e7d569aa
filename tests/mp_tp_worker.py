"""Worker for the fused tensor-parallel GEMM tests and micro-benchmark: one rank per GPU under torch.distributed.run.

ag_gemm and gemm_rs against all_gather / reduce_scatter + fp32 matmul, twice (bit-reproducibility and
               workspace parity), then a sequence-parallel column->row MLP, fused against the collective path,
               forward and backward.
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


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native
    from rustral_b200.parallel.fused_tp import FusedTP
    tp = FusedTP(None, dev)
    out = {"world": world}
    out.update(check(tp, rank, world, dev))
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
