"""Worker for the expert-parallel tests: one rank per GPU under torch.distributed.run.

Every rank routes its own tokens through experts spread over all ranks (fused dispatch / combine over peer memory) and
compares outputs and gradients with the single-device expert layer given ALL experts' weights.  Rank 0 prints JSON.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel_err(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native
    from rustral_b200.ops import moe as M
    from rustral_b200.parallel.expert_parallel import FusedEP, ep_moe_mlp
    out = {"world": world}
    if True:
        E, d, F, T, k = 2 * world, 128, 256, 200 + 8 * rank, 2
        g = torch.Generator().manual_seed(11)
        router_w = (torch.randn(E, d, generator=g) * 0.5).bfloat16().to(dev)
        w1_all = (torch.randn(E, 2 * F, d, generator=g) * 0.05).bfloat16().to(dev)
        w2_all = (torch.randn(E, d, F, generator=g) * 0.05).bfloat16().to(dev)
        El = E // world
        ep = FusedEP(None, dev, E, d, max_tokens=200 + 8 * world, k=k)
        errs = {}
        for kind in ("swiglu", "gelu"):
            w1k = w1_all if kind == "swiglu" else w1_all[:, :F].contiguous()
            gx = torch.Generator().manual_seed(100 + rank)
            x = torch.randn(T, d, generator=gx).bfloat16().to(dev)
            gy = torch.randn(T, d, generator=gx).bfloat16().to(dev)
            # fused expert-parallel path, twice (buffers are reused, results must repeat bit for bit)
            res = []
            for rep in range(2):
                xe = x.clone().requires_grad_()
                rw = router_w.clone().requires_grad_()
                w1 = w1k[rank * El:(rank + 1) * El].clone().requires_grad_()
                w2 = w2_all[rank * El:(rank + 1) * El].clone().requires_grad_()
                y, aux = ep_moe_mlp(xe, rw, w1, w2, ep, k=k, kind=kind)
                (y.float() * gy.float()).sum().backward()
                res.append((y.detach(), xe.grad, w1.grad, w2.grad, rw.grad))
            assert all(torch.equal(p, q) for p, q in zip(res[0], res[1])), "expert-parallel run is not reproducible"
            # single-device reference on this rank's tokens with all experts
            xr = x.clone().requires_grad_()
            rwr = router_w.clone().requires_grad_()
            w1r = w1k.clone().requires_grad_()
            w2r = w2_all.clone().requires_grad_()
            yr, _ = M.moe_mlp(xr, rwr, w1r, w2r, k=k, kind=kind)
            (yr.float() * gy.float()).sum().backward()
            dw1 = w1r.grad.float().clone(); dist.all_reduce(dw1)
            dw2 = w2r.grad.float().clone(); dist.all_reduce(dw2)
            errs[kind] = {"y": rel_err(res[0][0], yr), "dx": rel_err(res[0][1], xr.grad),
                          "dw1": rel_err(res[0][2], dw1[rank * El:(rank + 1) * El]),
                          "dw2": rel_err(res[0][3], dw2[rank * El:(rank + 1) * El]),
                          "drouter": rel_err(res[0][4], rwr.grad)}
        out["err"] = errs
        ep.close()
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
