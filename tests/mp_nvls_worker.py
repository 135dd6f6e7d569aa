"""Worker of the NVLink-multicast test: one rank per GPU under torch.distributed.run.  Every collective of
`parallel/nvls.py` against the same result computed from the peers' buffers with plain loads; rank 0 prints JSON.
(Ranks are ordered with NCCL barriers here; inside the trainer the flag kernels do it.)"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native as N
    from rustral_b200.parallel.nvls import MulticastBuffer
    N.kernels().rb_init()
    out = {"world": world}
    n = 1 << 20                                            # fp32 elements
    buf = MulticastBuffer(n * 4, None, dev)
    g = torch.Generator().manual_seed(100 + rank)
    mine = torch.randn(n, generator=g)
    buf.view(torch.float32, n).copy_(mine)
    torch.cuda.synchronize(); dist.barrier()
    # reference: the sum over ranks, in rank order, from the peers' buffers
    total = torch.zeros(n, device=dev)
    for r in range(world):
        total += buf.peer_view(r, torch.float32, n)
    per = n // world
    shard = torch.empty(per, device=dev)
    buf.reduce_into(shard, rank * per)
    torch.cuda.synchronize()
    ref = total[rank * per:(rank + 1) * per]
    out["reduce_max_err"] = float((shard - ref).abs().max())
    acc = torch.full((per,), 2.0, device=dev)
    buf.reduce_into(acc, rank * per, accumulate=True)
    torch.cuda.synchronize()
    out["accumulate_max_err"] = float((acc - ref - 2.0).abs().max())
    shard2 = torch.empty(per, device=dev)
    buf.reduce_into(shard2, rank * per)
    torch.cuda.synchronize()
    out["reduce_repeatable"] = bool(torch.equal(shard, shard2))
    dist.barrier()
    # all-reduce in place: every rank reduces its own slice through the switch and stores it to everybody
    buf.all_reduce_slice_(torch.float32)
    torch.cuda.synchronize(); dist.barrier()
    out["allreduce_max_err"] = float((buf.view(torch.float32, n) - total).abs().max())
    # bf16 elements
    dist.barrier()
    hb = (torch.randn(2 * n, generator=g) * 0.5).bfloat16()
    buf.view(torch.bfloat16, 2 * n).copy_(hb)
    torch.cuda.synchronize(); dist.barrier()
    tot16 = torch.zeros(2 * n, device=dev)
    for r in range(world):
        tot16 += buf.peer_view(r, torch.bfloat16, 2 * n).float()
    dist.barrier()
    buf.all_reduce_slice_(torch.bfloat16)
    torch.cuda.synchronize(); dist.barrier()
    got = buf.view(torch.bfloat16, 2 * n).float()
    out["allreduce_bf16_rel_err"] = float(((got - tot16).abs() / (tot16.abs() + 1.0)).max())
    # broadcast: rank 0's data lands in everybody's buffer
    dist.barrier()
    src = torch.arange(4096, dtype=torch.float32, device=dev) + 7.0
    if rank == 0:
        buf.broadcast_from(src, byte_offset=1024)
    torch.cuda.synchronize(); dist.barrier()
    out["broadcast_ok"] = bool(torch.equal(buf.view(torch.float32, 4096, byte_offset=1024), src))
    st = torch.tensor([N.read_status()[0]], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status_max"] = int(st)
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        merged = dict(gathered[0])
        for k in ("reduce_max_err", "accumulate_max_err", "allreduce_max_err", "allreduce_bf16_rel_err"):
            merged[k] = max(g_[k] for g_ in gathered)
        for k in ("reduce_repeatable", "broadcast_ok"):
            merged[k] = all(g_[k] for g_ in gathered)
        print(json.dumps(merged))
    dist.barrier()
    buf.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
