"""Worker for the peer-memory ring attention test: one rank per GPU under torch.distributed.run.

Forward and backward of contiguous and striped, causal and full attention over a sequence sharded across the ranks,
against an fp32 PyTorch attention of the whole sequence and against the send / recv ring; run twice for
bit-reproducibility; copy-kernel and copy-engine pulls.  Rank 0 prints one JSON line.  (Timings: the `ring` mode of
`rustral_b200.bench.comm_kernels`.)
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel_err(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def reference(q, k, v, causal):
    """fp32 attention over the full sequence with autograd; q [B,S,H,D], k / v [B,S,Hkv,D]."""
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    rep = q.shape[2] // k.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf.repeat_interleave(rep, 2)) / math.sqrt(q.shape[-1])
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), 1), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vf.repeat_interleave(rep, 2))
    return o, (qf, kf, vf)


def check(rank, world, dev, group):
    from rustral_b200 import _native as N
    from rustral_b200.parallel.peer_ring import PeerRing
    from rustral_b200.parallel.process_group import ProcessGroup
    from rustral_b200.parallel.sequence_parallel import RingAttention, SequenceParallelConfig, gather_sequence, shard_sequence
    B, S, H, Hkv, D = 2, 256 * world, 4, 2, 64
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(B, S, H, D, generator=gen).bfloat16().to(dev)
    k = torch.randn(B, S, Hkv, D, generator=gen).bfloat16().to(dev)
    v = torch.randn(B, S, Hkv, D, generator=gen).bfloat16().to(dev)
    do = torch.randn(B, S, H, D, generator=gen).bfloat16().to(dev)
    pg = ProcessGroup.from_torch(group)
    out = {"errs": {}, "repeatable": True, "relay_match": {}}
    rings = {"kernel": PeerRing(group, dev, B * (S // world) * Hkv * D, copy_ctas=64),
             "engine": PeerRing(group, dev, B * (S // world) * Hkv * D * 2, copy_ctas=-1)}     # also: block < capacity
    for striped in (False, True):
        for causal in (True, False):
            o_ref, (qf, kf, vf) = reference(q, k, v, causal)
            o_ref.backward(do.float())
            sh = lambda t: shard_sequence(t, world, rank, striped, 1)
            results = {}
            for name, ring in rings.items():
                for rep in range(2):
                    ql, kl, vl = (sh(t).clone().requires_grad_() for t in (q, k, v))
                    o = RingAttention(pg, SequenceParallelConfig(world, striped=striped, causal=causal)) \
                        .use_peer_memory(ring)(ql, kl, vl)
                    o.backward(sh(do))
                    cur = (o.detach(), ql.grad, kl.grad, vl.grad)
                    if rep and not all(torch.equal(a, b) for a, b in zip(cur, results[name])):
                        out["repeatable"] = False
                    results[name] = cur
            ql, kl, vl = (sh(t).clone().requires_grad_() for t in (q, k, v))
            o = RingAttention(pg, SequenceParallelConfig(world, striped=striped, causal=causal))(ql, kl, vl)
            o.backward(sh(do))
            relay = (o.detach(), ql.grad, kl.grad, vl.grad)
            tag = f"{'striped' if striped else 'contig'}_{'causal' if causal else 'full'}"
            refs = (sh(o_ref.detach()), sh(qf.grad), sh(kf.grad), sh(vf.grad))
            for name, res in results.items():
                out["errs"][f"{tag}_{name}"] = [rel_err(a, b) for a, b in zip(res, refs)]
            out["errs"][f"{tag}_relay"] = [rel_err(a, b) for a, b in zip(relay, refs)]
            out["relay_match"][tag] = max(rel_err(a, b) for a, b in zip(results["kernel"], relay))
    torch.cuda.synchronize()
    st = N.read_status()
    out["status"] = int(st[0])
    out["canaries_ok"] = all(r.check_canaries() for r in rings.values())
    for r in rings.values():
        r.close()
    return out


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    res = check(rank, world, dev, group)
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        merged = {"status_max": max(g["status"] for g in gathered), "canaries_ok": all(g["canaries_ok"] for g in gathered),
                  "repeatable": all(g["repeatable"] for g in gathered),
                  "errs": {key: max(max(g["errs"][key]) for g in gathered) for key in res["errs"]},
                  "relay_match": {key: max(g["relay_match"][key] for g in gathered) for key in res["relay_match"]}}
        print(json.dumps(merged))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
