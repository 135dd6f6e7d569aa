"""Peer-memory ring / context-parallel attention: kernels on one GPU, the sharded attention on two."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "mp_ring_worker.py")


@pytest.mark.gpu
def test_merge_fold_and_copy_kernels_match_fp32_reference():
    from rustral_b200 import _native as N
    from rustral_b200.parallel import peer_ring  # noqa: F401  (registers the signatures)
    from rustral_b200.parallel.sequence_parallel import _merge
    lib = N.kernels()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    B, S, H, D = 2, 67, 3, 64
    parts = []
    for i in range(3):
        o = torch.randn(B, S, H, D, generator=g).bfloat16().to(dev)
        lse = torch.randn(B, H, S, generator=g).mul(3).to(dev)
        if i == 1:
            lse[:, :, ::5] = float("-inf")            # rows with nothing visible in this block
        if i == 0:
            lse[:, :, 3] = float("-inf")              # ... and in the first block
        parts.append((o, lse))
    o_acc = torch.empty(B, S, H, D, dtype=torch.float32, device=dev)
    lse_acc = torch.empty(B, H, S, dtype=torch.float32, device=dev)
    acc = None
    for i, (o, lse) in enumerate(parts):
        N.check(lib.rb_attn_merge(o_acc.data_ptr(), lse_acc.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, H, D,
                                  1 if i == 0 else 0, N.stream_ptr()), "rb_attn_merge")
        dead = torch.isinf(lse).permute(0, 2, 1).unsqueeze(-1)
        acc = _merge(acc, (torch.where(dead, torch.zeros_like(o), o), lse))
    assert torch.allclose(lse_acc, acc[1], atol=1e-5, rtol=1e-5)
    assert torch.allclose(o_acc, acc[0], atol=1e-5, rtol=1e-4)
    # fold: bf16 slots, fp32 sum in rank order over the masked ranks
    W, n = 4, 4096 + 8
    slots = torch.randn(W, n, generator=g).bfloat16().to(dev)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    N.check(lib.rb_ring_fold(slots.data_ptr(), W, 0b1011, n, out.data_ptr(), N.stream_ptr()), "rb_ring_fold")
    ref = (slots[0].float() + slots[1].float() + slots[3].float()).bfloat16()
    assert torch.equal(out, ref)
    # copy: SM kernel and copy engine, odd multiple of 16 bytes
    src = torch.randint(0, 255, (16 * 100003,), dtype=torch.uint8, generator=g).to(dev)
    for ctas in (0, 7, -1):
        dst = torch.zeros_like(src)
        N.check(lib.rb_peer_copy(dst.data_ptr(), src.data_ptr(), src.numel(), ctas, N.stream_ptr()), "rb_peer_copy")
        assert torch.equal(dst, src)
    assert lib.rb_peer_copy(dst.data_ptr() + 8, src.data_ptr(), 32, 0, N.stream_ptr()) == -1      # misaligned: refused
    assert lib.rb_attn_merge(o_acc.data_ptr(), lse_acc.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, H, 60, 0,
                             N.stream_ptr()) == -1


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_ring_attention_two_gpus():
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29691", WORKER]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["status_max"] == 0 and out["canaries_ok"] and out["repeatable"], out
    for name, err in out["errs"].items():
        assert err < 2e-2, (name, out["errs"])
    for name, err in out["relay_match"].items():
        assert err < 1e-2, (name, out["relay_match"])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("causal,striped", [(True, False), (True, True), (False, False)])
def test_pull_and_deposit_schedules_agree(world, causal, striped):
    """Host-side schedule of the ring at larger world sizes: a rank deposits a key / value gradient with an owner
    exactly when the owner's fold mask expects it, every needed block is pulled once, nearest owner first, and
    causally invisible blocks are neither pulled nor expected."""
    from rustral_b200.parallel import sequence_parallel as sp
    from rustral_b200.parallel.peer_ring import PeerRing
    rings = []
    for r in range(world):
        ring = PeerRing.__new__(PeerRing)
        ring.world, ring.rank = world, r
        rings.append(ring)
    for r, ring in enumerate(rings):
        srcs = ring._sources(causal, striped)
        assert len({s for s, _ in srcs}) == len(srcs) and all(s != r for s, _ in srcs)
        dist_ = [(r - s) % world for s, _ in srcs]
        assert dist_ == sorted(dist_)                                  # nearest first
        for s, mode in srcs:
            assert mode == sp._block_mode(r, s, causal, striped) != "skip"
        visible = {s for s in range(world) if s != r and sp._block_mode(r, s, causal, striped) != "skip"}
        assert {s for s, _ in srcs} == visible
        if causal and not striped:
            assert visible == set(range(r))                            # only earlier shards
    for owner, ring in enumerate(rings):
        mask = ring._contributors(causal, striped)
        assert (mask >> owner) & 1                                     # the owner's own block
        for q in range(world):
            if q != owner:
                deposits = any(s == owner for s, _ in rings[q]._sources(causal, striped))
                assert deposits == bool((mask >> q) & 1), (owner, q)
