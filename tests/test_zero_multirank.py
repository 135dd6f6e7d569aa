"""ZeRO data parallelism over several ranks against the single-rank run of the same global batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "mp_zero_worker.py")


def _run(nproc, comm, device, port, extra_env=None, extra_args=()):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), WORKER, "--comm", comm, "--device", device, *extra_args]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


def test_zero_two_cpu_ranks_match_one_rank():
    one = _run(1, "nccl", "cpu", 29611)
    two = _run(2, "nccl", "cpu", 29612)
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 1e-4, (one["losses"], two["losses"])
    assert abs(one["checksum"] - two["checksum"]) < 1e-3 * abs(one["checksum"])
    assert two["losses"][-1] < two["losses"][0]


def test_zero_two_cpu_ranks_resume_from_per_rank_optimizer_state():
    """Each rank saves the Adam moments of ITS shard; a second trainer that loads weights + that state continues
    exactly like the first."""
    out = _run(2, "nccl", "cpu", 29613, extra_args=["--resume-check"])
    r = out["resume"]
    assert r["world"] == 2 and r["moments_numel"] == r["shard_len"]
    assert r["continued"] == r["resumed"]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("comm", ["nccl", "fused"])
def test_zero_two_gpus_match_one_gpu(comm):
    env = {"NCCL_NVLS_ENABLE": "0"}
    one = _run(1, "nccl", "cuda", 29621, env)
    two = _run(2, comm, "cuda", 29622 + (comm == "fused"), env)
    assert two["status"] == 0
    assert two["comm"] == ("FusedZeroComm" if comm == "fused" else "NcclZeroComm")
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 3e-2, (one["losses"], two["losses"])
    assert abs(one["checksum"] - two["checksum"]) < 2e-3 * abs(one["checksum"])
