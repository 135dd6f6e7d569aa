"""Tensor-, pipeline- and expert-parallel training of the parallel decoder LM on two GPUs (tiny configs)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(port, *args, nproc=2):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rustral_b200.bench.parallel_train", "--steps", "5", "--warmup", "1",
           "--lr", "3e-3", "--same-batch", *args]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["device_status"] == 0
    return out


pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def test_tensor_parallel_fused_matches_collectives():
    fused = _run(29671, "--config", "tiny", "--tp", "2", "--global-batch", "4", "--micro-batch", "1")
    plain = _run(29672, "--config", "tiny", "--tp", "2", "--global-batch", "4", "--micro-batch", "1", "--unfused")
    assert fused["config"]["fused"] and not plain["config"]["fused"]
    for a, b in zip(fused["losses"], plain["losses"]):
        assert abs(a - b) < 5e-2, (fused["losses"], plain["losses"])
    assert fused["losses"][-1] < fused["losses"][0] - 0.05, fused["losses"]


def test_pipeline_parallel_1f1b_trains():
    out = _run(29673, "--config", "tiny", "--pp", "2", "--global-batch", "8", "--micro-batch", "2")
    assert out["losses"][-1] < out["losses"][0] - 0.05, out["losses"]


def test_expert_parallel_trains():
    out = _run(29674, "--config", "tiny-moe", "--ep", "2", "--global-batch", "8", "--micro-batch", "2")
    assert out["losses"][-1] < out["losses"][0] - 0.05, out["losses"]


def test_fsdp_fused_weight_gather_trains():
    out = _run(29675, "--config", "tiny", "--fsdp", "2", "--global-batch", "8", "--micro-batch", "2")
    assert out["config"]["parallelism"].endswith("fsdp2")
    assert out["losses"][-1] < out["losses"][0] - 0.05, out["losses"]


def test_context_parallel_matches_single_gpu():
    """Sequences split over two GPUs (striped and contiguous ring attention over peer memory) follow the single-GPU
    loss trajectory."""
    one = _run(29676, "--config", "tiny", "--global-batch", "4", "--micro-batch", "2", nproc=1)
    for port, extra in ((29677, []), (29678, ["--cp-contiguous"])):
        cp = _run(port, "--config", "tiny", "--cp", "2", "--global-batch", "4", "--micro-batch", "2", *extra)
        assert "cp2" in cp["config"]["parallelism"]
        for a, b in zip(cp["losses"], one["losses"]):
            assert abs(a - b) < 5e-2, (cp["losses"], one["losses"])
        assert cp["losses"][-1] < cp["losses"][0] - 0.05, cp["losses"]
