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


@pytest.mark.parametrize("stage", [2, 3])
def test_zero_two_cpu_ranks_match_one_rank(stage):
    one = _run(1, "nccl", "cpu", 29611)
    two = _run(2, "nccl", "cpu", 29612, extra_args=["--zero-stage", str(stage)])
    assert two["parallelism"] == ("dp2-zero3-collective" if stage == 3 else "dp2-zero2-nccl")
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 1e-5, (one["losses"], two["losses"])
    assert abs(one["checksum"] - two["checksum"]) < 1e-5 * abs(one["checksum"])
    assert two["losses"][-1] < two["losses"][0]
    for x, y in zip(one["probe"], two["probe"]):
        assert abs(x - y) < 1e-6


def test_zero3_four_cpu_ranks_hold_a_quarter_of_the_state():
    """Stage 3 over four ranks: same trajectory as one rank, and every rank's share of parameters, gradient
    accumulator and optimizer state is a quarter of the padded total (plus the buckets in flight)."""
    one = _run(1, "nccl", "cpu", 29614, extra_args=["--layers", "6"])
    four = _run(4, "nccl", "cpu", 29615, extra_args=["--zero-stage", "3", "--layers", "6"])
    for a, b in zip(one["losses"], four["losses"]):
        assert abs(a - b) < 1e-5
    sb, full = four["state_bytes"], one["state_bytes"]
    sharded = sb["param_shard"] + sb["optimizer_shard"] + sb["grad_shard"]
    whole = full["param_full"] + full["grad_full"] + full["optimizer_full"]
    assert sharded <= 0.27 * whole                       # a quarter, plus bucket padding
    assert sb["param_landing"] < full["param_full"] and sb["grad_landing"] < full["grad_full"]


@pytest.mark.parametrize("stage", [2, 3])
def test_zero_two_cpu_ranks_resume_from_per_rank_optimizer_state(stage):
    """Each rank saves the Adam moments of ITS shard; a second trainer that loads weights + that state continues
    exactly like the first."""
    out = _run(2, "nccl", "cpu", 29613, extra_args=["--resume-check", "--zero-stage", str(stage)])
    r = out["resume"]
    assert r["world"] == 2 and r["moments_numel"] == r["shard_len"]
    assert r["continued"] == r["resumed"]


def test_zero3_trainer_can_be_closed_and_rebuilt_in_one_process():
    out = _run(2, "nccl", "cpu", 29616, extra_args=["--reopen", "--zero-stage", "3"])
    assert out["reopened"] == out["losses"]              # same seed, same data: the second trainer repeats the first


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("comm,stage", [("nccl", 2), ("fused", 2), ("nccl", 3), ("fused", 3)])
def test_zero_two_gpus_match_one_gpu(comm, stage):
    env = {"NCCL_NVLS_ENABLE": "0"}
    one = _run(1, "nccl", "cuda", 29621, env, extra_args=["--steps", "6"])
    two = _run(2, comm, "cuda", 29622 + 2 * stage + (comm == "fused"), env, extra_args=["--zero-stage", str(stage), "--steps", "6"])
    assert two["status"] == 0
    want = {("nccl", 2): "dp2-zero2-nccl", ("fused", 2): "dp2-zero2-push", ("nccl", 3): "dp2-zero3-collective",
            ("fused", 3): "dp2-zero3-peer"}[(comm, stage)]
    assert two["parallelism"] == want
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 3e-2, (one["losses"], two["losses"])
    assert abs(one["checksum"] - two["checksum"]) < 2e-3 * abs(one["checksum"])


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("stage", [2, 3])
def test_fused_zero_trainer_can_be_closed_and_rebuilt_in_one_process(stage):
    """The second trainer gets fresh symmetric buffers (very likely at the addresses of the freed ones): its kernels
    must read ITS peer tables.  Six steps, so that the captured CUDA graphs of both trainers run as well."""
    out = _run(2, "fused", "cuda", 29641 + stage, {"NCCL_NVLS_ENABLE": "0"},
               extra_args=["--reopen", "--zero-stage", str(stage), "--steps", "6"])
    assert out["status"] == 0
    assert out["reopened"] == out["losses"]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nvlink_multicast_collectives_match_peer_loads():
    """multimem.ld_reduce / multimem.st kernels (in-switch reduce-scatter, all-reduce, broadcast) against sums formed from
    the peers' buffers with plain loads."""
    env = dict(os.environ)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29661", os.path.join(ROOT, "tests", "mp_nvls_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    if "no NVLink multicast address" in res.stdout + res.stderr:
        pytest.skip("this machine has no NVLink multicast")
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["status_max"] == 0 and out["reduce_repeatable"] and out["broadcast_ok"]
    assert out["reduce_max_err"] < 1e-5 and out["accumulate_max_err"] < 1e-5 and out["allreduce_max_err"] < 1e-5
    assert out["allreduce_bf16_rel_err"] < 1e-2


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_zero3_with_in_switch_reduce_scatter_matches_one_gpu():
    """ZeRO-3 with the gradient reduce-scatter done by multimem.ld_reduce through the NVSwitch."""
    one = _run(1, "nccl", "cuda", 29671, extra_args=["--steps", "6"])
    two = _run(2, "fused", "cuda", 29672, {"RUSTRAL_Z3_REDUCE": "nvls"}, extra_args=["--zero-stage", "3", "--steps", "6"])
    assert two["status"] == 0 and two["parallelism"] == "dp2-zero3-peer-nvls"
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 3e-2, (one["losses"], two["losses"])
    assert abs(one["checksum"] - two["checksum"]) < 2e-3 * abs(one["checksum"])
