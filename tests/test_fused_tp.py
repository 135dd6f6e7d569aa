"""Fused tensor-parallel GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter) on two GPUs against the collective path."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "mp_tp_worker.py")


def _run(nproc, port):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), WORKER]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tp_two_gpus():
    out = _run(2, 29641)
    assert out["status_max"] == 0 and out["canaries_ok"]
    assert out["ag_gemm_err"] < 1e-2 and out["ag_gemm_repeatable"]
    assert out["gemm_rs_err"] < 1e-2 and out["gemm_rs_repeatable"]
    for name, err in out["layer_err"].items():
        assert err < 3e-2, (name, out["layer_err"])
    assert out["fsdp_gemm_err"] < 1e-2 and out["fsdp_gemm_repeatable"]
    for name, err in out["fsdp_layer_err"].items():
        assert err < 3e-2, (name, out["fsdp_layer_err"])


def test_fused_tp_rejects_bad_shapes_on_cpu():
    """Argument checks of the Python layer need no GPU."""
    from rustral_b200.parallel.fused_tp import FusedTP, ROW_BLOCK
    tp = FusedTP.__new__(FusedTP)
    tp.world = 2
    assert tp.supports(ROW_BLOCK) and tp.supports(4 * ROW_BLOCK)
    assert not tp.supports(0) and not tp.supports(ROW_BLOCK + 8)
