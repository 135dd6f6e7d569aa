"""Serving on the GPU: greedy tokens from the paged engine against the CPU reference engine on the same weights."""
import pytest
import torch

from rustral_b200.models.config import preset
from rustral_b200.runtime.fused_gpt import FlatParams
from rustral_b200.serve import ModelRunner, ServingEngine

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["gpt2-test", "llama-test"])
def test_gpu_engine_logits_match_cpu(name, cuda_status):
    cfg = preset(name)
    gpu = ModelRunner(cfg, device="cuda", num_blocks=64, seed=4)
    cpu = ModelRunner(cfg, device="cpu", num_blocks=64, seed=4)
    cpu.params.master.copy_(gpu.params.lowp.float().cpu())
    cpu.params.sync_lowp()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=g).tolist()
    for r in (gpu, cpu):
        assert r.cache.allocate(1, len(prompt) + 4)
    lg, lc = gpu.prefill(1, prompt), cpu.prefill(1, prompt)
    assert (lg.float().cpu() - lc).abs().max() < 0.05 * lc.abs().max() + 0.02
    tok = int(lc[:cfg.vocab_size].argmax())
    for step in range(3):
        n = len(prompt) + step + 1
        dg, dc = gpu.decode([1], [tok], [n]), cpu.decode([1], [tok], [n])
        assert (dg.float().cpu() - dc).abs().max() < 0.05 * dc.abs().max() + 0.02
        tok = int(dc[0, :cfg.vocab_size].argmax())


def test_gpu_engine_continuous_batching_completes(cuda_status):
    cfg = preset("llama-test")
    eng = ServingEngine(ModelRunner(cfg, device="cuda", num_blocks=128), max_batch_size=8)
    g = torch.Generator().manual_seed(1)
    ids = [eng.submit(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), 8) for n in (3, 30, 64, 17, 5)]
    done = eng.run_to_completion()
    assert len(done) == 5 and all(len(r.generated) == 8 for r in done)
    assert eng.runner.cache.free_blocks == 128


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("transport", ["peer", "nvls"])
def test_tensor_parallel_serving_matches_single_gpu(transport):
    """`nvls`: the per-layer all-reduces are summed inside the NVSwitch (multimem.ld_reduce); all ranks must still hold
    bit-identical logits, or their samplers would part ways."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ)
    env["TP_TRANSPORT"] = transport
    if transport == "peer":
        env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29681" if transport == "peer" else "29683", os.path.join(root, "tests", "mp_serve_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["status_max"] == 0 and out["ranks_identical"] and out["transport"] == transport
    assert out["prefill_rel_err"] < 3e-2, out
    # greedy decoding of random-init logits can flip on near ties; the first tokens must agree
    assert out["tokens_ref"][:4] == out["tokens_tp"][:4], out
