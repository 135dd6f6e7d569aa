"""The fused engine on the GPU against the same engine on the CPU reference path."""
import pytest
import torch

from rustral_b200.models.config import preset
from rustral_b200.runtime.fused_gpt import FusedGPTEngine

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["gpt2-test", "llama-test"])
def test_engine_gpu_matches_cpu(name, cuda_status):
    cfg = preset(name)
    cpu = FusedGPTEngine(cfg, "cpu", micro_batch=2, seed=5, max_grad_norm=1.0)
    gpu = FusedGPTEngine(cfg, "cuda", micro_batch=2, seed=5, max_grad_norm=1.0)
    # same starting point: the GPU works on the bf16 rounding of the weights, give the CPU engine the same values
    cpu.params.master.copy_(gpu.params.lowp.float().cpu())
    cpu.params.sync_lowp()
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len), generator=g)
    tg = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len), generator=g)
    lc = cpu.train_step(ids, tg, do_step=False)
    lg = gpu.train_step(ids.cuda(), tg.cuda(), do_step=False)
    assert abs(float(lc) - float(lg)) < 2e-2, (float(lc), float(lg))
    gc, gg = cpu.params.grad, gpu.params.grad.cpu()
    for s in cpu.params.specs:
        a, b = gc[s.offset:s.offset + s.numel], gg[s.offset:s.offset + s.numel]
        rel = (a - b).norm() / (a.norm() + 1e-8)
        assert rel < 6e-2, f"{s.name}: relative gradient error {rel:.3g}"
    # a few optimizer steps keep the two trajectories together
    for _ in range(3):
        lc = cpu.train_step(ids, tg)
        lg = gpu.train_step(ids.cuda(), tg.cuda())
    assert abs(float(lc) - float(lg)) < 5e-2, (float(lc), float(lg))


def test_trainer_public_api_loss_decreases(cuda_status):
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
    cfg = preset("gpt2-test")
    tr = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=4, lr=1e-3), torch.device("cuda"))
    tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), dtype=torch.int64).pin_memory()
    losses = [tr.step(tokens) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses
