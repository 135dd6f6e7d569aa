"""The parallel decoder LM (dense and mixture-of-experts) on one device: training reduces the loss on CPU, and the GPU
kernels give the same loss and gradients as the CPU reference path."""
import pytest
import torch

from rustral_b200.models.parallel_lm import MixedPrecisionAdamW, ParallelDecoderLM, ParallelLMConfig


def _cfg(moe: bool):
    return ParallelLMConfig(vocab_size=256, d_model=64, n_layer=2, n_head=2, n_kv_head=1, ffn_hidden=128, seq_len=32,
                            num_experts=4 if moe else 0, top_k=2)


@pytest.mark.parametrize("moe", [False, True])
def test_parallel_lm_trains_on_cpu(moe):
    cfg = _cfg(moe)
    model = ParallelDecoderLM(cfg, "cpu", seed=1)
    opt = MixedPrecisionAdamW(model, lr=3e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g)
    losses = []
    for _ in range(8):
        loss = model.forward_loss(tokens)
        loss.backward()
        opt.accumulate()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 0.2, losses
    assert cfg.num_params() > 0 and cfg.flops_per_token() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("moe", [False, True])
def test_parallel_lm_gpu_matches_cpu(moe):
    cfg = ParallelLMConfig(vocab_size=512, d_model=128, n_layer=2, n_head=2, n_kv_head=1, ffn_hidden=256, seq_len=128,
                           num_experts=4 if moe else 0, top_k=2)
    cpu = ParallelDecoderLM(cfg, "cpu", seed=3)
    gpu = ParallelDecoderLM(cfg, "cuda", seed=3)
    for n, p in cpu.params.items():            # same weights on both devices
        gpu.params[n].data.copy_(p.data)
    tokens = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=torch.Generator().manual_seed(5))
    lc = cpu.forward_loss(tokens)
    lc.backward()
    lg = gpu.forward_loss(tokens.cuda())
    lg.backward()
    assert abs(float(lc) - float(lg)) < 3e-2, (float(lc), float(lg))
    for n in ("l0.wqkv", "l1.wo", "wte", "head"):
        a, b = gpu.params[n].grad.float().cpu(), cpu.params[n].grad.float()
        assert (a - b).norm() / (b.norm() + 1e-9) < 8e-2, n
