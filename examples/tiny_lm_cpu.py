"""Tiny decoder-only LM on the CPU reference backend: 2 layers, d_model 128, 4 heads, FFN 512 (GELU), pre-LayerNorm,
learned positions, vocab 1024, seq 64, batch 8; token ids i.i.d. uniform from seed 0, targets = inputs shifted by one;
N(0, 0.02) init; Adam lr 1e-3 for 100 steps, loss logged, then a strict save / reload round trip.

    python examples/tiny_lm_cpu.py --steps 100 --out /tmp/tiny_lm
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustral_b200.io import safetensors_io as st          # noqa: E402
from rustral_b200.metrics import create_logger             # noqa: E402
from rustral_b200.models.config import preset              # noqa: E402
from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig   # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--out", default="/tmp/tiny_lm")
    ap.add_argument("--log-every", type=int, default=10)
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    cfg = preset("tiny-lm")
    tcfg = TrainConfig(global_batch=8, micro_batch=8, lr=1e-3, betas=(0.9, 0.999), weight_decay=0.0, max_grad_norm=0.0, seed=0)
    trainer = LMTrainer(cfg, tcfg, "cpu")
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g)     # one fixed batch: the loss must fall
    logger = create_logger(a.out, "tiny_lm", console=False)
    losses, t0 = [], time.perf_counter()
    for step in range(a.steps):
        loss = trainer.step(tokens)
        losses.append(loss)
        logger.log_scalar_with_step("train/loss", loss, step)
        if step % a.log_every == 0 or step == a.steps - 1:
            print(f"[step {step}] loss={loss:.4f}")
    dt = time.perf_counter() - t0
    logger.flush()
    path = os.path.join(a.out, "model.safetensors")
    st.save_file(trainer.state_dict(), path, {"rustral.model": json.dumps(cfg.to_dict())})
    reloaded = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=8, seed=123), "cpu")
    tensors, _ = st.load_file(path)
    reloaded.load_state_dict(tensors)
    a_log = trainer.engine.logits(tokens[:, :-1])
    b_log = reloaded.engine.logits(tokens[:, :-1])
    ok = bool(torch.equal(a_log, b_log))
    manifest = {"model": cfg.to_dict(), "steps": a.steps, "loss_start": losses[0], "loss_end": losses[-1],
                "ms_per_step": dt * 1e3 / a.steps, "tokens_per_s": a.steps * 8 * cfg.seq_len / dt,
                "checkpoint_roundtrip_ok": ok, "seed": 0}
    with open(os.path.join(a.out, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    print(json.dumps(manifest))
    return manifest


if __name__ == "__main__":
    main()
