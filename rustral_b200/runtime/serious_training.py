"""train_synthetic_classification: an end-to-end sanity run with a mid-run checkpoint round trip
(crates/runtime/src/serious_training.rs).  LCG-generated data, a linear softmax classifier, Adam."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import CpuBackend, ForwardCtx
from ..nn.linear import LinearBuilder
from ..optim import Adam
from .model_io import load_model, save_model


@dataclass
class SeriousTrainingConfig:
    seed: int = 42
    epochs: int = 400
    dataset_size: int = 128
    input_dim: int = 4
    num_classes: int = 3
    lr: float = 0.05
    checkpoint_dir: str | None = None


@dataclass
class SeriousTrainingOutcome:
    loss_start: float
    loss_end: float
    checkpoint_roundtrip_ok: bool


def _lcg_dataset(cfg):
    state = cfg.seed & 0xFFFFFFFF
    xs, ys = [], []
    centers = [[(c * 7 + d * 3) % 5 - 2.0 for d in range(cfg.input_dim)] for c in range(cfg.num_classes)]
    for i in range(cfg.dataset_size):
        c = i % cfg.num_classes
        row = []
        for d in range(cfg.input_dim):
            state = (1664525 * state + 1013904223) & 0xFFFFFFFF
            row.append(centers[c][d] + ((state >> 8) / float(1 << 24) - 0.5))
        xs.append(row)
        ys.append(c)
    return torch.tensor(xs), torch.tensor(ys)


def train_synthetic_classification(backend=None, cfg: SeriousTrainingConfig | None = None) -> SeriousTrainingOutcome:
    cfg = cfg or SeriousTrainingConfig()
    backend = backend or CpuBackend()
    x, y = _lcg_dataset(cfg)
    x = x.to(backend.device(), backend.dtype)
    y = y.to(backend.device())
    model = LinearBuilder(cfg.input_dim, cfg.num_classes).with_bias().seed(cfg.seed).build(backend)
    opt = Adam(lr=cfg.lr)
    ctx = ForwardCtx.train(backend)
    first = last = None
    ok = True
    for epoch in range(cfg.epochs):
        model.zero_grad()
        loss = ops.cross_entropy(model(x, ctx), y)
        loss.backward()
        opt.step(model.parameters())
        last = float(loss.detach())
        first = last if first is None else first
        if epoch == cfg.epochs // 2:
            blob = save_model(model)
            before = model(x, ForwardCtx.inference(backend)).detach().float().cpu()
            clone = LinearBuilder(cfg.input_dim, cfg.num_classes).with_bias().seed(cfg.seed + 99).build(backend)
            load_model(clone, blob)
            after = clone(x, ForwardCtx.inference(backend)).detach().float().cpu()
            ok = bool(torch.allclose(before, after, atol=1e-2 if backend.dtype != torch.float32 else 0.0))
            if cfg.checkpoint_dir:
                import os
                os.makedirs(cfg.checkpoint_dir, exist_ok=True)
                with open(os.path.join(cfg.checkpoint_dir, "mid.safetensors"), "wb") as f:
                    f.write(blob)
    return SeriousTrainingOutcome(first, last, ok)
