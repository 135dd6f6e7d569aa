"""save_model / load_model: strict safetensors checkpoints keyed by NamedParameters paths
(crates/runtime/src/model_io.rs:15-134).  F32 on disk, shapes preserved, metadata key `rustral.parameter_ids`.
Loading validates everything (missing keys, extra keys, shapes, element counts, dtype) before any parameter changes."""
from __future__ import annotations

import json

import torch

from ..core.errors import SerializationError, ShapeMismatch
from ..io import safetensors_io as st


def save_model(model) -> bytes:
    named = model.named_parameters()
    tensors = {n: p.tensor.detach().float().cpu() for n, p in named}
    meta = {"rustral.parameter_ids": json.dumps({n: int(p.id) for n, p in named})}
    return st.save_state_dict_typed(tensors, meta)


def load_model(model, blob: bytes) -> None:
    try:
        tensors, _ = st.load_state_dict_typed(blob, require_f32=True)
    except st.IoError as e:
        raise SerializationError(str(e)) from e
    named = dict(model.named_parameters())
    missing = sorted(k for k in named if k not in tensors)
    if missing:
        raise SerializationError(f"checkpoint is missing keys: {missing}")
    extra = sorted(k for k in tensors if k not in named)
    if extra:
        raise SerializationError(f"checkpoint has unexpected keys: {extra}")
    staged = []
    for k, p in named.items():
        t = tensors[k]
        if tuple(t.shape) != p.shape:
            raise ShapeMismatch(p.shape, t.shape, k)
        if t.numel() != p.numel():
            raise SerializationError(f"{k}: element count {t.numel()} != {p.numel()}")
        staged.append((p, t))
    for p, t in staged:
        p.set_(t.to(p.tensor.device))


def save_model_to_path(model, path: str) -> None:
    import os
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(save_model(model))
    os.replace(tmp, path)


def load_model_from_path(model, path: str) -> None:
    with open(path, "rb") as f:
        load_model(model, f.read())
