"""Hugging Face Hub interop (crates/hf/src/lib.rs): fetch `model.safetensors`, read it into name -> fp32 tensor, load it
into a Saveable module.  Network access is optional: with RUSTRAL_DATASET_OFFLINE=1 (or no network) only files already
in the cache are used."""
from __future__ import annotations

import os

import torch

from ..data.fetch import FetchError, fetch_url
from ..io import safetensors_io as st


def hub_url(model_id: str, revision: str = "main", filename: str = "model.safetensors") -> str:
    return f"https://huggingface.co/{model_id}/resolve/{revision}/{filename}"


def download_state_dict(model_id: str, revision: str = "main") -> dict:
    """name -> fp32 tensor (other dtypes are converted; the reference keeps only F32 entries)."""
    path = fetch_url(hub_url(model_id, revision), None, os.path.join("hf", model_id.replace("/", "--"), revision),
                     "model.safetensors")
    tensors, _ = st.load_file(path)
    return {k: v.float() for k, v in tensors.items() if v.is_floating_point()}


def save_state_dict_to_file(state: dict, path: str) -> None:
    st.save_file({k: torch.as_tensor(v, dtype=torch.float32) for k, v in state.items()}, path)


def load_from_hub(module, model_id: str, revision: str = "main", key_map=None, strict: bool = True) -> None:
    """Loads hub weights into a Saveable module; `key_map(name) -> name | None` renames / drops hub keys."""
    state = download_state_dict(model_id, revision)
    if key_map is not None:
        state = {nk: v for k, v in state.items() if (nk := key_map(k)) is not None}
    module.load_state_dict(state, strict=strict)


__all__ = ["hub_url", "download_state_dict", "save_state_dict_to_file", "load_from_hub", "FetchError"]
