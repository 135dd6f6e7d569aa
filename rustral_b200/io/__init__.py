"""Serialization: safetensors container and strict state-dict I/O."""
from .safetensors_io import (IoError, SafeTensorError, ShapeMismatchError, MissingTensor, DTypeMismatch, StateTensor,
                             serialize, deserialize, save_parameters, load_parameters, save_state_dict_typed,
                             load_state_dict_typed, save_state_dict, save_file, load_file)

__all__ = [n for n in dir() if not n.startswith("_")]
