"""Safetensors reader / writer and the strict state-dict I/O built on it (crates/io/src/lib.rs:17-278).

The container format is written and parsed here directly (8-byte little-endian header length, JSON header with
dtype / shape / data_offsets per tensor plus a ``__metadata__`` string map, then raw little-endian tensor bytes), so
checkpoints are byte-compatible with other safetensors tools without depending on one.  Loading is strict.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass

import numpy as np
import torch

from ..core.errors import CoreError


class IoError(CoreError):
    pass


class SafeTensorError(IoError):
    pass


class ShapeMismatchError(IoError):
    pass


class MissingTensor(IoError):
    pass


class DTypeMismatch(IoError):
    pass


_DT = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float64: "F64", torch.int64: "I64",
       torch.int32: "I32", torch.uint8: "U8", torch.int8: "I8", torch.bool: "BOOL"}
_RDT = {v: k for k, v in _DT.items()}
_SIZE = {"F32": 4, "BF16": 2, "F16": 2, "F64": 8, "I64": 8, "I32": 4, "U8": 1, "I8": 1, "BOOL": 1}


@dataclass
class StateTensor:
    shape: tuple
    dtype: str
    data: torch.Tensor


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype == torch.bool:
        return t.to(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def serialize(tensors: dict, metadata: dict | None = None) -> bytes:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    chunks, off = [], 0
    for name in sorted(tensors):
        t = tensors[name]
        if t.dtype not in _DT:
            raise DTypeMismatch(f"{name}: unsupported dtype {t.dtype}")
        raw = _raw_bytes(t)
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    return struct.pack("<Q", len(hjson)) + hjson + b"".join(chunks)


def deserialize(blob: bytes) -> tuple:
    """Returns (tensors: dict name -> torch.Tensor, metadata: dict)."""
    if len(blob) < 8:
        raise SafeTensorError("file too short for a safetensors header")
    (hlen,) = struct.unpack("<Q", blob[:8])
    if hlen <= 0 or 8 + hlen > len(blob):
        raise SafeTensorError("corrupt header length")
    try:
        header = json.loads(blob[8:8 + hlen].decode())
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafeTensorError(f"corrupt header: {e}") from e
    if not isinstance(header, dict):
        raise SafeTensorError("corrupt header: the top level must be an object")
    meta = header.pop("__metadata__", {}) or {}
    if not isinstance(meta, dict):
        raise SafeTensorError("corrupt header: __metadata__ must be an object")
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        try:
            dt, shape = info["dtype"], tuple(info["shape"])
            lo, hi = info["data_offsets"]
            ok = isinstance(dt, str) and all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape) \
                and isinstance(lo, int) and isinstance(hi, int)
        except (KeyError, TypeError, ValueError):
            ok = False
        if not ok:
            raise SafeTensorError(f"{name}: malformed entry (needs dtype, shape, data_offsets)")
        if dt not in _RDT:
            raise DTypeMismatch(f"{name}: unknown dtype {dt}")
        n = 1
        for d in shape:
            n *= d
        if lo < 0 or hi < lo or hi - lo != n * _SIZE[dt] or base + hi > len(blob):
            raise SafeTensorError(f"{name}: data range does not match shape {shape} of dtype {dt}")
        raw = blob[base + lo:base + hi]
        if dt == "BF16":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).copy()).view(torch.bfloat16)
        elif dt == "BOOL":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy()).bool()
        else:
            npdt = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I64": np.int64, "I32": np.int32,
                    "U8": np.uint8, "I8": np.int8}[dt]
            t = torch.from_numpy(np.frombuffer(raw, dtype=npdt).copy())
        out[name] = t.reshape(shape)
    return out, meta


# ---- the reference's entry points -----------------------------------------------------------------------------
def save_parameters(named_params) -> bytes:
    """[(name, Parameter)] -> safetensors bytes (F32, shapes preserved)."""
    return serialize({n: p.tensor.detach().float() for n, p in named_params})


def load_parameters(blob: bytes) -> dict:
    """name -> flat fp32 tensor, F32 entries only (other dtypes are skipped, as the reference does)."""
    tensors, _ = deserialize(blob)
    return {n: t.reshape(-1) for n, t in tensors.items() if t.dtype == torch.float32}


def save_state_dict_typed(state: dict, metadata: dict | None = None) -> bytes:
    """name -> tensor (any supported dtype) with shapes; metadata is a string map."""
    return serialize(state, metadata)


def load_state_dict_typed(blob: bytes, require_f32: bool = True) -> tuple:
    tensors, meta = deserialize(blob)
    if require_f32:
        bad = [n for n, t in tensors.items() if t.dtype != torch.float32]
        if bad:
            raise DTypeMismatch(f"non-F32 tensors in a strict F32 load: {bad}")
    return tensors, meta


def save_state_dict(state: dict) -> bytes:
    """name -> 1-D fp32 data."""
    return serialize({n: torch.as_tensor(v, dtype=torch.float32).reshape(-1) for n, v in state.items()})


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    import os
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(serialize(tensors, metadata))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def load_file(path: str) -> tuple:
    with open(path, "rb") as f:
        return deserialize(f.read())
