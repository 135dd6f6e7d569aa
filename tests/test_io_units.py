"""safetensors reader / writer (crates/io/src/lib.rs `mod tests`): every storage type round-trips bit for bit, the header
layout is the published format, and every kind of damaged file is refused with an IoError rather than a stray exception."""
import json
import struct

import pytest
import torch

from rustral_b200.core import CpuBackend, Parameter
from rustral_b200.io import safetensors_io as st

DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.uint8, torch.int8, torch.bool]


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_storage_type_round_trips_bit_for_bit(dtype):
    g = torch.Generator().manual_seed(1)
    if dtype == torch.bool:
        t = torch.rand(3, 5, generator=g) > 0.5
    elif dtype.is_floating_point:
        t = (torch.randn(3, 5, generator=g) * 100).to(dtype)
    else:
        t = torch.randint(0, 100, (3, 5), generator=g).to(dtype)
    back, meta = st.deserialize(st.serialize({"t": t}))
    assert meta == {} and back["t"].dtype == dtype and back["t"].shape == (3, 5) and torch.equal(back["t"], t)


def test_header_layout_is_the_published_format():
    blob = st.serialize({"b": torch.arange(6, dtype=torch.float32).view(2, 3), "a": torch.tensor([1, 2], dtype=torch.int64)},
                        {"format": "pt", "step": 7})
    (hlen,) = struct.unpack("<Q", blob[:8])
    assert hlen % 8 == 0
    header = json.loads(blob[8:8 + hlen])
    assert header["__metadata__"] == {"format": "pt", "step": "7"}                      # metadata values are strings
    assert header["a"] == {"dtype": "I64", "shape": [2], "data_offsets": [0, 16]}        # names sorted, offsets contiguous
    assert header["b"] == {"dtype": "F32", "shape": [2, 3], "data_offsets": [16, 40]}
    assert len(blob) == 8 + hlen + 40
    assert struct.unpack("<6f", blob[8 + hlen + 16:]) == (0.0, 1.0, 2.0, 3.0, 4.0, 5.0)  # little-endian row-major payload


def test_scalars_empty_tensors_and_non_contiguous_inputs():
    x = torch.arange(12.0).view(3, 4)
    back, _ = st.deserialize(st.serialize({"scalar": torch.tensor(2.5), "empty": torch.zeros(0, 4), "t": x.t()}))
    assert back["scalar"].shape == () and float(back["scalar"]) == 2.5
    assert back["empty"].shape == (0, 4) and torch.equal(back["t"], x.t())


def _with_header(header: dict, payload: bytes = b"") -> bytes:
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + payload


@pytest.mark.parametrize("blob,why", [
    (b"\x01\x02", "too short"),
    (struct.pack("<Q", 10 ** 9) + b"{}", "header length beyond the file"),
    (struct.pack("<Q", 0), "zero header length"),
    (struct.pack("<Q", 4) + b"\xff\xfe\x00\x01", "not UTF-8"),
    (struct.pack("<Q", 5) + b"{oops", "not JSON"),
    (_with_header([1, 2, 3]), "top level is not an object"),
    (_with_header({"t": {"dtype": "F32", "shape": [2]}}, b"\0" * 8), "entry without offsets"),
    (_with_header({"t": "F32"}), "entry is not an object"),
    (_with_header({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8), "range shorter than the shape"),
    (_with_header({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4), "range beyond the file"),
    (_with_header({"t": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, b"\0" * 8), "negative dimension"),
    (_with_header({"t": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8), "reversed range"),
    (_with_header({"t": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8), "unknown storage type"),
])
def test_damaged_files_are_refused_with_an_io_error(blob, why):
    with pytest.raises(st.IoError):
        st.deserialize(blob)


def test_reference_entry_points_flat_f32_and_strict_typed_loads(tmp_path):
    be = CpuBackend()
    w = be.normal_parameter("w", (2, 3), 1, 1.0)
    blob = st.save_parameters([("layer.w", w), ("layer.b", Parameter("b", torch.zeros(3)))])
    flat = st.load_parameters(blob)
    assert set(flat) == {"layer.w", "layer.b"} and flat["layer.w"].shape == (6,) and torch.equal(flat["layer.w"], w.tensor.detach().reshape(-1))
    mixed = st.save_state_dict_typed({"w": torch.ones(2), "ids": torch.tensor([1, 2])}, {"k": "v"})
    with pytest.raises(st.DTypeMismatch):
        st.load_state_dict_typed(mixed)                          # strict: F32 only
    tensors, meta = st.load_state_dict_typed(mixed, require_f32=False)
    assert meta == {"k": "v"} and tensors["ids"].dtype == torch.int64
    assert list(st.load_parameters(mixed)) == ["w"]              # the flat loader skips what is not F32
    flat2, _ = st.deserialize(st.save_state_dict({"v": [1, 2, 3], "m": torch.ones(2, 2)}))
    assert flat2["v"].dtype == torch.float32 and flat2["m"].shape == (4,)
    with pytest.raises(st.DTypeMismatch):
        st.serialize({"c": torch.zeros(2, dtype=torch.complex64)})
    path = tmp_path / "f.safetensors"
    st.save_file({"x": torch.arange(3.0)}, str(path), {"a": 1})
    assert not (tmp_path / "f.safetensors.partial").exists()
    back, meta = st.load_file(str(path))
    assert torch.equal(back["x"], torch.arange(3.0)) and meta == {"a": "1"}
