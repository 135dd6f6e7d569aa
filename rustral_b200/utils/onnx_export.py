"""ONNX export of a Linear as MatMul + Add, opset 17, dynamic batch (crates/onnx-export/src/lib.rs).

The ModelProto is serialised with a minimal protobuf writer (varints and length-delimited fields), so no protobuf
toolchain is needed; field numbers follow onnx.proto."""
from __future__ import annotations

import struct

import torch


def _varint(n: int) -> bytes:
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _ld(num: int, payload: bytes) -> bytes:          # length-delimited
    return _field(num, 2, _varint(len(payload)) + payload)


def _vi(num: int, v: int) -> bytes:
    return _field(num, 0, _varint(v))


def _s(num: int, text: str) -> bytes:
    return _ld(num, text.encode())


def _tensor(name: str, t: torch.Tensor) -> bytes:
    t = t.detach().float().contiguous()
    body = b"".join(_vi(1, d) for d in t.shape) + _vi(2, 1) + _s(8, name) + _ld(9, t.numpy().tobytes())   # dims, FLOAT, name, raw_data
    return body


def _value_info(name: str, dims) -> bytes:
    shape = b""
    for d in dims:
        dim = _s(2, d) if isinstance(d, str) else _vi(1, d)        # dim_param | dim_value
        shape += _ld(1, dim)
    tensor_type = _vi(1, 1) + _ld(2, shape)                           # elem_type FLOAT, shape
    return _s(1, name) + _ld(2, _ld(1, tensor_type))                  # name, type{tensor_type}


def _node(op: str, inputs, outputs, name: str) -> bytes:
    return b"".join(_s(1, i) for i in inputs) + b"".join(_s(2, o) for o in outputs) + _s(3, name) + _s(4, op)


class OnnxExportError(ValueError):
    """A weight or bias whose size does not match the declared layer (crates/onnx-export/src/lib.rs:17-24); `kind` is
    "weight_len" or "bias_len", `expected` / `got` are element counts."""

    def __init__(self, kind: str, expected: int, got: int, message: str):
        super().__init__(message)
        self.kind, self.expected, self.got = kind, expected, got


def export_linear_f32(in_features: int, out_features: int, weight: torch.Tensor, bias: torch.Tensor | None = None) -> bytes:
    """weight: [out, in] (this framework's layout) -> ONNX initializer W [in, out]; graph Y = X @ W (+ B)."""
    if tuple(weight.shape) != (out_features, in_features):
        raise OnnxExportError("weight_len", in_features * out_features, weight.numel(),
                              f"weight must be [out_features, in_features] = [{out_features}, {in_features}], got {tuple(weight.shape)}")
    if bias is not None and bias.numel() != out_features:
        raise OnnxExportError("bias_len", out_features, bias.numel(), f"bias must have {out_features} elements, got {bias.numel()}")
    W = weight.detach().float().t().contiguous()
    nodes = _ld(1, _node("MatMul", ["X", "W"], ["XW" if bias is not None else "Y"], "matmul"))
    inits = _ld(5, _tensor("W", W))
    if bias is not None:
        nodes += _ld(1, _node("Add", ["XW", "B"], ["Y"], "add"))
        inits += _ld(5, _tensor("B", bias))
    graph = nodes + _s(2, "linear") + inits + _ld(11, _value_info("X", ["batch", in_features])) + \
        _ld(12, _value_info("Y", ["batch", out_features]))
    opset = _s(1, "") + _vi(2, 17)
    model = _vi(1, 9) + _s(2, "rustral-b200") + _s(3, "0.1.0") + _ld(7, graph) + _ld(8, opset)    # ir_version 9
    return model


def export_linear(linear) -> bytes:
    return export_linear_f32(linear.config.in_dim, linear.config.out_dim, linear.weight.tensor,
                             None if linear.bias is None else linear.bias.tensor)
