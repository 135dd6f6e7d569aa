"""The ONNX exporter's bytes parsed by the protobuf library against a schema declared here with the field numbers of
onnx.proto (the `onnx` package itself is not installed), and the exported graph evaluated with numpy
(crates/onnx-export/src/lib.rs `mod tests`)."""
import numpy as np
import pytest
import torch
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.nn import LinearBuilder
from rustral_b200.utils import onnx_export

F = descriptor_pb2.FieldDescriptorProto


def _schema():
    fd = descriptor_pb2.FileDescriptorProto(name="onnx_subset.proto", package="onnx", syntax="proto2")

    def msg(name, fields):
        m = fd.message_type.add(name=name)
        for fname, num, ftype, label, tname in fields:
            f = m.field.add(name=fname, number=num, type=ftype, label=label)
            if tname:
                f.type_name = ".onnx." + tname
    O, R = F.LABEL_OPTIONAL, F.LABEL_REPEATED
    msg("Dimension", [("dim_value", 1, F.TYPE_INT64, O, None), ("dim_param", 2, F.TYPE_STRING, O, None)])
    msg("TensorShapeProto", [("dim", 1, F.TYPE_MESSAGE, R, "Dimension")])
    msg("TypeTensor", [("elem_type", 1, F.TYPE_INT32, O, None), ("shape", 2, F.TYPE_MESSAGE, O, "TensorShapeProto")])
    msg("TypeProto", [("tensor_type", 1, F.TYPE_MESSAGE, O, "TypeTensor")])
    msg("ValueInfoProto", [("name", 1, F.TYPE_STRING, O, None), ("type", 2, F.TYPE_MESSAGE, O, "TypeProto")])
    msg("TensorProto", [("dims", 1, F.TYPE_INT64, R, None), ("data_type", 2, F.TYPE_INT32, O, None), ("name", 8, F.TYPE_STRING, O, None),
                        ("raw_data", 9, F.TYPE_BYTES, O, None)])
    msg("NodeProto", [("input", 1, F.TYPE_STRING, R, None), ("output", 2, F.TYPE_STRING, R, None), ("name", 3, F.TYPE_STRING, O, None),
                      ("op_type", 4, F.TYPE_STRING, O, None)])
    msg("GraphProto", [("node", 1, F.TYPE_MESSAGE, R, "NodeProto"), ("name", 2, F.TYPE_STRING, O, None),
                       ("initializer", 5, F.TYPE_MESSAGE, R, "TensorProto"), ("input", 11, F.TYPE_MESSAGE, R, "ValueInfoProto"),
                       ("output", 12, F.TYPE_MESSAGE, R, "ValueInfoProto")])
    msg("OperatorSetIdProto", [("domain", 1, F.TYPE_STRING, O, None), ("version", 2, F.TYPE_INT64, O, None)])
    msg("ModelProto", [("ir_version", 1, F.TYPE_INT64, O, None), ("producer_name", 2, F.TYPE_STRING, O, None),
                       ("producer_version", 3, F.TYPE_STRING, O, None), ("graph", 7, F.TYPE_MESSAGE, O, "GraphProto"),
                       ("opset_import", 8, F.TYPE_MESSAGE, R, "OperatorSetIdProto")])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("onnx.ModelProto"))


MODEL = _schema()


def _parse(blob):
    m = MODEL()
    m.ParseFromString(blob)
    assert m.SerializeToString(deterministic=True) and len(m.SerializeToString()) == len(blob)     # nothing unknown, nothing lost
    return m


def _run(model, x):
    """Evaluates the graph with numpy: initializers are fp32 raw data, nodes are MatMul / Add."""
    env = {"X": x}
    for t in model.graph.initializer:
        assert t.data_type == 1                                            # FLOAT
        env[t.name] = np.frombuffer(t.raw_data, dtype="<f4").reshape(tuple(t.dims))
    for n in model.graph.node:
        a, b = (env[i] for i in n.input)
        env[n.output[0]] = a @ b if n.op_type == "MatMul" else a + b
        assert n.op_type in ("MatMul", "Add")
    return env[model.graph.output[0].name]


@pytest.mark.parametrize("bias", [True, False])
def test_exported_linear_parses_and_computes_the_layers_output(bias):
    be = CpuBackend()
    b = LinearBuilder(5, 3).seed(4)
    lin = (b.with_bias() if bias else b).build(be)
    if bias:
        lin.bias.tensor.data.copy_(torch.tensor([0.5, -1.0, 2.0]))
    m = _parse(onnx_export.export_linear(lin))
    assert m.ir_version == 9 and m.producer_name == "rustral-b200" and [(o.domain, o.version) for o in m.opset_import] == [("", 17)]
    g = m.graph
    assert [n.op_type for n in g.node] == (["MatMul", "Add"] if bias else ["MatMul"]) and g.name == "linear"
    assert [t.name for t in g.initializer] == (["W", "B"] if bias else ["W"]) and list(g.initializer[0].dims) == [5, 3]
    xin, yout = g.input[0], g.output[0]
    assert xin.name == "X" and yout.name == "Y" and xin.type.tensor_type.elem_type == 1
    dims = lambda v: [(d.dim_param or d.dim_value) for d in v.type.tensor_type.shape.dim]
    assert dims(xin) == ["batch", 5] and dims(yout) == ["batch", 3]        # dynamic batch, static features
    x = np.random.default_rng(0).standard_normal((7, 5)).astype(np.float32)
    want = lin(torch.from_numpy(x), ForwardCtx.inference(be)).detach().numpy()
    assert np.allclose(_run(m, x), want, atol=1e-5)
    assert g.node[-1].output[0] == "Y" and (not bias or g.node[0].output[0] == g.node[1].input[0])


def test_export_rejects_a_weight_of_the_wrong_layout_and_handles_large_dims():
    with pytest.raises(ValueError):
        onnx_export.export_linear_f32(4, 3, torch.zeros(4, 3))             # [in, out] instead of [out, in]
    m = _parse(onnx_export.export_linear_f32(300, 200, torch.ones(200, 300)))   # dims above 127 need multi-byte varints
    assert list(m.graph.initializer[0].dims) == [300, 200] and len(m.graph.initializer[0].raw_data) == 300 * 200 * 4
