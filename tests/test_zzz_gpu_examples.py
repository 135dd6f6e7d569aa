"""The small examples on the B200 backend (`--device cuda:0`: bf16 parameters, native kernels, layer sizes that need the
padded GEMM path).  Shortened runs; what is asserted is that they run, stay finite and move in the right direction."""
import importlib
import math
import os
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _run(name, argv):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    return importlib.import_module(name).main(argv + ["--device", "cuda:0"])


def test_xor_and_custom_layer_on_the_gpu(cuda_status, tmp_path):
    r = _run("xor", ["--epochs", "100"])
    assert r["manual"] == [0, 1, 1, 0] and r["loss_last"] < 0.05
    c = _run("custom_layer", ["--out", str(tmp_path / "layer.safetensors")])
    assert c["roundtrip"] and c["loss_last"] < c["loss_first"]


def test_image_and_sequence_models_on_the_gpu(cuda_status):
    m = _run("mnist", ["--epochs", "2", "--train", "512"])
    assert m["accuracy_after"] > m["accuracy_before"]
    c = _run("char_rnn", ["--steps", "30"])
    assert c["loss_last"] < c["loss_first"] and math.isfinite(c["loss_last"])
    g = _run("nanogpt", ["--steps", "40"])
    assert g["loss_last"] < g["loss_first"] and g["roundtrip"]


def test_transformer_moe_and_diffusion_examples_on_the_gpu(cuda_status):
    b = _run("bert_fine_tuning", ["--pretrain-steps", "30", "--finetune-steps", "20"])
    assert b["accuracy_after"] > 0.9
    m = _run("moe_training", ["--steps", "40"])
    assert m["accuracy"] > 0.9 and m["imbalance_after"] < m["imbalance_before"]
    d = _run("diffusion_model", ["--steps", "100"])
    assert d["loss_last"] < d["loss_first"] and d["sample_distance"] < d["noise_distance"]
    s = _run("transformer_seq2seq", ["--steps", "60"])
    assert math.isfinite(s["loss"])


def test_tour_examples_on_the_gpu(cuda_status):
    assert _run("building_blocks", [])["logits_shape"] == (4, 5)
    f = _run("backend_agnostic_fusion", [])
    assert f["patterns"] == ["matmul_bias_gelu", "matmul_bias", "matmul_bias_relu"] and set(f["results"]) == {"matmul_bias", "matmul_bias_relu", "matmul_bias_gelu"}
    assert all(err < 0.1 for _, err in f["results"].values())          # bf16: the unfused chain rounds three times, the fused one once
    r = _run("linear_readout", [])
    assert r["accuracy"] > 0.9
    mp = _run("mixed_precision_training", ["--steps", "40"])
    assert mp["skipped"] >= 1 and math.isfinite(mp["loss_mixed"])
