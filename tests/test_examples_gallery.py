"""Every small example runs end to end with reduced settings and reaches the result it advertises
(the reference's examples are exercised by `cargo test --examples` and its smoke tests in crates/runtime/tests)."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _run(name, argv, by_name=False):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)                       # the examples import their shared helpers as top-level modules
    if by_name:                                        # spawned ranks re-import the module by its name
        return importlib.import_module(name).main(argv)
    spec = importlib.util.spec_from_file_location(f"rustral_gallery_{name}", os.path.join(ROOT, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.main(argv)


def test_xor_is_learned_by_the_manual_loop_and_by_the_trainer():
    r = _run("xor", ["--epochs", "300"])
    assert r["manual"] == [0, 1, 1, 0] and r["trainer"] == [0, 1, 1, 0] and r["accuracy"] == 1.0
    assert r["loss_last"] < 0.05 < r["loss_first"]


def test_digit_convnet_learns():
    r = _run("mnist", ["--epochs", "4", "--train", "768"])
    assert r["accuracy_after"] > 0.85 and r["accuracy_after"] > r["accuracy_before"] + 0.5


def test_residual_network_trains_with_batch_norm_and_schedule():
    r = _run("resnet_image_classification", ["--epochs", "3", "--train", "512"])
    assert r["accuracy"] > 0.5 and "blocks.1.bn2.bias" in r["names"] and "stem.weight" in r["names"]


def test_char_rnn_and_nanogpt_reduce_the_loss_and_generate_text():
    r = _run("char_rnn", ["--steps", "60"])
    assert r["loss_last"] < r["loss_first"] - 0.8 and len(r["sample"]) == 84 and r["sample"].startswith("the ")
    g = _run("nanogpt", ["--steps", "80"])
    assert g["loss_last"] < g["loss_first"] - 1.0 and g["roundtrip"] and len(g["text"]) == 64


def test_diffusion_samples_land_near_the_data():
    r = _run("diffusion_model", ["--steps", "300"])
    assert r["loss_last"] < 0.6 * r["loss_first"] and r["sample_distance"] < 0.7 * r["noise_distance"]


def test_moe_training_balances_the_experts():
    r = _run("moe_training", ["--steps", "120"])
    assert r["accuracy"] > 0.97 and r["imbalance_after"] < min(1.3, r["imbalance_before"]) and min(r["tokens_per_expert"]) > 0


def test_seq2seq_reverses_sequences_by_greedy_decoding():
    r = _run("transformer_seq2seq", ["--steps", "350"])
    assert r["exact"] >= 0.9 * r["total"] and r["loss"] < 0.1


def test_bert_style_pretraining_then_fine_tuning():
    r = _run("bert_fine_tuning", ["--pretrain-steps", "100", "--finetune-steps", "40"])
    assert r["mlm_loss"] < 3.5 and r["accuracy_after"] > 0.95 > r["accuracy_before"]


def test_loss_scaling_recovers_from_overflow():
    r = _run("mixed_precision_training", ["--steps", "80"])
    assert r["skipped"] >= 1 and r["lowest_scale"] < 2.0 ** 127 and r["loss_mixed"] < 0.2 * r["loss_first"]
    assert abs(r["loss_mixed"] - r["loss_fp32"]) < 0.5 * r["loss_fp32"] + 1.0


def test_readouts_custom_layer_and_fusion_tour(tmp_path):
    r = _run("linear_readout", [])
    assert r["accuracy"] > 0.97 and r["multi_accuracy"] > 0.85 and all(l in ("negative", "neutral", "positive") for l in r["first"])
    c = _run("custom_layer", ["--out", str(tmp_path / "layer.safetensors")])
    assert c["names"] == ["norm.weight", "norm.bias", "value.weight", "gate_weight", "gate_bias"]
    assert c["roundtrip"] and c["loss_last"] < 0.3 * c["loss_first"] and os.path.getsize(c["path"]) > 2000
    f = _run("backend_agnostic_fusion", [])
    assert all(ok and err < 1e-4 for ok, err in f["results"].values())
    assert f["patterns"] == ["matmul_bias_gelu", "matmul_bias", "matmul_bias_relu"] and f["pool"]["hits"] == 2 and f["top"][0] == "matmul"
    b = _run("building_blocks", [])
    assert b["logits_shape"] == (4, 5) and len(b["rows"]) == 16 and dict((n, s) for n, s, _ in b["rows"])["LSTM over 10 steps"] == (10, 4, 48)
    assert len(_run("linear_benchmark", ["--iters", "1"])["rows"]) == 3


def test_dashboard_example_renders_frames_and_reports_the_leak(tmp_path):
    import json
    r = _run("train_dashboard", ["--plain", "--epochs", "2", "--batches", "10", "--dump", str(tmp_path / "state.json")])
    assert len(r["frames"]) == 2 and "loss" in r["frames"][-1] and "leak forgotten_buffer" in r["frames"][-1]
    assert r["has_leaks"] and r["accuracy"] > 0.5
    assert json.load(open(tmp_path / "state.json"))["epoch"] == 1


@pytest.mark.parametrize("overlap", [False, True])
def test_data_parallel_example_keeps_ranks_identical(overlap):
    r = _run("dp_cpu_gloo", ["--world", "2", "--steps", "30", "--port", "29531" if overlap else "29532"] + (["--overlap"] if overlap else []), by_name=True)
    assert r["identical"] and r["world"] == 2 and r["loss_last"] < r["loss_first"]
