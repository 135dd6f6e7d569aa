"""End-to-end smoke of the CPU tiny-LM example (config: 2 layers, d128, vocab 1024, seq 64, batch 8, Adam 1e-3)."""
import importlib.util
import json
import os


def test_tiny_lm_cpu_trains_and_roundtrips(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("tiny_lm_cpu", os.path.join(root, "examples", "tiny_lm_cpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    m = mod.main(["--steps", "12", "--out", str(tmp_path)])
    assert m["loss_end"] < m["loss_start"] - 0.3 and m["checkpoint_roundtrip_ok"]
    assert abs(m["loss_start"] - 6.93) < 0.2                      # ln(1024) at initialisation
    assert json.load(open(tmp_path / "manifest.json"))["steps"] == 12
    assert (tmp_path / "model.safetensors").exists() and (tmp_path / "tiny_lm.jsonl").exists()
