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


class HfError(RuntimeError):
    """crates/hf/src/lib.rs:53-75: `kind` is "hub" (the download failed or the file is not in the repository), "io" or
    "tensor" (the file is not a readable safetensors file)."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def download_state_dict(model_id: str, revision: str = "main") -> dict:
    """name -> fp32 tensor (other dtypes are converted; the reference keeps only F32 entries)."""
    try:
        path = fetch_url(hub_url(model_id, revision), None, os.path.join("hf", model_id.replace("/", "--"), revision),
                         "model.safetensors")
    except FetchError as e:
        raise HfError("hub", f"file 'model.safetensors' of repo '{model_id}' (revision {revision}) could not be fetched: {e}") from e
    except OSError as e:
        raise HfError("io", str(e)) from e
    try:
        tensors, _ = st.load_file(path)
    except st.IoError as e:
        raise HfError("tensor", f"{path}: {e}") from e
    return {k: v.float() for k, v in tensors.items() if v.is_floating_point()}


def save_state_dict_to_file(state: dict, path: str) -> None:
    st.save_file({k: torch.as_tensor(v, dtype=torch.float32) for k, v in state.items()}, path)


def load_from_hub(module, model_id: str, revision: str = "main", key_map=None, strict: bool = True) -> None:
    """Loads hub weights into a Saveable module; `key_map(name) -> name | None` renames / drops hub keys."""
    state = download_state_dict(model_id, revision)
    if key_map is not None:
        state = {nk: v for k, v in state.items() if (nk := key_map(k)) is not None}
    module.load_state_dict(state, strict=strict)


__all__ = ["hub_url", "download_state_dict", "save_state_dict_to_file", "load_from_hub", "FetchError", "HfError"]


# ---- checkpoint name conversion ---------------------------------------------------------------------------------
def _strip(state: dict, prefix: str) -> dict:
    return {(k[len(prefix):] if k.startswith(prefix) else k): v for k, v in state.items()}


def convert_hf_gpt2(state: dict, n_layer: int | None = None) -> dict:
    """Hugging Face GPT-2 names and layouts -> this framework's (`FlatParams.load_state_dict`).  GPT-2 stores its
    projections as Conv1D weights [in, out]; they are transposed to [out, in], and the fused c_attn is cut into
    wq / wk / wv.  The tied `lm_head.weight` and the causal-mask buffers (`attn.bias`, `attn.masked_bias`) are dropped."""
    s = _strip(state, "transformer.")
    out = {"tok_embed.embed": s["wte.weight"].float(), "pos_embed.embed": s["wpe.weight"].float(),
           "final_norm.weight": s["ln_f.weight"].float(), "final_norm.bias": s["ln_f.bias"].float()}
    layers = n_layer if n_layer is not None else 1 + max(int(k.split(".")[1]) for k in s if k.startswith("h."))
    for l in range(layers):
        h, p = f"h.{l}.", f"layers.{l}."
        d = s[h + "ln_1.weight"].shape[0]
        w, b = s[h + "attn.c_attn.weight"].float(), s[h + "attn.c_attn.bias"].float()
        for i, nm in enumerate(("wq", "wk", "wv")):
            out[p + f"attn.{nm}.weight"] = w[:, i * d:(i + 1) * d].t().contiguous()
            out[p + f"attn.{nm}.bias"] = b[i * d:(i + 1) * d].clone()
        out[p + "attn.wo.weight"] = s[h + "attn.c_proj.weight"].float().t().contiguous()
        out[p + "attn.wo.bias"] = s[h + "attn.c_proj.bias"].float()
        out[p + "ffn.fc1.weight"] = s[h + "mlp.c_fc.weight"].float().t().contiguous()
        out[p + "ffn.fc1.bias"] = s[h + "mlp.c_fc.bias"].float()
        out[p + "ffn.fc2.weight"] = s[h + "mlp.c_proj.weight"].float().t().contiguous()
        out[p + "ffn.fc2.bias"] = s[h + "mlp.c_proj.bias"].float()
        for src, dst in (("ln_1", "ln1"), ("ln_2", "ln2")):
            out[p + dst + ".weight"] = s[h + src + ".weight"].float()
            out[p + dst + ".bias"] = s[h + src + ".bias"].float()
    return out


def convert_hf_llama(state: dict, n_layer: int | None = None, tie_embeddings: bool = False) -> dict:
    """Hugging Face Llama names -> this framework's.  Layouts already agree ([out, in] matrices, rotate-half rotary
    pairs); gate_proj and up_proj are stacked into ffn.gate_up (gate rows first)."""
    s = _strip(state, "model.")
    out = {"tok_embed.embed": s["embed_tokens.weight"].float(), "final_norm.weight": s["norm.weight"].float()}
    if not tie_embeddings:
        out["head.weight"] = (s["lm_head.weight"] if "lm_head.weight" in s else s["embed_tokens.weight"]).float()
    layers = n_layer if n_layer is not None else 1 + max(int(k.split(".")[1]) for k in s if k.startswith("layers."))
    for l in range(layers):
        h, p = f"layers.{l}.", f"layers.{l}."
        for src, dst in (("q_proj", "wq"), ("k_proj", "wk"), ("v_proj", "wv"), ("o_proj", "wo")):
            out[p + f"attn.{dst}.weight"] = s[h + f"self_attn.{src}.weight"].float()
        out[p + "ffn.gate_up.weight"] = torch.cat([s[h + "mlp.gate_proj.weight"].float(), s[h + "mlp.up_proj.weight"].float()], 0)
        out[p + "ffn.down.weight"] = s[h + "mlp.down_proj.weight"].float()
        out[p + "ln1.weight"] = s[h + "input_layernorm.weight"].float()
        out[p + "ln2.weight"] = s[h + "post_attention_layernorm.weight"].float()
    return out


def export_hf_llama(state: dict, ffn_dim: int | None = None, tie_embeddings: bool = False) -> dict:
    """The inverse of `convert_hf_llama`: this framework's names -> Hugging Face Llama names, so that a model trained
    here loads into `transformers.LlamaForCausalLM.load_state_dict`."""
    out = {"model.embed_tokens.weight": state["tok_embed.embed"], "model.norm.weight": state["final_norm.weight"]}
    if not tie_embeddings:
        out["lm_head.weight"] = state["head.weight"]
    layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("layers."))
    for l in range(layers):
        p, h = f"layers.{l}.", f"model.layers.{l}."
        for src, dst in (("wq", "q_proj"), ("wk", "k_proj"), ("wv", "v_proj"), ("wo", "o_proj")):
            out[h + f"self_attn.{dst}.weight"] = state[p + f"attn.{src}.weight"]
        gu = state[p + "ffn.gate_up.weight"]
        f = ffn_dim or gu.shape[0] // 2
        out[h + "mlp.gate_proj.weight"], out[h + "mlp.up_proj.weight"] = gu[:f].clone(), gu[f:].clone()
        out[h + "mlp.down_proj.weight"] = state[p + "ffn.down.weight"]
        out[h + "input_layernorm.weight"] = state[p + "ln1.weight"]
        out[h + "post_attention_layernorm.weight"] = state[p + "ln2.weight"]
    return out


def export_hf_gpt2(state: dict) -> dict:
    """The inverse of `convert_hf_gpt2`: this framework's names -> Hugging Face GPT-2 names and Conv1D layouts
    (`transformer.*`, projections as [in, out]; the tied `lm_head.weight` is included)."""
    out = {"transformer.wte.weight": state["tok_embed.embed"], "transformer.wpe.weight": state["pos_embed.embed"],
           "transformer.ln_f.weight": state["final_norm.weight"], "transformer.ln_f.bias": state["final_norm.bias"],
           "lm_head.weight": state["tok_embed.embed"]}
    layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("layers."))
    for l in range(layers):
        p, h = f"layers.{l}.", f"transformer.h.{l}."
        out[h + "attn.c_attn.weight"] = torch.cat([state[p + f"attn.{nm}.weight"].t() for nm in ("wq", "wk", "wv")], 1).contiguous()
        out[h + "attn.c_attn.bias"] = torch.cat([state[p + f"attn.{nm}.bias"] for nm in ("wq", "wk", "wv")], 0)
        out[h + "attn.c_proj.weight"], out[h + "attn.c_proj.bias"] = state[p + "attn.wo.weight"].t().contiguous(), state[p + "attn.wo.bias"]
        out[h + "mlp.c_fc.weight"], out[h + "mlp.c_fc.bias"] = state[p + "ffn.fc1.weight"].t().contiguous(), state[p + "ffn.fc1.bias"]
        out[h + "mlp.c_proj.weight"], out[h + "mlp.c_proj.bias"] = state[p + "ffn.fc2.weight"].t().contiguous(), state[p + "ffn.fc2.bias"]
        for src, dst in (("ln1", "ln_1"), ("ln2", "ln_2")):
            out[h + dst + ".weight"], out[h + dst + ".bias"] = state[p + src + ".weight"], state[p + src + ".bias"]
    return out


def config_from_hf(hf_config) -> "GPTConfig":
    """GPTConfig for a Hugging Face GPT-2 or Llama configuration object (or dict)."""
    from ..models.config import GPTConfig
    c = hf_config if isinstance(hf_config, dict) else hf_config.to_dict()
    if c.get("model_type") == "gpt2":
        return GPTConfig(vocab_size=c["vocab_size"], seq_len=c["n_positions"], n_layer=c["n_layer"], n_head=c["n_head"],
                         d_model=c["n_embd"], ffn_dim=c.get("n_inner") or 4 * c["n_embd"], arch="gpt2", n_kv_head=c["n_head"],
                         norm_eps=c.get("layer_norm_epsilon", 1e-5), tie_embeddings=True)
    if c.get("model_type") == "llama":
        rope = c.get("rope_theta") or (c.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        return GPTConfig(vocab_size=c["vocab_size"], seq_len=c["max_position_embeddings"], n_layer=c["num_hidden_layers"],
                         n_head=c["num_attention_heads"], d_model=c["hidden_size"], ffn_dim=c["intermediate_size"], arch="llama",
                         n_kv_head=c.get("num_key_value_heads") or c["num_attention_heads"], rope_theta=float(rope),
                         norm_eps=c.get("rms_norm_eps", 1e-5), tie_embeddings=bool(c.get("tie_word_embeddings", False)))
    raise ValueError(f"unsupported Hugging Face model type {c.get('model_type')!r}")


__all__ += ["convert_hf_gpt2", "convert_hf_llama", "export_hf_llama", "export_hf_gpt2", "config_from_hf"]


def main(argv=None) -> int:
    """python -m rustral_b200.utils.hf convert --arch {gpt2,llama} IN.safetensors OUT.safetensors
    Rewrites a Hugging Face checkpoint file under this framework's parameter names (fp32), ready for
    `LMTrainer.load_state_dict` or `python -m rustral_b200.serve.http_server --weights`."""
    import argparse
    ap = argparse.ArgumentParser(prog="rustral_b200.utils.hf", description=main.__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("convert")
    c.add_argument("--arch", choices=["gpt2", "llama"], required=True)
    c.add_argument("--tie-embeddings", action="store_true", help="(llama) the model shares its embedding with the LM head")
    c.add_argument("src")
    c.add_argument("dst")
    a = ap.parse_args(argv)
    tensors, _ = st.load_file(a.src)
    out = convert_hf_gpt2(tensors) if a.arch == "gpt2" else convert_hf_llama(tensors, tie_embeddings=a.tie_embeddings)
    save_state_dict_to_file(out, a.dst)
    print(f"wrote {a.dst}: {len(out)} tensors, {sum(v.numel() for v in out.values())} parameters")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
