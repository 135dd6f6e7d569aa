"""Model registry (crates/model-zoo/src/lib.rs + registry.json): named entries pointing at hub ids and local presets."""
from __future__ import annotations

from dataclasses import dataclass

REGISTRY_JSON = {
    "schema_version": "1.0",
    "entries": [
        {"id": "tiny-lm", "huggingface_model_id": None, "revision": None, "status": "builtin",
         "notes": "2-layer d128 decoder for the CPU reference backend", "local_artifact_workflow": "rustral_b200.models.preset('tiny-lm')"},
        {"id": "gpt2-small", "huggingface_model_id": "openai-community/gpt2", "revision": "main", "status": "architecture",
         "notes": "12 layers, d768, 12 heads, GELU, learned positions, tied head", "local_artifact_workflow": "rustral_b200.utils.hf.load_from_hub"},
        {"id": "llama-8b", "huggingface_model_id": "meta-llama/Meta-Llama-3-8B", "revision": "main", "status": "architecture",
         "notes": "32 layers, d4096, GQA 32/8, SwiGLU 14336, RoPE theta 500000", "local_artifact_workflow": "rustral_b200.utils.hf.load_from_hub"},
        {"id": "moe-8x", "huggingface_model_id": None, "revision": None, "status": "architecture",
         "notes": "24 layers, d2048, 8 SwiGLU experts of 8192, top-2", "local_artifact_workflow": "rustral_b200.nn.moe.ExpertLayer"},
    ],
}


@dataclass
class RegistryEntry:
    id: str
    huggingface_model_id: str | None
    revision: str | None
    status: str
    notes: str
    local_artifact_workflow: str


@dataclass
class Registry:
    schema_version: str
    entries: list

    def get(self, model_id: str) -> RegistryEntry | None:
        for e in self.entries:
            if e.id == model_id:
                return e
        return None


def registry() -> Registry:
    return Registry(REGISTRY_JSON["schema_version"], [RegistryEntry(**e) for e in REGISTRY_JSON["entries"]])
