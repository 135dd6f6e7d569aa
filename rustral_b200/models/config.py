"""Model configurations for the decoder-only families (GPT-2 style and Llama style) and named presets."""
from __future__ import annotations

from dataclasses import dataclass, asdict


@dataclass
class GPTConfig:
    """Decoder-only transformer.

    arch "gpt2": pre-LayerNorm, learned positions, GELU MLP, biases, tied input/output embedding.
    arch "llama": RMSNorm, rotary positions, grouped-query attention, SwiGLU MLP, no biases, untied head.
    """
    vocab_size: int = 50257
    seq_len: int = 1024
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    ffn_dim: int = 3072
    arch: str = "gpt2"
    n_kv_head: int = 0
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = True
    init_std: float = 0.02
    vocab_multiple: int = 128      # the embedding / head are padded to this multiple for aligned GEMM tiles

    def __post_init__(self):
        if self.n_kv_head == 0:
            self.n_kv_head = self.n_head
        if self.d_model % self.n_head or self.n_head % self.n_kv_head:
            raise ValueError("d_model % n_head and n_head % n_kv_head must both be 0")
        if self.arch not in ("gpt2", "llama"):
            raise ValueError(f"unknown arch {self.arch!r}")
        if self.arch == "llama":
            self.tie_embeddings = False

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    @property
    def vocab_padded(self) -> int:
        m = self.vocab_multiple
        return (self.vocab_size + m - 1) // m * m

    @property
    def qkv_dim(self) -> int:
        return (self.n_head + 2 * self.n_kv_head) * self.head_dim

    def num_parameters(self, padded: bool = False) -> int:
        v = self.vocab_padded if padded else self.vocab_size
        d, f = self.d_model, self.ffn_dim
        if self.arch == "gpt2":
            per_layer = 2 * 2 * d + (self.qkv_dim * d + self.qkv_dim) + (d * d + d) + (f * d + f) + (d * f + d)
            return v * d + self.seq_len * d + self.n_layer * per_layer + 2 * d
        per_layer = 2 * d + self.qkv_dim * d + d * d + 2 * f * d + d * f
        return v * d + self.n_layer * per_layer + d + v * d

    def flops_per_token(self) -> float:
        """Training FLOPs per token: 6 x (matmul parameters) + causal attention."""
        d, f = self.d_model, self.ffn_dim
        mlp = (2 if self.arch == "gpt2" else 3) * f * d
        per_layer = self.qkv_dim * d + d * d + mlp
        matmul_params = self.n_layer * per_layer + self.vocab_padded * d
        attn = self.n_layer * 2 * self.seq_len * d      # QK^T and PV, causal half, per token, forward MACs*2/2
        return 6.0 * matmul_params + 3.0 * attn

    def to_dict(self) -> dict:
        return asdict(self)


PRESETS = {
    # tiny LM for the CPU reference backend
    "tiny-lm": dict(vocab_size=1024, seq_len=64, n_layer=2, n_head=4, d_model=128, ffn_dim=512, arch="gpt2",
                    tie_embeddings=False, vocab_multiple=1),
    # GPT-2 small: the headline training benchmark
    "gpt2-small": dict(vocab_size=50257, seq_len=1024, n_layer=12, n_head=12, d_model=768, ffn_dim=3072, arch="gpt2"),
    # Llama-style 8B: tensor / pipeline parallel training and serving
    "llama-8b": dict(vocab_size=128256, seq_len=4096, n_layer=32, n_head=32, n_kv_head=8, d_model=4096, ffn_dim=14336,
                     arch="llama", rope_theta=500000.0),
    # small shapes for tests
    "gpt2-test": dict(vocab_size=1000, seq_len=128, n_layer=2, n_head=4, d_model=256, ffn_dim=1024, arch="gpt2"),
    "llama-test": dict(vocab_size=1000, seq_len=128, n_layer=2, n_head=4, n_kv_head=2, d_model=256, ffn_dim=512,
                       arch="llama", rope_theta=10000.0),
}


def preset(name: str, **overrides) -> GPTConfig:
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return GPTConfig(**cfg)
