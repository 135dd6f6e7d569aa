"""Encoder, decoder and encoder-decoder stacks (crates/nn/src/transformer.rs:53-1088).

Built to the intended semantics: encoder layers transform their input (the reference's Module::forward of an
encoder layer returns it unchanged, transformer.rs:304-308), decoder layers apply their causal mask (never applied
in the reference, :662), and the encoder-decoder has real cross-attention (absent in the reference, :1028-1032).
Parameter names follow transformer.rs:323-368,515-566,893-954: token_embedding. / layers.{i}. / final_norm. / lm_head.
and per layer self_attn. / ff_linear1. / ff_linear2. / norm1. / norm2. (decoder with memory: cross_attn. / norm3.).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Saveable, Trainable, InvalidArgument
from .attention import SelfAttention, SelfAttentionConfig, scaled_dot_product_attention
from .dropout import Dropout
from .embedding import Embedding
from .linear import LinearBuilder
from .normalization import LayerNorm


class PositionalEncoding(Module):
    """Fixed sinusoidal table (base 10000), added to the embeddings; not trainable."""

    def __init__(self, d_model: int, max_len: int = 512, device="cpu", dtype=torch.float32, dropout: float = 0.0):
        pos = torch.arange(max_len, dtype=torch.float32)[:, None]
        div = torch.exp(torch.arange(0, d_model, 2, dtype=torch.float32) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, :d_model // 2]
        self.table = pe.to(device=device, dtype=dtype)
        self.max_len = max_len
        self._dropout = Dropout(dropout)

    def forward(self, x, ctx: ForwardCtx):
        """x: [B, S, d]."""
        S = x.shape[-2]
        if S > self.max_len:
            raise InvalidArgument(f"sequence length {S} exceeds max_len {self.max_len}")
        pe = self.table[:S].unsqueeze(0).expand_as(x).contiguous()
        return self._dropout(ops.binary("add", x.contiguous(), pe) if not x.requires_grad else x + pe, ctx)


@dataclass
class TransformerEncoderConfig:
    d_model: int
    num_heads: int
    num_layers: int
    ff_dim: int
    dropout: float = 0.1
    max_seq_len: int = 512
    pre_norm: bool = True
    vocab_size: int = 0


class TransformerEncoderLayer(Module, Trainable, Saveable):
    def __init__(self, config, self_attn, ff1, ff2, norm1, norm2, causal: bool = False):
        self.config = config
        self.self_attn, self.ff_linear1, self.ff_linear2, self.norm1, self.norm2 = self_attn, ff1, ff2, norm1, norm2
        self._dropout = Dropout(config.dropout)
        self._causal = causal

    @classmethod
    def new(cls, backend, config, seed: int = 42, causal: bool = False):
        c = config
        sa = SelfAttention.new(backend, SelfAttentionConfig(c.d_model, c.num_heads, dropout=c.dropout, causal=causal), seed)
        ff1 = LinearBuilder(c.d_model, c.ff_dim).with_bias().seed(seed + 3).scale(0.02).zero_bias().activation("gelu").build(backend)
        ff2 = LinearBuilder(c.ff_dim, c.d_model).with_bias().seed(seed + 5).scale(0.02).zero_bias().build(backend)
        return cls(c, sa, ff1, ff2, LayerNorm.new(backend, c.d_model), LayerNorm.new(backend, c.d_model), causal)

    def forward(self, x, ctx: ForwardCtx, mask=None):
        if self.config.pre_norm:
            x = self.self_attn.forward(self.norm1(x, ctx), ctx, mask, residual=x)
            return self.ff_linear2(self._dropout(self.ff_linear1(self.norm2(x, ctx), ctx), ctx), ctx, residual=x)
        x = self.norm1(self.self_attn.forward(x, ctx, mask, residual=x), ctx)
        return self.norm2(self.ff_linear2(self._dropout(self.ff_linear1(x, ctx), ctx), ctx, residual=x), ctx)

    def __call__(self, x, ctx=None, mask=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), mask)


class TransformerEncoder(Module, Trainable, Saveable):
    def __init__(self, config, token_embedding, pos_encoding, layers, final_norm):
        self.config = config
        self.token_embedding = token_embedding
        self._pos = pos_encoding
        self.layers = layers
        self.final_norm = final_norm

    @classmethod
    def new(cls, backend, config: TransformerEncoderConfig, vocab_size: int | None = None, seed: int = 42):
        v = vocab_size or config.vocab_size
        emb = Embedding.new(backend, v, config.d_model, seed)
        pe = PositionalEncoding(config.d_model, config.max_seq_len, backend.device(), backend.dtype)
        layers = [TransformerEncoderLayer.new(backend, config, seed + 100 * (i + 1)) for i in range(config.num_layers)]
        return cls(config, emb, pe, layers, LayerNorm.new(backend, config.d_model))

    def forward(self, ids, ctx: ForwardCtx, mask=None):
        """ids: int64 [B, S] (a flat list is treated as one sequence).  Returns [B, S, d_model]."""
        ids = torch.as_tensor(ids, dtype=torch.int64)
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        x = self._pos(self.token_embedding(ids, ctx), ctx)
        for layer in self.layers:
            x = layer.forward(x, ctx, mask)
        return self.final_norm(x, ctx)

    def cls_token(self, ids, ctx: ForwardCtx):
        """Representation of the first position: [B, d_model]."""
        return self.forward(ids, ctx)[:, 0]


@dataclass
class TransformerDecoderConfig(TransformerEncoderConfig):
    pass


class TransformerDecoderLayer(TransformerEncoderLayer):
    """Causal self-attention (+ cross-attention over an encoder memory when one is passed) + feed-forward."""

    def __init__(self, config, self_attn, ff1, ff2, norm1, norm2, cross_attn=None, norm3=None):
        super().__init__(config, self_attn, ff1, ff2, norm1, norm2, causal=True)
        if cross_attn is not None:
            self.cross_attn, self.norm3 = cross_attn, norm3

    @classmethod
    def new(cls, backend, config, seed: int = 42, cross_attention: bool = False):
        base = TransformerEncoderLayer.new(backend, config, seed, causal=True)
        ca = n3 = None
        if cross_attention:
            ca = SelfAttention.new(backend, SelfAttentionConfig(config.d_model, config.num_heads, dropout=config.dropout), seed + 7)
            n3 = LayerNorm.new(backend, config.d_model)
        return cls(config, base.self_attn, base.ff_linear1, base.ff_linear2, base.norm1, base.norm2, ca, n3)

    def _cross(self, x, memory, ctx):
        ca = self.cross_attn
        c = ca.config
        B, S, _ = x.shape
        h = self.norm3(x, ctx)
        q = ca._proj[0](h, ctx).reshape(B, S, c.num_heads, c.head_dim)
        k = ca._proj[1](memory, ctx).reshape(B, memory.shape[1], c.num_kv_heads, c.head_dim)
        v = ca._proj[2](memory, ctx).reshape(B, memory.shape[1], c.num_kv_heads, c.head_dim)
        a = scaled_dot_product_attention(q, k, v, None, False)
        return ca._proj[3](a.reshape(B, S, -1), ctx, x)

    def forward(self, x, ctx: ForwardCtx, mask=None, memory=None):
        x = self.self_attn.forward(self.norm1(x, ctx), ctx, mask, residual=x)
        if memory is not None and hasattr(self, "cross_attn"):
            x = self._cross(x, memory, ctx)
        return self.ff_linear2(self._dropout(self.ff_linear1(self.norm2(x, ctx), ctx), ctx), ctx, residual=x)

    def __call__(self, x, ctx=None, mask=None, memory=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), mask, memory)


class TransformerDecoder(Module, Trainable, Saveable):
    def __init__(self, config, token_embedding, pos_encoding, layers, final_norm, lm_head):
        self.config = config
        self.token_embedding = token_embedding
        self._pos = pos_encoding
        self.layers = layers
        self.final_norm = final_norm
        self.lm_head = lm_head

    @classmethod
    def new(cls, backend, config: TransformerDecoderConfig, vocab_size: int | None = None, seed: int = 42,
            cross_attention: bool = False):
        v = vocab_size or config.vocab_size
        emb = Embedding.new(backend, v, config.d_model, seed)
        pe = PositionalEncoding(config.d_model, config.max_seq_len, backend.device(), backend.dtype)
        layers = [TransformerDecoderLayer.new(backend, config, seed + 100 * (i + 1), cross_attention)
                  for i in range(config.num_layers)]
        head = LinearBuilder(config.d_model, v).seed(seed + 9).scale(0.02).build(backend)
        return cls(config, emb, pe, layers, LayerNorm.new(backend, config.d_model), head)

    def hidden(self, ids, ctx: ForwardCtx, memory=None):
        ids = torch.as_tensor(ids, dtype=torch.int64)
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        x = self._pos(self.token_embedding(ids, ctx), ctx)
        for layer in self.layers:
            x = layer.forward(x, ctx, None, memory)
        return self.final_norm(x, ctx)

    def forward(self, ids, ctx: ForwardCtx, memory=None):
        """Logits [B, S, vocab]."""
        return self.lm_head(self.hidden(ids, ctx, memory), ctx)

    def generate_token(self, ids, ctx: ForwardCtx, memory=None) -> int:
        """Greedy next token of one sequence (full re-forward; the serving engine has the cached path)."""
        logits = self.forward(ids, ctx, memory)
        return int(ops.argmax_rows(logits[0, -1:].contiguous())[0])


@dataclass
class EncoderDecoderConfig:
    """Configurations of both halves (crates/nn/src/transformer.rs:963-985).  With `shared_embeddings` and equal
    vocabularies the decoder uses the encoder's token-embedding parameter (one tensor, listed once under the encoder)."""
    encoder: TransformerEncoderConfig
    decoder: "TransformerDecoderConfig"
    shared_embeddings: bool = True

    @classmethod
    def symmetric(cls, d_model: int, num_heads: int, num_layers: int, ff_dim: int, **kw) -> "EncoderDecoderConfig":
        return cls(TransformerEncoderConfig(d_model, num_heads, num_layers, ff_dim, **kw),
                   TransformerDecoderConfig(d_model, num_heads, num_layers, ff_dim, **kw), True)

    def with_shared_embeddings(self, shared: bool) -> "EncoderDecoderConfig":
        self.shared_embeddings = shared
        return self


class TransformerEncoderDecoder(Module, Trainable, Saveable):
    def __init__(self, encoder: TransformerEncoder, decoder: TransformerDecoder):
        self.encoder, self.decoder = encoder, decoder

    @classmethod
    def from_config(cls, backend, config: EncoderDecoderConfig, src_vocab: int, tgt_vocab: int, seed: int = 42):
        enc = TransformerEncoder.new(backend, config.encoder, src_vocab, seed)
        dec = TransformerDecoder.new(backend, config.decoder, tgt_vocab, seed + 1000, cross_attention=True)
        model = cls(enc, dec)
        model.config = config
        if config.shared_embeddings and src_vocab == tgt_vocab and config.encoder.d_model == config.decoder.d_model:
            dec.token_embedding = enc.token_embedding          # one Parameter object: gradients of both uses accumulate
        return model

    @classmethod
    def new(cls, backend, config: TransformerEncoderConfig, src_vocab: int, tgt_vocab: int, seed: int = 42):
        dec_cfg = TransformerDecoderConfig(**config.__dict__)
        return cls(TransformerEncoder.new(backend, config, src_vocab, seed),
                   TransformerDecoder.new(backend, dec_cfg, tgt_vocab, seed + 1000, cross_attention=True))

    def forward(self, src_tgt, ctx: ForwardCtx):
        src, tgt = src_tgt
        memory = self.encoder.forward(src, ctx)
        return self.decoder.forward(tgt, ctx, memory)

    def generate(self, src, ctx: ForwardCtx, bos: int, eos: int, max_len: int = 32) -> list:
        memory = self.encoder.forward(src, ctx)
        out = [bos]
        for _ in range(max_len):
            tok = self.decoder.generate_token(out, ctx, memory)
            out.append(tok)
            if tok == eos:
                break
        return out
