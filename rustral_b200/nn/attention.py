"""Attention modules (crates/nn/src/attention.rs:19-960, crates/nn/src/tape_transformer.rs:27-298).

All of them are real multi-head attention with a per-row softmax; on CUDA the score matrix is never
materialised (flash kernels).  The reference's SelfAttention is one head of width head_dim and soft-maxes over
the whole flattened score matrix (attention.rs:79-144); the intended semantics are built here instead.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Saveable, Trainable, InvalidArgument
from .dropout import Dropout
from .linear import Linear, LinearBuilder
from .normalization import LayerNorm


@dataclass
class SelfAttentionConfig:
    d_model: int
    num_heads: int
    head_dim: int = 0
    dropout: float = 0.0
    num_kv_heads: int = 0       # 0 = same as num_heads (MHA); fewer = GQA / MQA
    causal: bool = False
    rope_theta: float = 0.0     # > 0 applies rotary embeddings to q and k
    bias: bool = True

    def __post_init__(self):
        if self.d_model % self.num_heads:
            raise InvalidArgument("d_model must be divisible by num_heads")
        if self.head_dim == 0:
            self.head_dim = self.d_model // self.num_heads
        if self.num_kv_heads == 0:
            self.num_kv_heads = self.num_heads
        if self.num_heads % self.num_kv_heads:
            raise InvalidArgument("num_heads must be divisible by num_kv_heads")


def causal_mask(backend, seq_len: int, neg: float = float("-inf")) -> torch.Tensor:
    """[S, S] additive mask with `neg` above the diagonal (crates/nn/src/attention.rs:496)."""
    m = torch.zeros(seq_len, seq_len, dtype=torch.float32)
    m.masked_fill_(torch.triu(torch.ones(seq_len, seq_len, dtype=torch.bool), 1), neg)
    return m.to(backend.device())


def causal_mask_tape(backend, seq_len: int) -> torch.Tensor:
    """The tape variant uses -1e9 instead of -inf (crates/nn/src/tape_transformer.rs:280-298)."""
    return causal_mask(backend, seq_len, -1e9)


class KeyPaddingMask:
    """A key-padding mask given as the number of real keys per batch entry (the keys behind them are padding).  The
    flash kernels take it directly: padded key blocks are skipped, no [S, S] mask tensor exists."""

    def __init__(self, lengths):
        self.lengths = lengths if torch.is_tensor(lengths) else torch.tensor(list(lengths), dtype=torch.int32)

    @classmethod
    def from_token_ids(cls, ids: torch.Tensor, pad_id: int = 0):
        """Lengths of right-padded id rows [B, S]: position of the last non-pad token + 1."""
        keep = ids != pad_id
        pos = torch.arange(1, ids.shape[1] + 1, device=ids.device)
        return cls((keep * pos).amax(-1).to(torch.int32))


    @classmethod
    def from_additive(cls, mask: torch.Tensor, check: bool = True):
        """Lengths from an additive key mask of shape [B, Sk], [B, 1, Sk] or [B, 1, 1, Sk] (0 for real keys, -inf or a large
        negative number for padding), so that code that builds such tensors can use the flash kernels.  The padding has
        to be a suffix of every row; with `check` that is verified (one read-back of B x Sk booleans) and a mask of any
        other form gives None, which the caller passes on as the tensor it has."""
        m = mask.reshape(mask.shape[0], -1) if mask.dim() > 2 and mask.numel() == mask.shape[0] * mask.shape[-1] else mask
        if m.dim() != 2:
            return None
        real = m > -1e4
        lengths = real.sum(-1).to(torch.int32)
        if check:
            pos = torch.arange(m.shape[1], device=m.device)[None, :]
            if not bool((real == (pos < lengths[:, None])).all()):
                return None
        return cls(lengths)


def scaled_dot_product_attention(q, k, v, mask=None, causal: bool = False, scale: float | None = None):
    """q [B,S,H,D], k/v [B,Sk,Hkv,D].  `mask`: None, a `KeyPaddingMask` (flash kernels, padded keys skipped) or an
    additive tensor broadcastable to [B,H,S,Sk] (reference math in fp32, O(S^2) memory: arbitrary masks are rare and
    are not what the kernels are built for)."""
    if mask is None:
        return ops.flash_attention(q, k, v, causal, scale)
    if isinstance(mask, KeyPaddingMask):
        return ops.flash_attention(q, k, v, causal, scale, kv_lens=mask.lengths)
    B, Sq, H, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    rep = H // kf.shape[1]
    s = qf @ kf.repeat_interleave(rep, 1).transpose(-1, -2) * scale + mask.float()
    return (torch.softmax(s, -1) @ vf.repeat_interleave(rep, 1)).permute(0, 2, 1, 3).to(q.dtype)


class SelfAttention(Module, Trainable, Saveable):
    """Multi-head self-attention.  Parameter names: q_proj / k_proj / v_proj / out_proj (.weight, .bias)."""

    names = ("q_proj", "k_proj", "v_proj", "out_proj")

    def __init__(self, config: SelfAttentionConfig, q: Linear, k: Linear, v: Linear, o: Linear):
        self.config = config
        self._proj = (q, k, v, o)
        self._dropout = Dropout(config.dropout)

    @classmethod
    def new(cls, backend, config: SelfAttentionConfig, seed: int = 42, scale: float = 0.02):
        c = config
        hd = c.head_dim
        mk = lambda i, o, s: LinearBuilder(i, o).with_bias(c.bias).seed(s).scale(scale).zero_bias().build(backend)
        return cls(c, mk(c.d_model, c.num_heads * hd, seed + 11), mk(c.d_model, c.num_kv_heads * hd, seed + 13),
                   mk(c.d_model, c.num_kv_heads * hd, seed + 17), mk(c.num_heads * hd, c.d_model, seed + 19))

    def _children(self):
        for n, p in zip(self.names, self._proj):
            yield n, p

    def qkv(self, x, ctx):
        c = self.config
        B, S, _ = x.shape
        q = self._proj[0](x, ctx).reshape(B, S, c.num_heads, c.head_dim)
        k = self._proj[1](x, ctx).reshape(B, S, c.num_kv_heads, c.head_dim)
        v = self._proj[2](x, ctx).reshape(B, S, c.num_kv_heads, c.head_dim)
        return q, k, v

    def forward(self, x, ctx: ForwardCtx, mask=None, residual=None, pos_offset: int = 0):
        """x: [B, S, d_model] (a rank-2 [S, d_model] input is treated as batch 1)."""
        squeeze = x.dim() == 2
        if squeeze:
            x = x.unsqueeze(0)
            residual = residual.unsqueeze(0) if residual is not None else None
        c = self.config
        B, S, _ = x.shape
        q, k, v = self.qkv(x, ctx)
        if c.rope_theta > 0:
            q = ops.rope(q, S, pos_offset=pos_offset, theta=c.rope_theta)
            k = ops.rope(k, S, pos_offset=pos_offset, theta=c.rope_theta)
        with ctx.profile("attention", q.shape):
            # an additive mask tensor is taken to hold the causal part itself; key-padding lengths only hide keys
            a = scaled_dot_product_attention(q, k, v, mask, c.causal and (mask is None or isinstance(mask, KeyPaddingMask)))
        a = self._dropout(a.reshape(B, S, c.num_heads * c.head_dim), ctx)
        y = self._proj[3](a, ctx, residual)
        return y.squeeze(0) if squeeze else y

    def __call__(self, x, ctx=None, mask=None, residual=None, pos_offset: int = 0):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), mask, residual, pos_offset)


class MultiHeadAttention(Module, Trainable, Saveable):
    """Wrapper whose parameters live under ``attention.`` (crates/nn/src/attention.rs:243-308)."""

    def __init__(self, attention: SelfAttention):
        self.attention = attention

    @classmethod
    def new(cls, backend, d_model: int, num_heads: int, dropout: float = 0.0, seed: int = 42, **kw):
        return cls(SelfAttention.new(backend, SelfAttentionConfig(d_model, num_heads, dropout=dropout, **kw), seed))

    def forward(self, x, ctx: ForwardCtx, mask=None):
        return self.attention.forward(x, ctx, mask)


class TapeMultiHeadAttention(SelfAttention):
    """The trainable attention of the reference's tape stack: wq / wk / wv / wo, each Linear(d, d), additive mask
    (crates/nn/src/tape_transformer.rs:47-143).  Same math as SelfAttention; only the parameter names differ."""
    names = ("wq", "wk", "wv", "wo")

    def forward_tape_with_mask(self, x, mask, ctx: ForwardCtx):
        return self.forward(x, ctx, mask)


@dataclass
class FlashAttentionConfig:
    d_model: int
    num_heads: int
    block_size: int = 128
    causal: bool = False
    dropout: float = 0.0


class FlashAttention(SelfAttention):
    """Tiled O(S)-memory attention with q/k/v/out projections (crates/nn/src/attention.rs:640-903); input layout
    [B, S, d_model].  `block_size` is advisory: the kernel's tile is fixed per head dimension."""

    @classmethod
    def new(cls, backend, config: FlashAttentionConfig, seed: int = 42):
        sc = SelfAttentionConfig(config.d_model, config.num_heads, dropout=config.dropout, causal=config.causal)
        obj = super().new(backend, sc, seed)
        obj.flash_config = config
        return obj


@dataclass
class AttentionMemoryStats:
    """Activation bytes of standard vs flash attention (crates/nn/src/attention.rs:924-960)."""
    standard_bytes: int
    flash_bytes: int
    savings_ratio: float

    @classmethod
    def calculate(cls, batch: int, seq: int, heads: int, head_dim: int, block_size: int = 128, elem_bytes: int = 2):
        qkv = 3 * batch * seq * heads * head_dim * elem_bytes
        standard = qkv + batch * heads * seq * seq * elem_bytes * 2      # scores + probabilities
        flash = qkv + batch * heads * seq * 4 + heads * block_size * block_size * 4
        return cls(standard, flash, standard / max(flash, 1))


class TapeFeedForward(Module, Trainable, Saveable):
    """fc1 -> GELU -> fc2 (crates/nn/src/tape_transformer.rs:161-203); the GELU rides in fc1's GEMM epilogue."""

    def __init__(self, fc1: Linear, fc2: Linear):
        self.fc1, self.fc2 = fc1, fc2

    @classmethod
    def new(cls, backend, d_model: int, ffn_dim: int, seed: int = 42, bias: bool = True, scale: float = 0.02,
            activation: str = "gelu"):
        fc1 = LinearBuilder(d_model, ffn_dim).with_bias(bias).seed(seed + 31).scale(scale).zero_bias()
        if bias:
            fc1 = fc1.activation(activation)
        fc2 = LinearBuilder(ffn_dim, d_model).with_bias(bias).seed(seed + 37).scale(scale).zero_bias()
        obj = cls(fc1.build(backend), fc2.build(backend))
        obj._act = activation
        return obj

    def forward(self, x, ctx: ForwardCtx, residual=None):
        h = self.fc1(x, ctx)
        if self.fc1.activation == "none":
            h = ops.unary(getattr(self, "_act", "gelu"), h) if not h.requires_grad else getattr(ops, getattr(self, "_act", "gelu"))(h)
        return self.fc2(h, ctx, residual)

    def __call__(self, x, ctx=None, residual=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), residual)


class SwiGLUFeedForward(Module, Trainable, Saveable):
    """down( silu(gate(x)) * up(x) ) with gate and up stacked in one [2F, d] weight (Llama-style MLP)."""

    def __init__(self, gate_up: Linear, down: Linear):
        self.gate_up, self.down = gate_up, down

    @classmethod
    def new(cls, backend, d_model: int, ffn_dim: int, seed: int = 42, scale: float = 0.02):
        return cls(LinearBuilder(d_model, 2 * ffn_dim).seed(seed + 31).scale(scale).build(backend),
                   LinearBuilder(ffn_dim, d_model).seed(seed + 37).scale(scale).build(backend))

    def forward(self, x, ctx: ForwardCtx, residual=None):
        return self.down(ops.swiglu(self.gate_up(x, ctx)), ctx, residual)

    def __call__(self, x, ctx=None, residual=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), residual)


@dataclass
class TapeTransformerEncoderConfig:
    d_model: int
    num_heads: int
    ffn_dim: int
    layer_norm_eps: float = 1e-5
    bias: bool = True
    causal: bool = False
    dropout: float = 0.0


class TapeTransformerEncoderLayer(Module, Trainable, Saveable):
    """Pre-LN block: x + Attn(LN1 x); x + FFN(LN2 x).  Names ln1. / attn.{wq,wk,wv,wo}. / ln2. / ffn.{fc1,fc2}.
    (crates/nn/src/tape_transformer.rs:209-274).  Both residual adds happen in GEMM epilogues."""

    def __init__(self, config, ln1, attn, ln2, ffn):
        self.config = config
        self.ln1, self.attn, self.ln2, self.ffn = ln1, attn, ln2, ffn

    @classmethod
    def new(cls, backend, config: TapeTransformerEncoderConfig, seed: int = 42):
        c = config
        sa = SelfAttentionConfig(c.d_model, c.num_heads, dropout=c.dropout, causal=c.causal, bias=c.bias)
        return cls(c, LayerNorm.new(backend, c.d_model, c.layer_norm_eps), TapeMultiHeadAttention.new(backend, sa, seed + 41),
                   LayerNorm.new(backend, c.d_model, c.layer_norm_eps),
                   TapeFeedForward.new(backend, c.d_model, c.ffn_dim, seed + 47, c.bias))

    def forward(self, x, ctx: ForwardCtx, mask=None):
        x = self.attn.forward(self.ln1(x, ctx), ctx, mask, residual=x)
        return self.ffn.forward(self.ln2(x, ctx), ctx, residual=x)

    def forward_tape_with_mask(self, x, mask, ctx):
        return self.forward(x, ctx, mask)

    def __call__(self, x, ctx=None, mask=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), mask)


class TransformerEncoderBlock(Module, Trainable, Saveable):
    """Pre-norm block named self_attn. / norm1. / ff1. / ff2. / norm2. (crates/nn/src/attention.rs:388-431)."""

    def __init__(self, self_attn, norm1, ff1, ff2, norm2):
        self.self_attn, self.norm1, self.ff1, self.ff2, self.norm2 = self_attn, norm1, ff1, ff2, norm2

    @classmethod
    def new(cls, backend, d_model: int, num_heads: int, ff_dim: int, dropout: float = 0.0, seed: int = 42, causal=False):
        sa = SelfAttention.new(backend, SelfAttentionConfig(d_model, num_heads, dropout=dropout, causal=causal), seed)
        ff1 = LinearBuilder(d_model, ff_dim).with_bias().seed(seed + 3).scale(0.02).zero_bias().activation("gelu").build(backend)
        ff2 = LinearBuilder(ff_dim, d_model).with_bias().seed(seed + 5).scale(0.02).zero_bias().build(backend)
        return cls(sa, LayerNorm.new(backend, d_model), ff1, ff2, LayerNorm.new(backend, d_model))

    def forward(self, x, ctx: ForwardCtx, mask=None):
        x = self.self_attn.forward(self.norm1(x, ctx), ctx, mask, residual=x)
        return self.ff2(self.ff1(self.norm2(x, ctx), ctx), ctx, residual=x)

    def __call__(self, x, ctx=None, mask=None):
        return self.forward(x, ctx if ctx is not None else ForwardCtx.inference(), mask)
