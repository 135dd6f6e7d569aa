"""Inference-side model execution for the decoder families: prefill of a prompt and batched single-token decode
against a paged KV cache.  Every matmul is the tcgen05 GEMM, prompt attention is the flash kernel, decode attention
the paged kernel; K and V of new tokens go straight from the packed QKV projection into their cache slots.

This is the model forward the reference's ServingEngine lacks (it fabricates token 1, crates/nn/src/continuous_batching.rs:516-526)
and the cached decode its TransformerDecoder::generate_token does not have (full re-forward per token, crates/nn/src/transformer.rs:837-862).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..models.config import GPTConfig
from ..ops import attention as attn_ops
from ..ops import norm as norm_ops
from ..ops import paged as paged_ops
from ..ops import rotary as rope_ops
from ..ops.matmul import gemm
from ..runtime.fused_gpt import FlatParams
from .kv_cache import PagedCache


class ModelRunner:
    def __init__(self, cfg: GPTConfig, params: FlatParams | None = None, device=None, num_blocks: int = 1024,
                 block_size: int = 16, seed: int = 0):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.cfg = cfg
        self.device = torch.device(device)
        self.params = params if params is not None else FlatParams(cfg, self.device, seed)
        self.dtype = self.params.lowp.dtype
        self.cache = PagedCache(num_blocks, block_size, cfg.n_layer, cfg.n_kv_head, cfg.head_dim, self.dtype, self.device)
        self.block_size = block_size

    # ---- shared layer body ------------------------------------------------------------------------------------
    def _norm(self, x, name):
        P, rms = self.params, self.cfg.arch == "llama"
        y, _, _ = norm_ops.norm_forward(x, P.w(name + ".weight"), None if rms else P.w(name + ".bias"), self.cfg.norm_eps, rms)
        return y

    def _mlp(self, x1, p):
        P, cfg = self.params, self.cfg
        h = self._norm(x1, p + "ln2")
        if cfg.arch == "llama":
            gu = gemm(h, P.w(p + "ffn.gate_up.weight"))
            return gemm(rope_ops.swiglu_forward(gu), P.w(p + "ffn.down.weight"), residual=x1)
        h = gemm(h, P.w(p + "ffn.fc1.weight"), bias=P.w(p + "ffn.fc1.bias"), act="gelu")
        return gemm(h, P.w(p + "ffn.fc2.weight"), bias=P.w(p + "ffn.fc2.bias"), residual=x1)

    def _head(self, x):
        P, cfg = self.params, self.cfg
        xf = self._norm(x, "final_norm")
        return gemm(xf, P.w("tok_embed.embed" if cfg.tie_embeddings else "head.weight"))

    def _embed(self, ids, positions):
        P, cfg = self.params, self.cfg
        x = ops.embedding_forward(ids, P.w("tok_embed.embed"))
        if cfg.arch == "gpt2":
            x = ops.binary("add", x, ops.gather_rows(P.w("pos_embed.embed"), positions))
        return x

    # ---- prefill -------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, seq_id: int, tokens: list) -> torch.Tensor:
        """Runs the whole prompt, fills the cache slots of `seq_id` (which must have blocks reserved) and returns the
        logits of the last position, [vocab_padded]."""
        cfg, P = self.cfg, self.params
        L = len(tokens)
        H, Hk, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        rms = cfg.arch == "llama"
        ids = torch.tensor(tokens, dtype=torch.int64, device=self.device)
        pos = torch.arange(L, dtype=torch.int64, device=self.device)
        table = self.cache.block_table(seq_id)
        bt = torch.tensor(table, dtype=torch.int64, device=self.device)
        slots = bt[pos // self.block_size] * self.block_size + pos % self.block_size
        x = self._embed(ids, pos)
        scale = 1.0 / math.sqrt(D)
        for l in range(cfg.n_layer):
            p = f"layers.{l}."
            h = self._norm(x, p + "ln1")
            qkv = gemm(h, P.w(p + "attn.wqkv.weight"), bias=None if rms else P.w(p + "attn.wqkv.bias"))
            if rms:
                rope_ops.rope_(qkv, H + Hk, D, L, theta=cfg.rope_theta)
            k2, v2 = qkv[:, H * D:(H + Hk) * D], qkv[:, (H + Hk) * D:]
            paged_ops.kv_append(k2, v2, self.cache.k[l], self.cache.v[l], slots)
            q = qkv[:, :H * D].view(1, L, H, D)
            if self.device.type == "cuda":
                a, _ = attn_ops.attention_forward(q, k2.view(1, L, Hk, D), v2.view(1, L, Hk, D), True, scale, want_lse=False)
            else:
                a = attn_ops.attention_reference(q, k2.view(1, L, Hk, D), v2.view(1, L, Hk, D), True, scale)
            x = gemm(a.reshape(L, H * D), P.w(p + "attn.wo.weight"), bias=None if rms else P.w(p + "attn.wo.bias"), residual=x)
            x = self._mlp(x, p)
        return self._head(x[L - 1:L].contiguous())[0]

    # ---- decode ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def decode(self, seq_ids: list, last_tokens: list, context_lens: list) -> torch.Tensor:
        """One new token per sequence.  context_lens[i] counts the tokens in the cache AFTER this token is appended.
        Returns logits [batch, vocab_padded]."""
        cfg, P = self.cfg, self.params
        B = len(seq_ids)
        H, Hk, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        rms = cfg.arch == "llama"
        dev = self.device
        ids = torch.tensor(last_tokens, dtype=torch.int64, device=dev)
        ctx = torch.tensor(context_lens, dtype=torch.int32, device=dev)
        pos = (ctx - 1).to(torch.int64)
        tables = [self.cache.block_table(s) for s in seq_ids]
        max_blocks = max(len(t) for t in tables)
        bt_host = torch.zeros((B, max_blocks), dtype=torch.int32)
        for i, t in enumerate(tables):
            bt_host[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
        bt = bt_host.to(dev)
        slots = bt.gather(1, (pos // self.block_size).view(B, 1)).view(B).to(torch.int64) * self.block_size + pos % self.block_size
        x = self._embed(ids, pos)
        scale = 1.0 / math.sqrt(D)
        for l in range(cfg.n_layer):
            p = f"layers.{l}."
            h = self._norm(x, p + "ln1")
            qkv = gemm(h, P.w(p + "attn.wqkv.weight"), bias=None if rms else P.w(p + "attn.wqkv.bias"))
            if rms:
                rope_ops.rope_(qkv, H + Hk, D, positions=pos, theta=cfg.rope_theta)
            paged_ops.kv_append(qkv[:, H * D:(H + Hk) * D], qkv[:, (H + Hk) * D:], self.cache.k[l], self.cache.v[l], slots)
            a = paged_ops.paged_attention_decode(qkv[:, :H * D], self.cache.k[l], self.cache.v[l], bt, ctx, scale)
            x = gemm(a, P.w(p + "attn.wo.weight"), bias=None if rms else P.w(p + "attn.wo.bias"), residual=x)
            x = self._mlp(x, p)
        return self._head(x)
