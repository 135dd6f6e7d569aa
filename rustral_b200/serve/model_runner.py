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
    """`tp` (a parallel.tp_inference.TPInferenceComm) makes this rank one shard of a tensor-parallel model: `params`
    then holds this rank's shard (serve.weights.InferenceWeights), the cache holds this rank's KV heads, and the
    attention-output, down-projection and LM-head results are exchanged with one-shot peer-memory collectives.  All
    ranks run the same calls in the same order and obtain bit-identical logits."""

    def __init__(self, cfg: GPTConfig, params=None, device=None, num_blocks: int = 1024,
                 block_size: int = 16, seed: int = 0, tp=None):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.cfg = cfg
        self.device = torch.device(device)
        self.tp = tp
        self.tp_world = tp.world if tp is not None else 1
        if tp is not None:
            if cfg.arch != "llama" or cfg.n_head % tp.world or cfg.n_kv_head % tp.world or cfg.ffn_dim % tp.world or \
                    cfg.vocab_padded % (8 * tp.world):
                raise ValueError("tensor-parallel serving: llama-style model whose heads, FFN and vocabulary divide evenly")
            if params is None:
                from .weights import InferenceWeights
                params = InferenceWeights.random_llama(cfg, self.device, tp.rank, tp.world, seed)
        self.params = params if params is not None else FlatParams(cfg, self.device, seed)
        self.dtype = self.params.lowp.dtype
        self.n_head, self.n_kv_head = cfg.n_head // self.tp_world, cfg.n_kv_head // self.tp_world
        self.cache = PagedCache(num_blocks, block_size, cfg.n_layer, self.n_kv_head, cfg.head_dim, self.dtype, self.device)
        self.block_size = block_size
        self.use_graphs = True          # CUDA-graph replay of decode steps
        self._graphs: dict = {}

    def _row_parallel(self, a, w, bias, residual):
        """a @ w^T (+ bias) + residual; with tensor parallelism the partial products are summed over the ranks."""
        if self.tp is None:
            return gemm(a, w, bias=bias, residual=residual)
        rows = a.shape[0]
        gemm(a, w, out=self.tp.staging(rows, w.shape[0]))
        return self.tp.all_reduce(rows, w.shape[0], residual=residual)

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
            return self._row_parallel(rope_ops.swiglu_forward(gu), P.w(p + "ffn.down.weight"), None, x1)
        h = gemm(h, P.w(p + "ffn.fc1.weight"), bias=P.w(p + "ffn.fc1.bias"), act="gelu")
        return gemm(h, P.w(p + "ffn.fc2.weight"), bias=P.w(p + "ffn.fc2.bias"), residual=x1)

    def _head(self, x):
        P, cfg = self.params, self.cfg
        xf = self._norm(x, "final_norm")
        if self.tp is not None:
            w = P.w("head.weight")
            gemm(xf, w, out=self.tp.staging(xf.shape[0], w.shape[0]))
            return self.tp.all_gather_cols(xf.shape[0], w.shape[0])
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
        H, Hk, D = self.n_head, self.n_kv_head, cfg.head_dim
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
            x = self._row_parallel(a.reshape(L, H * D), P.w(p + "attn.wo.weight"), None if rms else P.w(p + "attn.wo.bias"), x)
            x = self._mlp(x, p)
        logits = self._head(x[L - 1:L].contiguous())[0]
        if self.tp is not None:
            self.tp.end_step()
        return logits

    # ---- mixed step: prompt chunks and decode tokens through the same GEMMs ---------------------------------------------
    @torch.no_grad()
    def step_mixed(self, chunks: list, dec_ids: list, dec_tok: list, dec_len: list):
        """One model pass over several prompt chunks and the decode batch.

        `chunks`: list of (seq_id, tokens, start, want_logits): `tokens` are positions [start, start + len) of the
        sequence's prefix; everything before `start` is already in the cache.  `dec_*`: as for `decode`.  All rows go
        through the projections, the MLP and the collectives together (the weights are read once per step); attention
        runs per part: the flash kernel for a chunk (its keys are the sequence's cached prefix, gathered from the pages,
        plus the chunk itself; causal mask aligned to the end), the paged kernel for the decode rows.
        Returns (list of logits [vocab_padded] or None per chunk, decode logits [len(dec_ids), vocab_padded] or None).
        (Batched and chunked prefill of the reference's scheduler: crates/nn/src/continuous_batching.rs:248-295.)"""
        cfg, P, dev, bs = self.cfg, self.params, self.device, self.block_size
        H, Hk, D = self.n_head, self.n_kv_head, cfg.head_dim
        rms = cfg.arch == "llama"
        nd = len(dec_ids)
        ids_h, pos_h, slot_h, spans, ctx_slots = [], [], [], [], []
        for seq_id, tokens, start, _ in chunks:
            table = self.cache.block_table(seq_id)
            L = len(tokens)
            r0 = len(ids_h)
            ids_h += list(tokens)
            pos_h += list(range(start, start + L))
            slot_h += [table[p_ // bs] * bs + p_ % bs for p_ in range(start, start + L)]
            spans.append((r0, r0 + L))
            # cache slots of the whole visible prefix (earlier chunks and this one)
            ctx_slots.append(None if start == 0 else
                             torch.tensor([table[p_ // bs] * bs + p_ % bs for p_ in range(start + L)], dtype=torch.int64, device=dev))
        rd = len(ids_h)
        for seq_id, tok, n in zip(dec_ids, dec_tok, dec_len):
            table = self.cache.block_table(seq_id)
            ids_h.append(tok)
            pos_h.append(n - 1)
            slot_h.append(table[(n - 1) // bs] * bs + (n - 1) % bs)
        T = len(ids_h)
        ids = torch.tensor(ids_h, dtype=torch.int64, device=dev)
        pos = torch.tensor(pos_h, dtype=torch.int64, device=dev)
        slots = torch.tensor(slot_h, dtype=torch.int64, device=dev)
        if nd:
            width = max(len(self.cache.block_table(s_)) for s_ in dec_ids)
            bt = self._fill_tables(dec_ids, width).to(dev)
            ctx = torch.tensor(dec_len, dtype=torch.int32, device=dev)
        x = self._embed(ids, pos)
        scale = 1.0 / math.sqrt(D)
        nb = self.cache.k[0].shape[0]
        for l in range(cfg.n_layer):
            p = f"layers.{l}."
            h = self._norm(x, p + "ln1")
            qkv = gemm(h, P.w(p + "attn.wqkv.weight"), bias=None if rms else P.w(p + "attn.wqkv.bias"))
            if rms:
                rope_ops.rope_(qkv, H + Hk, D, positions=pos, theta=cfg.rope_theta)
            k2, v2 = qkv[:, H * D:(H + Hk) * D], qkv[:, (H + Hk) * D:]
            paged_ops.kv_append(k2, v2, self.cache.k[l], self.cache.v[l], slots)
            a = torch.empty((T, H * D), dtype=qkv.dtype, device=dev)
            for (r0, r1), cs in zip(spans, ctx_slots):
                L = r1 - r0
                q = qkv[r0:r1, :H * D].view(1, L, H, D)
                if cs is None:
                    kk, vv = k2[r0:r1].view(1, L, Hk, D), v2[r0:r1].view(1, L, Hk, D)
                else:
                    kk = ops.gather_rows(self.cache.k[l].view(nb * bs, Hk * D), cs).view(1, -1, Hk, D)
                    vv = ops.gather_rows(self.cache.v[l].view(nb * bs, Hk * D), cs).view(1, -1, Hk, D)
                if dev.type == "cuda":
                    attn_ops.attention_forward(q, kk, vv, True, scale, out=a[r0:r1].view(1, L, H, D), want_lse=False)
                else:
                    a[r0:r1] = attn_ops.attention_reference(q, kk, vv, True, scale).reshape(L, H * D)
            if nd:
                paged_ops.paged_attention_decode(qkv[rd:, :H * D], self.cache.k[l], self.cache.v[l], bt, ctx, scale, out=a[rd:])
            x = self._row_parallel(a, P.w(p + "attn.wo.weight"), None if rms else P.w(p + "attn.wo.bias"), x)
            x = self._mlp(x, p)
        # logits only where a token is sampled: the last row of every chunk that completes its prompt, and the decode rows
        want = [r1 - 1 for (r0, r1), c in zip(spans, chunks) if c[3]]
        rows = want + list(range(rd, T))
        chunk_logits, dec_logits = [None] * len(chunks), None
        if rows:
            sel = x if rows == list(range(T)) else x.index_select(0, torch.tensor(rows, dtype=torch.int64, device=dev))
            logits = self._head(sel.contiguous())
            it = iter(range(len(want)))
            for i, c in enumerate(chunks):
                if c[3]:
                    chunk_logits[i] = logits[next(it)]
            if nd:
                dec_logits = logits[len(want):]
        if self.tp is not None:
            self.tp.end_step()
        return chunk_logits, dec_logits

    # ---- decode ------------------------------------------------------------------------------------------------------
    def _decode_body(self, ids, ctx, bt):
        """The device-side part of a decode step on static tensors (captured into a CUDA graph per batch size)."""
        cfg, P = self.cfg, self.params
        B = ids.shape[0]
        H, Hk, D = self.n_head, self.n_kv_head, cfg.head_dim
        rms = cfg.arch == "llama"
        pos = (ctx - 1).to(torch.int64)
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
            x = self._row_parallel(a, P.w(p + "attn.wo.weight"), None if rms else P.w(p + "attn.wo.bias"), x)
            x = self._mlp(x, p)
        logits = self._head(x)
        if self.tp is not None:
            self.tp.end_step()
        return logits

    def _fill_tables(self, seq_ids, width: int) -> torch.Tensor:
        tables = [self.cache.block_table(s) for s in seq_ids]
        bt_host = torch.zeros((len(seq_ids), width), dtype=torch.int32)
        for i, t in enumerate(tables):
            bt_host[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
        return bt_host

    @torch.no_grad()
    def decode(self, seq_ids: list, last_tokens: list, context_lens: list) -> torch.Tensor:
        """One new token per sequence.  context_lens[i] counts the tokens in the cache AFTER this token is appended.
        Returns logits [batch, vocab_padded] (with CUDA graphs: valid until the next decode call)."""
        B = len(seq_ids)
        dev = self.device
        if self.use_graphs and dev.type == "cuda":
            return self._decode_graphed(seq_ids, last_tokens, context_lens)
        ids = torch.tensor(last_tokens, dtype=torch.int64, device=dev)
        ctx = torch.tensor(context_lens, dtype=torch.int32, device=dev)
        max_blocks = max(len(self.cache.block_table(s)) for s in seq_ids)
        bt = self._fill_tables(seq_ids, max_blocks).to(dev)
        return self._decode_body(ids, ctx, bt)

    def _decode_graphed(self, seq_ids, last_tokens, context_lens) -> torch.Tensor:
        """Replays one captured CUDA graph per batch size: the ~10 launches per layer of a decode step are
        launch-bound from Python, the graph submits them in one call.  Inputs live in static device tensors that
        are refreshed (three small copies) before each replay."""
        B = len(seq_ids)
        dev = self.device
        width = (self.cfg.seq_len + self.block_size - 1) // self.block_size
        g = self._graphs.get(B)
        if g is None:
            ids = torch.zeros(B, dtype=torch.int64, device=dev)
            ctx = torch.ones(B, dtype=torch.int32, device=dev)
            bt = torch.zeros((B, width), dtype=torch.int32, device=dev)
            g = {"ids": ids, "ctx": ctx, "bt": bt, "graph": None, "out": None}
            self._graphs[B] = g
        g["ids"].copy_(torch.tensor(last_tokens, dtype=torch.int64), non_blocking=True)
        g["ctx"].copy_(torch.tensor(context_lens, dtype=torch.int32), non_blocking=True)
        g["bt"].copy_(self._fill_tables(seq_ids, width), non_blocking=True)
        if g["graph"] is None:
            # first use of this batch size: one eager run (lazy kernel configuration, tensor-map cache), then capture
            out = self._decode_body(g["ids"], g["ctx"], g["bt"])
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g["out"] = self._decode_body(g["ids"], g["ctx"], g["bt"])
            g["graph"] = graph
            return out
        g["graph"].replay()
        return g["out"]
