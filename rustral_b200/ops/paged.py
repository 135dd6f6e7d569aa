"""Paged KV-cache ops: append and decode attention through a block table."""
from __future__ import annotations

import math

import torch

from .. import _native as N

N.optional_sig("rb_kv_append", [N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_void_p, N.c_void_p, N.c_void_p, N.c_ll, N.c_int,
                                N.c_int, N.c_ll, N.c_void_p])
N.optional_sig("rb_paged_attention_decode", [N.c_void_p, N.c_ll, N.c_void_p, N.c_ll, N.c_void_p, N.c_void_p, N.c_void_p,
                                             N.c_int, N.c_void_p, N.c_int, N.c_int, N.c_int, N.c_int, N.c_int, N.c_ll,
                                             N.c_float, N.c_void_p, N.c_void_p])
N.optional_sig("rb_paged_attention_scratch_floats", [N.c_int, N.c_int, N.c_int, N.c_int, N.c_int], N.c_ll)
N._LAUNCHES["rb_paged_attention_decode"] = 2


def kv_append(k_new, v_new, k_cache, v_cache, slot_mapping):
    """k_new / v_new: [tokens, kv_heads * head_dim] (row-strided views allowed); caches: [blocks, block_size, kv_heads, D];
    slot_mapping: int64 [tokens] = block * block_size + offset (negative = skip)."""
    tokens = k_new.shape[0]
    nb, bs, hk, d = k_cache.shape
    if not k_new.is_cuda:
        kc, vc = k_cache.view(nb * bs, hk * d), v_cache.view(nb * bs, hk * d)
        ok = slot_mapping >= 0
        kc[slot_mapping[ok]] = k_new[ok].to(kc.dtype)
        vc[slot_mapping[ok]] = v_new[ok].to(vc.dtype)
        return
    N.check(N.kernels().rb_kv_append(k_new.data_ptr(), k_new.stride(0), v_new.data_ptr(), v_new.stride(0), k_cache.data_ptr(),
                                     v_cache.data_ptr(), slot_mapping.data_ptr(), tokens, hk, d, nb * bs, N.stream_ptr()),
            "rb_kv_append")


def paged_attention_decode(q, k_cache, v_cache, block_tables, context_lens, scale=None, out=None):
    """q: [batch, heads * head_dim] (or [batch, heads, head_dim]); block_tables int32 [batch, max_blocks];
    context_lens int32 [batch].  Returns [batch, heads * head_dim]."""
    nb, bs, hk, d = k_cache.shape
    B = q.shape[0]
    q2 = q.reshape(B, -1)
    heads = q2.shape[1] // d
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if not q.is_cuda:
        o = torch.zeros(B, heads, d)
        kc, vc = k_cache.view(nb * bs, hk, d).float(), v_cache.view(nb * bs, hk, d).float()
        for b in range(B):
            n = int(context_lens[b])
            toks = torch.arange(n)
            slots = block_tables[b, toks // bs].long() * bs + toks % bs
            kk = kc[slots].repeat_interleave(heads // hk, 1)          # [n, heads, d]
            vv = vc[slots].repeat_interleave(heads // hk, 1)
            s = torch.einsum("hd,nhd->hn", q2[b].float().view(heads, d), kk) * scale
            o[b] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv)
        r = o.reshape(B, heads * d).to(q.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    out = out if out is not None else torch.empty((B, heads * d), dtype=q.dtype, device=q.device)
    lib = N.kernels()
    scratch = torch.empty(lib.rb_paged_attention_scratch_floats(B, heads, d, block_tables.shape[1], bs), dtype=torch.float32,
                          device=q.device)
    N.check(lib.rb_paged_attention_decode(q2.data_ptr(), q2.stride(0), out.data_ptr(), out.stride(0),
                                          k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                                          block_tables.shape[1], context_lens.data_ptr(), B, heads, hk, d, bs, nb,
                                          scale, scratch.data_ptr(), N.stream_ptr()), "rb_paged_attention_decode")
    return out
