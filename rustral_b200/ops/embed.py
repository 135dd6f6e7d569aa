"""Token (+ learned position) embedding: gather forward, ordered scatter-add backward."""
from __future__ import annotations

import torch

from .. import _native as N

_scratch: dict = {}


def _int_scratch(device, n: int) -> torch.Tensor:
    key = N.stream_key(device)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=torch.int32, device=device)
        _scratch[key] = buf
    return buf


def embedding_forward(ids: torch.Tensor, wte: torch.Tensor, wpe=None, seq_len: int = 0, out=None) -> torch.Tensor:
    """ids: int64 [tokens]; wte: [vocab, dim]; wpe: [max_pos, dim] added by position ``t % seq_len``."""
    tokens = ids.numel()
    dim = wte.shape[1]
    flat = ids.reshape(-1)
    if not wte.is_cuda:
        y = wte[flat]
        if wpe is not None:
            pos = torch.arange(tokens) % seq_len
            y = (y.float() + wpe[pos].float()).to(wte.dtype)
        if out is not None:
            out.copy_(y)
            y = out
        return y
    if wte.dtype != torch.bfloat16:
        raise TypeError("embedding: CUDA tables must be bf16")
    flat = flat.to(torch.int64)
    y = out if out is not None else torch.empty((tokens, dim), dtype=wte.dtype, device=wte.device)
    if tokens == 0:
        return y
    N.check(N.kernels().rb_embedding_fwd(flat.data_ptr(), wte.data_ptr(), N.ptr(wpe), y.data_ptr(), tokens, dim,
                                         seq_len, wte.shape[0], N.stream_ptr()), "rb_embedding_fwd")
    return y


def embedding_backward(ids, dy2, dwte, dwpe=None, seq_len: int = 0):
    """Accumulates into fp32 ``dwte`` [vocab, dim] (and ``dwpe`` [>=seq_len, dim]); rows are summed in token order."""
    flat = ids.reshape(-1)
    tokens, dim = dy2.shape
    if not dy2.is_cuda:
        if dwte is not None:
            dwte.index_add_(0, flat, dy2.float())
        if dwpe is not None:
            pos = torch.arange(tokens) % seq_len
            dwpe.index_add_(0, pos, dy2.float())
        return
    lib = N.kernels()
    flat = flat.to(torch.int64)
    vocab = dwte.shape[0] if dwte is not None else 1
    scratch = _int_scratch(dy2.device, int(lib.rb_embedding_bwd_scratch_ints(tokens, vocab)))
    N.check(lib.rb_embedding_bwd(flat.data_ptr(), dy2.data_ptr(), N.ptr(dwte), N.ptr(dwpe), scratch.data_ptr(), tokens,
                                 dim, seq_len, vocab, N.stream_ptr()), "rb_embedding_bwd")


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte):
        ctx.save_for_backward(ids)
        ctx.wshape = wte.shape
        ctx.wdtype = wte.dtype
        return embedding_forward(ids, wte).reshape(*ids.shape, wte.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        dw = torch.zeros(ctx.wshape, dtype=torch.float32, device=dy.device)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        embedding_backward(ids, dy2, dw)
        return None, dw.to(ctx.wdtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather ``table[ids]`` with a deterministic gradient (crates/nn/src/embedding.rs:71-79)."""
    if not N.wants_grad(table):
        return embedding_forward(ids, table).reshape(*ids.shape, table.shape[1])
    return _EmbeddingFn.apply(ids, table)
