"""Embedding table with row-gather forward (crates/nn/src/embedding.rs:11-79)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, Trainable, InvalidArgument


@dataclass
class EmbeddingConfig:
    vocab_size: int
    dim: int


class Embedding(Module, Trainable, Saveable):
    """Parameter name: ``embed`` [vocab, dim], initialised N(0, 0.02)."""

    def __init__(self, config: EmbeddingConfig, table: Parameter, vocab=None):
        self.config = config
        self.embed = table
        self._vocab = vocab

    @classmethod
    def new(cls, backend, vocab_size: int, dim: int, seed: int = 7, scale: float = 0.02, vocab=None):
        return cls(EmbeddingConfig(vocab_size, dim), backend.normal_parameter("embed", (vocab_size, dim), seed, scale), vocab)

    def forward(self, ids, ctx: ForwardCtx):
        ids = ids if torch.is_tensor(ids) else torch.as_tensor(ids, dtype=torch.int64)
        if not ids.is_cuda:
            # checked on the host while the ids are there; ids that already live on the GPU are not read back (that would
            # stall the stream on every call): the kernel skips an out-of-range id and the index-checking build reports it
            if ids.numel() and (int(ids.max()) >= self.config.vocab_size or int(ids.min()) < 0):
                raise InvalidArgument("Embedding: token id out of range")
        ids = ids.to(device=self.embed.tensor.device, dtype=torch.int64)
        with ctx.profile("embedding", ids.shape):
            return ops.embedding(ids, self.embed.tensor)

    def lookup(self, token: str, ctx=None):
        """Embedding of a symbol through the attached vocabulary."""
        if self._vocab is None:
            raise InvalidArgument("Embedding has no vocabulary attached")
        return self([self._vocab.id_or_unk(token)], ctx)

    def _children(self):
        yield "embed", self.embed
