"""Token sampling: greedy, temperature, top-k, nucleus (crates/nn/src/continuous_batching.rs:454-490).
The reference's temperature sampler draws with a constant r = 0.5; this one uses a seeded generator."""
from __future__ import annotations

import torch

from .. import ops


class Sampler:
    def __init__(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0):
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self._gen = torch.Generator().manual_seed(seed)

    @classmethod
    def greedy(cls):
        return cls(0.0)

    def sample(self, logits: torch.Tensor) -> torch.Tensor:
        """logits: [batch, vocab] -> int64 [batch] on the logits' device."""
        if self.temperature <= 0.0:
            return ops.argmax_rows(logits)
        x = logits.float().cpu() / self.temperature
        if self.top_k > 0:
            kth = torch.topk(x, min(self.top_k, x.shape[-1]), -1).values[..., -1:]
            x = x.masked_fill(x < kth, float("-inf"))
        p = torch.softmax(x, -1)
        if self.top_p < 1.0:
            sp, si = torch.sort(p, -1, descending=True)
            keep = (torch.cumsum(sp, -1) - sp) < self.top_p
            sp = sp * keep
            p = torch.zeros_like(p).scatter_(-1, si, sp)
            p = p / p.sum(-1, keepdim=True)
        return torch.multinomial(p, 1, generator=self._gen)[:, 0].to(logits.device)
