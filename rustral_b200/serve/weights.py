"""Inference weights: bf16 only, optionally sharded for tensor parallelism, under the parameter names the model
runner uses.  Column-parallel matrices (QKV, gate/up, LM head) keep `1 / world` of their rows, row-parallel ones
(attention output, down projection) `1 / world` of their columns; norms and the embedding are replicated."""
from __future__ import annotations

import math
import zlib

import torch

from ..models.config import GPTConfig


class InferenceWeights:
    def __init__(self, tensors: dict, dtype):
        self.tensors = tensors
        self.lowp = next(iter(tensors.values())).new_empty(0, dtype=dtype)   # dtype / device carrier

    def w(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())

    def load_state_dict(self, state: dict, cfg: GPTConfig) -> None:
        """Strict load of an UNSHARDED Llama-style checkpoint in the trainer's format (`FlatParams.state_dict`: fp32,
        vocabulary unpadded, attention projections under attn.wq / wk / wv): every expected key present, no extra
        key, shapes equal; nothing is written before all checks pass.  Tensor-parallel ranks load the full set and
        cut their shard with `shard_of`."""
        from ..core.errors import SerializationError, ShapeMismatch
        plan = {}                                         # checkpoint key -> (destination tensor, row slice)
        hd = cfg.head_dim
        q_end, k_end = cfg.n_head * hd, (cfg.n_head + cfg.n_kv_head) * hd
        for name, t in self.tensors.items():
            if ".attn.wqkv." in name:
                for nm, sl in (("wq", slice(0, q_end)), ("wk", slice(q_end, k_end)), ("wv", slice(k_end, t.shape[0]))):
                    plan[name.replace("wqkv", nm)] = (t, sl)
            elif name in ("tok_embed.embed", "head.weight"):
                plan[name] = (t, slice(0, cfg.vocab_size))
            else:
                plan[name] = (t, slice(0, t.shape[0]))
        missing = [k for k in plan if k not in state]
        extra = [k for k in state if k not in plan]
        if missing:
            raise SerializationError(f"missing keys: {missing}")
        if extra:
            raise SerializationError(f"unexpected keys: {extra}")
        for k, (t, sl) in plan.items():
            want = (sl.stop - sl.start, *t.shape[1:])
            if tuple(state[k].shape) != want:
                raise ShapeMismatch(want, state[k].shape, k)
        with torch.no_grad():
            for k, (t, sl) in plan.items():
                t[sl].copy_(state[k].to(t.device, t.dtype))

    # ------------------------------------------------------------------------------------------------ constructors
    @classmethod
    def random_llama(cls, cfg: GPTConfig, device, rank: int = 0, world: int = 1, seed: int = 0) -> "InferenceWeights":
        """Random-init Llama-style shard generated on the device (a full 8B model never exists on one GPU)."""
        if cfg.arch != "llama":
            raise ValueError("random_llama: llama-style configs only")
        dev = torch.device(device)
        dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
        d, hd = cfg.d_model, cfg.head_dim
        hq, hk, f, v = cfg.n_head // world, cfg.n_kv_head // world, cfg.ffn_dim // world, cfg.vocab_padded // world

        def rnd(shape, name, shard, std):
            g = torch.Generator(device=dev).manual_seed((zlib.crc32(f"{seed}/{name}".encode()) & 0x7FFFFFFF) * 64 + shard)
            return torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=g).to(dt)

        t = {"tok_embed.embed": rnd((cfg.vocab_padded, d), "tok_embed", 0, cfg.init_std),
             "final_norm.weight": torch.ones(d, dtype=dt, device=dev),
             "head.weight": rnd((v, d), "head", rank, cfg.init_std)}
        s2 = cfg.init_std / math.sqrt(2 * cfg.n_layer)
        for l in range(cfg.n_layer):
            p = f"layers.{l}."
            t[p + "ln1.weight"] = torch.ones(d, dtype=dt, device=dev)
            t[p + "ln2.weight"] = torch.ones(d, dtype=dt, device=dev)
            t[p + "attn.wqkv.weight"] = rnd(((hq + 2 * hk) * hd, d), p + "wqkv", rank, cfg.init_std)
            t[p + "attn.wo.weight"] = rnd((d, hq * hd), p + "wo", rank, s2)
            t[p + "ffn.gate_up.weight"] = rnd((2 * f, d), p + "gate_up", rank, cfg.init_std)
            t[p + "ffn.down.weight"] = rnd((d, f), p + "down", rank, s2)
        return cls(t, dt)

    @classmethod
    def shard_of(cls, full, cfg: GPTConfig, rank: int, world: int) -> "InferenceWeights":
        """This rank's shard of a full Llama-style parameter set (`full.w(name)` gives the unsharded tensors)."""
        d, hd = cfg.d_model, cfg.head_dim
        H, Hk, F = cfg.n_head, cfg.n_kv_head, cfg.ffn_dim
        hq, hk, f, v = H // world, Hk // world, F // world, cfg.vocab_padded // world
        t = {"tok_embed.embed": full.w("tok_embed.embed"), "final_norm.weight": full.w("final_norm.weight"),
             "head.weight": full.w("head.weight")[rank * v:(rank + 1) * v].contiguous()}
        for l in range(cfg.n_layer):
            p = f"layers.{l}."
            t[p + "ln1.weight"], t[p + "ln2.weight"] = full.w(p + "ln1.weight"), full.w(p + "ln2.weight")
            wqkv = full.w(p + "attn.wqkv.weight")
            q = wqkv[:H * hd][rank * hq * hd:(rank + 1) * hq * hd]
            k = wqkv[H * hd:(H + Hk) * hd][rank * hk * hd:(rank + 1) * hk * hd]
            vv = wqkv[(H + Hk) * hd:][rank * hk * hd:(rank + 1) * hk * hd]
            t[p + "attn.wqkv.weight"] = torch.cat([q, k, vv], 0).contiguous()
            t[p + "attn.wo.weight"] = full.w(p + "attn.wo.weight")[:, rank * hq * hd:(rank + 1) * hq * hd].contiguous()
            gu = full.w(p + "ffn.gate_up.weight")
            t[p + "ffn.gate_up.weight"] = torch.cat([gu[:F][rank * f:(rank + 1) * f], gu[F:][rank * f:(rank + 1) * f]], 0).contiguous()
            t[p + "ffn.down.weight"] = full.w(p + "ffn.down.weight")[:, rank * f:(rank + 1) * f].contiguous()
        return cls(t, full.lowp.dtype)
