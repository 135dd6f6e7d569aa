"""The reference's micro-benchmark workloads (crates/bench/src/bin/rustral_workloads.rs:64-75) on this framework.

    python -m rustral_b200.bench.workloads --device cuda --repeats 20 > bench.json

Shapes are the reference's: matmul 128/256/512 cubed, softmax_dim, fused_linear_bias_gelu, attention small / medium,
conv2d, lstm_forward, mlp_train_step, optimizer_step (10M parameters), transformer_encoder.forward, decoder prefill /
decode, kv_cache prefill / decode, model_io save / load.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import Sample, samples_to_json, time_runs
from .. import ops
from ..core import B200Backend, CpuBackend, ForwardCtx
from ..nn import (Conv2d, Conv2dConfig, LinearBuilder, LstmCell, TransformerDecoder, TransformerDecoderConfig,
                  TransformerEncoder, TransformerEncoderConfig)
from ..optim import Adam, Sgd
from ..core import Parameter


def build_workloads(backend, heavy: bool = False) -> list:
    dev, dt = backend.device(), backend.dtype
    ctx = ForwardCtx.inference(backend)
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dev, dt)
    w = []
    for n in (128, 256, 512):
        a, b = rnd(n, n), rnd(n, n)
        w.append((f"matmul.{n}x{n}x{n}", {"m": n, "k": n, "n": n}, lambda a=a, b=b: backend.ops().matmul(a, b)))
    for r, c in ((32, 64), (32, 256), (64, 1024)):
        x = rnd(r, c)
        w.append((f"softmax_dim.{r}x{c}", {"rows": r, "cols": c}, lambda x=x: ops.softmax(x)))
    for b_, i, o in ((32, 256, 1024), (32, 1024, 256)):
        x, wt, bs = rnd(b_, i), rnd(o, i), rnd(o)
        w.append((f"fused_linear_bias_gelu.{b_}x{i}->{o}", {"batch": b_, "in": i, "out": o},
                  lambda x=x, wt=wt, bs=bs: backend.fusion_ops().fused_linear_bias_gelu(x, wt, bs)))
    for name, d, h, s in (("attention.small", 64, 4, 32), ("attention.medium", 256, 8, 128)):
        hd = max(64, d // h) if dev.type == "cuda" else d // h       # the flash kernels take head dims 64 / 128
        q, k, v = rnd(1, s, h, hd), rnd(1, s, h, hd), rnd(1, s, h, hd)
        w.append((name, {"d_model": d, "heads": h, "seq": s, "head_dim": hd}, lambda q=q, k=k, v=v: ops.flash_attention(q, k, v, False)))
    for name, c, hw, o in (("conv2d.small", 1, 28, 8), ("conv2d.medium", 3, 64, 16), ("conv2d.large", 3, 224, 32)):
        conv = Conv2d.new(backend, Conv2dConfig(o, 3, 3, in_channels=c))
        x = rnd(4, c, hw, hw)
        w.append((name, {"channels": c, "hw": hw, "out": o}, lambda conv=conv, x=x: conv(x, ctx)))
    for name, hsz, steps in (("lstm_forward.small", 128, 10), ("lstm_forward.medium", 256, 50), ("lstm_forward.large", 512, 100)):
        cell = LstmCell.new(backend, hsz, hsz)
        xs = rnd(steps, 1, hsz)
        w.append((name, {"hidden": hsz, "steps": steps}, lambda cell=cell, xs=xs: cell.forward_sequence(xs, ctx)))
    l1 = LinearBuilder(128, 256).with_bias().activation("relu").build(backend)
    l2 = LinearBuilder(256, 64).with_bias().build(backend)
    opt = Adam(lr=1e-3)
    x, y = rnd(32, 128), rnd(32, 64)
    tctx = ForwardCtx.train(backend)

    def mlp_step():
        for p in l1.parameters() + l2.parameters():
            p.zero_grad()
        loss = ((l2(l1(x, tctx), tctx).float() - y.float()) ** 2).mean()
        loss.backward()
        opt.step(l1.parameters() + l2.parameters())
    w.append(("mlp_train_step", {"batch": 32, "dims": [128, 256, 64]}, mlp_step))
    n_opt = 100_000_000 if heavy else 10_000_000
    slabs = [Parameter(f"p{i}", torch.zeros(n_opt // 8, dtype=torch.float32, device=dev)) for i in range(8)]
    grads = {p.id: torch.ones_like(p.tensor) for p in slabs}
    sgd, adam = Sgd(lr=0.01), Adam(lr=1e-3)
    w.append(("optimizer_step.sgd", {"params": n_opt}, lambda: sgd.step(slabs, grads)))
    w.append(("optimizer_step.adam", {"params": n_opt}, lambda: adam.step(slabs, grads)))
    enc = TransformerEncoder.new(backend, TransformerEncoderConfig(128, 4, 2, 512, 0.0, 256), 1024)
    ids = torch.randint(0, 1024, (1, 128), generator=g)
    w.append(("transformer_encoder.forward", {"layers": 2, "d_model": 128, "heads": 4, "ffn": 512, "seq": 128, "vocab": 1024},
              lambda: enc.forward(ids.to(dev), ctx)))
    dec = TransformerDecoder.new(backend, TransformerDecoderConfig(128, 4, 2, 512, 0.0, 256), 1024)
    ids64, ids128 = torch.randint(0, 1024, (1, 64), generator=g).to(dev), torch.randint(0, 1024, (1, 128), generator=g).to(dev)
    w.append(("decoder.prefill", {"seq": 64}, lambda: dec.forward(ids64, ctx)))
    w.append(("decoder.decode_step.no_cache", {"seq": 128}, lambda: dec.generate_token(ids128, ctx)))
    from ..serve import CacheConfig, KVCache
    kc = KVCache(CacheConfig(4, 32, 256), dev)
    k64, k1 = rnd(1, 4, 64, 32), rnd(1, 4, 1, 32)

    def kv_prefill():
        kc.reset()
        kc.append(k64, k64)

    def kv_decode():
        if kc.len >= 255:
            kc.reset()
        kc.append(k1, k1)
    w.append(("kv_cache.prefill", {"tokens": 64, "heads": 4, "head_dim": 32}, kv_prefill))
    w.append(("kv_cache.decode_step", {"tokens": 1}, kv_decode))
    from ..io import safetensors_io as st
    big = {f"t{i}": torch.zeros(1_000_000) for i in range(50)}
    blob = [st.serialize(big)]
    w.append(("model_io.save", {"params": 50_000_000}, lambda: blob.__setitem__(0, st.serialize(big))))
    w.append(("model_io.load", {"params": 50_000_000}, lambda: st.deserialize(blob[0])))
    return w


def run(device: str = "cpu", repeats: int = 10, warmup: int = 3, heavy: bool = False, only: str | None = None) -> str:
    backend = CpuBackend() if device == "cpu" else B200Backend()
    samples = []
    for name, params, fn in build_workloads(backend, heavy):
        if only and only not in name:
            continue
        host_only = name.startswith(("model_io", "kv_cache")) and device == "cpu"
        runs = time_runs(fn, warmup, repeats, cuda=(device != "cpu") and not name.startswith("model_io"))
        samples.append(Sample(name, backend.name, str(backend.device()), str(backend.dtype).replace("torch.", ""), None, params, runs))
    return samples_to_json(samples)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--heavy", action="store_true")
    ap.add_argument("--only", default=None)
    a = ap.parse_args()
    print(run(a.device, a.repeats, a.warmup, a.heavy, a.only))
