"""Micro-benchmarks of single kernels with roofline fractions.

    python -m rustral_b200.bench.kernels gemm --m 32768 --n 2304 --k 768 [--act gelu] [--iters 10]
    python -m rustral_b200.bench.kernels gemm-fp8 --m 8192 --n 8192 --k 8192
    python -m rustral_b200.bench.kernels attention --batch 32 --seq 1024 --heads 12 --head-dim 64 [--impl tc2|tc|mma] [--backward]
    python -m rustral_b200.bench.kernels norm --rows 32768 --n 768
    python -m rustral_b200.bench.kernels adam --numel 124000000
    python -m rustral_b200.bench.kernels launch-overhead [--calls 5000]

Timing: CUDA events around each call on the current stream, `--warmup` untimed calls first, a 256 MiB buffer is
overwritten between timed calls so every call starts with a cold L2; the median is reported.  Fractions are
against the copy bandwidth and cuBLAS bf16 throughput measured on the same GPU type (`MEASURED_PEAKS.json` at the
repository root when present, else 6650 GB/s and 1590 TFLOP/s).  One JSON line per run.

`launch-overhead` measures the host side instead: small operations (a 128^3 product, softmax and LayerNorm of 32 x 256,
an elementwise add) are issued `--calls` times back to back and the wall time per call is reported (the GPU work is a few
microseconds, so the issue rate is the host's), next to the same call bracketed by two CUDA events, which is how the
workload table times one call, and next to `torch.add` / `torch.mm` on the same tensors as the yardstick of what a
native-extension launch costs on this machine.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def peaks() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timed(fn, warmup: int, iters: int) -> float:
    """Median milliseconds per call, cold L2."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def report(name: str, ms: float, flops: float, nbytes: float, extra: dict) -> dict:
    pk = peaks()
    out = {"kernel": name, "us": round(ms * 1e3, 2), **extra}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_bf16_peak"] = round(out["tflops"] / pk["bf16_tflops"], 3)
    if nbytes:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out["frac_of_hbm_peak"] = round(out["gbs"] / pk["hbm_gbs"], 3)
    out["peaks"] = pk["source"]
    print(json.dumps(out))
    return out


def bench_gemm(a):
    from ..ops.matmul import gemm
    dev = "cuda"
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16()
    out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
    pre = torch.empty_like(out) if a.act != "none" else None
    bias = torch.zeros(a.n, dtype=torch.bfloat16, device=dev) if a.bias or a.act != "none" else None
    fn = lambda: gemm(x, w, out=out, act=a.act, aux_out=pre, bias=bias, block_n=a.block_n)
    ms = timed(fn, a.warmup, a.iters)
    nbytes = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n * (2 if pre is not None else 1))
    return report("gemm_bf16_tcgen05", ms, 2.0 * a.m * a.n * a.k, nbytes,
                  {"m": a.m, "n": a.n, "k": a.k, "act": a.act})


def bench_gemm_fp8(a):
    """e4m3 x e4m3 product with per-row and per-column scales and a bf16 output, against the bf16 kernel on the same shape."""
    from ..ops import quant as Q
    from ..ops.matmul import gemm
    dev = "cuda"
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16()
    a8, sa = Q.quantize_fp8_rows(x)
    b8, sb = Q.quantize_fp8_rows(w)
    out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: Q.gemm_fp8(a8, sa, b8, sb, out=out, block_n=a.block_n), a.warmup, a.iters)
    ms16 = timed(lambda: gemm(x, w, out=out), a.warmup, a.iters)
    msq = timed(lambda: Q.quantize_fp8_rows(x, out=a8, scales=sa), a.warmup, a.iters)
    flops = 2.0 * a.m * a.n * a.k
    return report("gemm_e4m3_tcgen05", ms, flops, 0,
                  {"m": a.m, "n": a.n, "k": a.k, "bf16_us": round(ms16 * 1e3, 2), "bf16_tflops": round(flops / ms16 / 1e9, 1),
                   "speedup_over_bf16": round(ms16 / ms, 3), "quantize_rows_us": round(msq * 1e3, 2),
                   "quantize_gbs": round(3.0 * a.m * a.k / msq / 1e6, 1)})


def bench_attention(a):
    from ..ops import attention as A
    B, S, H, D = a.batch, a.seq, a.heads, a.head_dim
    hk = a.kv_heads or H
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    q, k, v = mk(B, S, H, D), mk(B, S, hk, D), mk(B, S, hk, D)
    o = torch.empty_like(q)
    sc = 1.0 / math.sqrt(D)
    flops_fwd = 4.0 * B * H * S * S * D * (0.5 if a.causal else 1.0)
    if not a.backward:
        ms = timed(lambda: A.attention_forward(q, k, v, a.causal, sc, out=o, impl=a.impl), a.warmup, a.iters)
        return report(f"attention_fwd_{a.impl}", ms, flops_fwd, 0, {"batch": B, "seq": S, "heads": H, "head_dim": D})
    o, lse = A.attention_forward(q, k, v, a.causal, sc, impl=a.impl)
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    bwd_impl = a.bwd_impl or None
    ms = timed(lambda: A.attention_backward(do, q, k, v, o, lse, a.causal, sc, dq, dk, dv, impl=bwd_impl), a.warmup, a.iters)
    return report("attention_bwd", ms, 2.5 * flops_fwd, 0, {"batch": B, "seq": S, "heads": H, "head_dim": D})


def bench_norm(a):
    from ..ops import norm as Nn
    x = torch.randn(a.rows, a.n, device="cuda").bfloat16()
    g = torch.ones(a.n, device="cuda").bfloat16()
    b = torch.zeros(a.n, device="cuda").bfloat16()
    if a.backward:
        # backward with the residual-branch gradient folded in: reads x, dy, dres and writes dx (2 bytes each)
        y, mean, rstd = Nn.norm_forward(x, g, b, 1e-5, False)
        dy, dres = torch.randn_like(x), torch.randn_like(x)
        dg = torch.empty(a.n, dtype=torch.float32, device="cuda")
        db = torch.empty(a.n, dtype=torch.float32, device="cuda")
        dx = torch.empty_like(x)
        fn = lambda: Nn.norm_backward(dy, x, g, mean, rstd, False, dres=dres, dgamma=dg, dbeta=db, dx_out=dx)
        ms = timed(fn, a.warmup, a.iters)
        return report("layer_norm_bwd", ms, 0, 8.0 * a.rows * a.n, {"rows": a.rows, "n": a.n})
    fn = lambda: Nn.layer_norm(x, g, b, 1e-5)
    ms = timed(fn, a.warmup, a.iters)
    return report("layer_norm_fwd", ms, 0, 4.0 * a.rows * a.n, {"rows": a.rows, "n": a.n})


def bench_adam(a):
    from ..ops import optim as O
    n = a.numel
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 1e-3
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    lowp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    fn = lambda: O.adam_step(p, m, v, g, lr=1e-3, step=1, p_lowp=lowp)
    ms = timed(fn, a.warmup, a.iters)
    return report("adam_step", ms, 0, n * (4 * 4 + 3 * 4 + 2.0), {"numel": n})


def bench_paged(a):
    """Decode attention over a paged KV cache: `batch` sequences of `context` cached tokens, pages handed out in a
    shuffled order so that consecutive pages of a sequence are not adjacent in memory."""
    import math
    from ..ops import paged
    B, H, Hk, D, bs = a.batch, a.heads, a.kv_heads, a.head_dim, a.block_size
    per = (a.context + bs - 1) // bs
    nb = B * per + 1
    g = torch.Generator().manual_seed(0)
    kc = torch.randn(nb, bs, Hk, D, generator=g).bfloat16().cuda()
    vc = torch.randn(nb, bs, Hk, D, generator=g).bfloat16().cuda()
    bt = (torch.randperm(nb - 1, generator=g)[:B * per] + 1).to(torch.int32).view(B, per).cuda()
    ctx = torch.full((B,), a.context, dtype=torch.int32, device="cuda")
    q = torch.randn(B, H * D, generator=g).bfloat16().cuda()
    out = torch.empty_like(q)
    fn = lambda: paged.paged_attention_decode(q, kc, vc, bt, ctx, 1.0 / math.sqrt(D), out=out)
    ms = timed(fn, a.warmup, a.iters)
    kv_bytes = 2.0 * B * a.context * Hk * D * 2
    return report("paged_decode_attention", ms, 0, kv_bytes,
                  {"batch": B, "context": a.context, "heads": H, "kv_heads": Hk, "head_dim": D, "block_size": bs,
                   "kv_cache_bytes": int(kv_bytes)})


def bench_launch_overhead(a):
    import time

    from .. import ops
    from ..core import B200Backend
    table = B200Backend("cuda:0").ops()
    x = torch.randn(128, 128, device="cuda").bfloat16()
    y = torch.randn(128, 128, device="cuda").bfloat16()
    r = torch.randn(32, 256, device="cuda").bfloat16()
    w, b = torch.ones(256, device="cuda").bfloat16(), torch.zeros(256, device="cuda").bfloat16()
    cases = [("op_table.matmul 128^3", lambda: table.matmul(x, y)), ("ops.gemm 128^3", lambda: ops.gemm(x, y, b_mn=True)),
             ("ops.linear 128^3", lambda: ops.linear(x, y)), ("ops.softmax 32x256", lambda: ops.softmax(r)),
             ("ops.layer_norm 32x256", lambda: ops.layer_norm(r, w, b, 1e-5)), ("ops.gelu 32x256", lambda: ops.gelu(r)),
             ("ops.binary add 32x256", lambda: ops.binary("add", r, r)),
             ("torch.add 32x256", lambda: torch.add(r, r)), ("torch.mm 128^3", lambda: torch.mm(x, y))]
    rows = []
    for name, fn in cases:
        for _ in range(50):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(a.calls):
            fn()
        host_us = (time.perf_counter() - t0) / a.calls * 1e6
        torch.cuda.synchronize()
        ev = []
        for _ in range(50):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ev.append(e0.elapsed_time(e1) * 1e3)
        ev.sort()
        rows.append({"call": name, "host_us_per_call": round(host_us, 2), "event_bracketed_us": round(ev[len(ev) // 2], 2)})
    out = {"kernel": "launch-overhead", "calls": a.calls, "rows": rows}
    print(json.dumps(out))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.kernels")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192)
    g.add_argument("--act", default="none")
    g.add_argument("--bias", action="store_true")
    g.add_argument("--block-n", type=int, default=0)
    g8 = sub.add_parser("gemm-fp8")
    g8.add_argument("--m", type=int, default=8192)
    g8.add_argument("--n", type=int, default=8192)
    g8.add_argument("--k", type=int, default=8192)
    g8.add_argument("--block-n", type=int, default=0)
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=32)
    t.add_argument("--seq", type=int, default=1024)
    t.add_argument("--heads", type=int, default=12)
    t.add_argument("--kv-heads", type=int, default=0)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--impl", default="tc2", help="tc2 (two query tiles per CTA; tc2:<n> picks a variant), tc (one tile per CTA) or mma")
    t.add_argument("--no-causal", dest="causal", action="store_false")
    t.add_argument("--backward", action="store_true")
    t.add_argument("--bwd-impl", default="", help="backward implementation: tc2, tc or mma (default: the library default)")
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=32768)
    n.add_argument("--n", type=int, default=768)
    n.add_argument("--backward", action="store_true")
    d = sub.add_parser("adam")
    d.add_argument("--numel", type=int, default=124_000_000)
    pg = sub.add_parser("paged")
    pg.add_argument("--batch", type=int, default=64)
    pg.add_argument("--context", type=int, default=4096)
    pg.add_argument("--heads", type=int, default=32)
    pg.add_argument("--kv-heads", type=int, default=8)
    pg.add_argument("--head-dim", type=int, default=128)
    pg.add_argument("--block-size", type=int, default=16)
    lo = sub.add_parser("launch-overhead")
    lo.add_argument("--calls", type=int, default=5000)
    a = ap.parse_args(argv)
    return {"launch-overhead": bench_launch_overhead, "paged": bench_paged, "gemm": bench_gemm, "gemm-fp8": bench_gemm_fp8, "attention": bench_attention, "norm": bench_norm, "adam": bench_adam}[a.op](a)


if __name__ == "__main__":
    main()
