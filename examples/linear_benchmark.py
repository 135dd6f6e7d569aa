"""Linear-layer forward time on the CPU reference backend and, when a GPU is present, on the B200 backend, for the three
shapes the reference times (256 x 256 -> 128, 1024 x 512 -> 256, 128 x 4096 -> 2048), with the largest element-wise
difference between the two results (crates/candle-backend/examples/benchmark.rs).

    python examples/linear_benchmark.py [--iters 5]
"""
import time

import torch

from _common import parser

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.nn import LinearBuilder

SHAPES = [(256, 256, 128), (1024, 512, 256), (128, 4096, 2048)]


def time_forward(layer, x, iters, cuda):
    ctx = ForwardCtx.inference()
    with torch.no_grad():
        y = layer(x, ctx)                                              # warm-up (and tensor-map / plan caches on the GPU)
        if cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                y = layer(x, ctx)
            e1.record()
            e1.synchronize()
            return y, e0.elapsed_time(e1) / iters
        t0 = time.perf_counter()
        for _ in range(iters):
            y = layer(x, ctx)
        return y, (time.perf_counter() - t0) * 1e3 / iters


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    cpu = CpuBackend()
    gpu = None
    if torch.cuda.is_available():
        from rustral_b200.core import B200Backend
        gpu = B200Backend("cuda:0")
    rows = []
    print(f"{'batch x in -> out':<24} {'cpu ms':>10} {'b200 ms':>10} {'max |diff|':>12}")
    for batch, fin, fout in SHAPES:
        x = torch.randn(batch, fin, generator=torch.Generator().manual_seed(a.seed))
        layer = LinearBuilder(fin, fout).with_bias().seed(a.seed + 1).build(cpu)
        y_cpu, ms_cpu = time_forward(layer, x, a.iters, False)
        ms_gpu = diff = None
        if gpu is not None:
            twin = LinearBuilder(fin, fout).with_bias().seed(a.seed + 1).build(gpu)     # same seed: same weights, in bf16
            y_gpu, ms_gpu = time_forward(twin, x.to(gpu.device(), gpu.dtype), a.iters, True)
            diff = float((y_gpu.float().cpu() - y_cpu).abs().max())
        rows.append({"shape": (batch, fin, fout), "cpu_ms": ms_cpu, "b200_ms": ms_gpu, "max_abs_diff": diff})
        print(f"{batch:>5} x {fin:>4} -> {fout:<6}    {ms_cpu:>10.3f} {('%.3f' % ms_gpu) if ms_gpu is not None else '-':>10} "
              f"{('%.2e' % diff) if diff is not None else '-':>12}")
    return {"rows": rows}


if __name__ == "__main__":
    main()
