"""The same code on either backend: capability queries, the fused linear patterns (matmul + bias + activation in one
GEMM epilogue on the B200, one C++ loop on the CPU) checked against their unfused op-by-op form, pattern matching over
an op trace, the operation and memory profilers, and the tensor pool
(crates/runtime/examples/backend_agnostic_fusion.rs, advanced_optimizations.rs, memory_layout_optimization.rs).

    python examples/backend_agnostic_fusion.py [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import (DType, FusionOptimizer, FusionPattern, FusionTestHarness, MemoryProfiler, OperationProfiler,
                               PatternMatcher, PoolStrategy, TensorPool, generate_random_data)
from rustral_b200.nn import FusionHelper


def main(argv=None):
    a = parser(__doc__).parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    caps = backend.capabilities()
    print(f"backend {backend.name}: bf16={caps.supports_bf16} fused={caps.supports_fused_ops} tensor cores={caps.supports_tensor_cores} "
          f"graphs={caps.supports_cuda_graphs} compute units={caps.num_compute_units} conv layout={caps.preferred_conv_layout.name} "
          f"training dtype={caps.recommended_training_dtype.name}")
    ops = backend.ops()
    x = generate_random_data((64, 256), a.seed).to(dev, dt)
    w = generate_random_data((128, 256), a.seed + 1, 256 ** -0.5).to(dev, dt)
    b = generate_random_data((128,), a.seed + 2, 0.1).to(dev, dt)

    # fused pattern against the op-by-op form, numerics and time
    fuse, harness, results = FusionOptimizer(backend), FusionTestHarness(repeats=20), {}
    for pattern, act in ((FusionPattern.MATMUL_BIAS, None), (FusionPattern.MATMUL_BIAS_RELU, ops.relu), (FusionPattern.MATMUL_BIAS_GELU, ops.gelu)):
        def unfused():
            y = ops.add_row_vector(ops.matmul(x, ops.transpose(w)), b)
            return act(y) if act else y
        r = harness.run_test(unfused, lambda: fuse.apply(pattern, x, w, b), DType.BF16 if dt == torch.bfloat16 else DType.F32)
        results[pattern.value] = r
        print(f"{pattern.value:<18} max |fused - unfused| {r.max_abs_err:.2e}  unfused {r.unfused_ms:.3f} ms  fused {r.fused_ms:.3f} ms  x{r.speedup:.2f}")
    y = FusionHelper.try_linear_gelu(x, w, b)
    assert y.shape == (64, 128)

    # what a graph rewriter would fuse in a recorded op sequence
    trace = ["matmul", "add_row_vector", "gelu", "matmul", "add_row_vector", "softmax", "matmul", "add_row_vector", "relu"]
    found = PatternMatcher().find(trace)
    print("patterns in the trace:", [(i, n, p.value) for i, n, p in found])

    # per-operation timing and memory accounting
    prof = OperationProfiler(use_cuda_events=(a.device != "cpu"))
    for _ in range(5):
        with prof.guard("matmul", x.shape):
            h = ops.matmul(x, ops.transpose(w))
        with prof.guard("softmax", h.shape):
            ops.softmax(h)
    prof.resolve()
    top = prof.most_expensive_ops(2)
    print("most expensive:", [(name, s.count, round(s.total_ms, 3)) for name, s in top])
    mem = MemoryProfiler(capacity_bytes=1 << 20)
    with mem.track_tensor("activations", h):
        risk = mem.predict_oom_risk(planned_bytes=900 << 10)
        print(f"tracking {h.numel() * h.element_size()} B of activations in a 1 MiB budget; planning 900 KiB more -> OOM risk {risk}")
    print(f"allocations still open after the block: {len(mem.find_leaks())}")

    # buffer reuse between steps
    pool = TensorPool(PoolStrategy.STANDARD)
    for _ in range(3):
        t = pool.acquire((64, 128), dt, dev)
        pool.release(t)
        pool.begin_step()
    print("tensor pool:", pool.stats())
    return {"results": {k: (v.passed, v.max_abs_err) for k, v in results.items()}, "patterns": [p.value for _, _, p in found],
            "pool": pool.stats(), "top": [name for name, _ in top]}


if __name__ == "__main__":
    main()
