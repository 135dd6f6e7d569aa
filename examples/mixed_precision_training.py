"""Mixed-precision training with dynamic loss scaling: an fp16-style run whose loss scale starts far too high, so the
first steps overflow, are skipped, and halve the scale until gradients are finite; the scale then grows back after every
`growth_interval` clean steps.  The result is compared with plain fp32 training of the same model
(crates/runtime/examples/mixed_precision_training.rs).

    python examples/mixed_precision_training.py [--steps 120] [--device cuda:0]
"""
import torch

from _common import backend_for, parser

from rustral_b200.core import ForwardCtx
from rustral_b200.nn import LinearBuilder, MSELoss, Sequential
from rustral_b200.optim import Adam, LossScaleScheduler, MixedPrecisionOptimizer
from rustral_b200.optim.mixed_precision import DType, MixedPrecisionStats


def make_model(backend, seed):
    return Sequential(LinearBuilder(16, 64).with_bias().seed(seed).activation("gelu").build(backend),
                      LinearBuilder(64, 1).with_bias().seed(seed + 1).build(backend))


def main(argv=None):
    ap = parser(__doc__)
    ap.add_argument("--steps", type=int, default=120)
    a = ap.parse_args(argv)
    backend = backend_for(a.device)
    dev, dt = backend.device(), backend.dtype
    g = torch.Generator().manual_seed(a.seed)
    x = torch.randn(512, 16, generator=g)
    y = 30.0 * torch.sin(x[:, :4].sum(1, keepdim=True))        # losses in the hundreds: 2^127 times that is not finite
    x, y = x.to(dev, dt), y.to(dev)
    mse = MSELoss()

    def run(mixed: bool):
        model = make_model(backend, a.seed)
        scaler = LossScaleScheduler(initial_scale=2.0 ** 127, growth_interval=25, max_scale=2.0 ** 127)
        opt = MixedPrecisionOptimizer(Adam(lr=3e-2), DType.FLOAT16, scaler) if mixed else Adam(lr=3e-2)
        scales, losses = [], []
        for _ in range(a.steps):
            model.zero_grad()
            loss = mse(model(x, ForwardCtx.train(backend)).float(), y)
            (opt.scale_loss(loss) if mixed else loss).backward()
            opt.step(model.parameters())
            losses.append(float(loss.detach()))
            if mixed:
                scales.append(scaler.scale)
        return losses, scales, (opt.skipped_steps if mixed else 0)
    ref_losses, _, _ = run(False)
    losses, scales, skipped = run(True)
    settled = min(scales)
    print(f"loss scale: start 2^127, lowest {settled:.3g}, final {scales[-1]:.3g}; {skipped} of {a.steps} steps skipped for overflow")
    print(f"final loss: fp32 {ref_losses[-1]:.5f}, loss-scaled {losses[-1]:.5f}")
    st = MixedPrecisionStats.for_dtype(DType.FLOAT16)
    print(f"storage: {st.bytes_per_param} B/parameter + {st.master_bytes_per_param} B fp32 master copy")
    return {"skipped": skipped, "lowest_scale": settled, "final_scale": scales[-1], "loss_fp32": ref_losses[-1], "loss_mixed": losses[-1],
            "loss_first": losses[0]}


if __name__ == "__main__":
    main()
