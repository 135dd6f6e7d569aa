"""Layer sizes and batch sizes at the edge of what the kernels address: row pitches that are not multiples of 16 bytes
(they run on zero-padded copies) and empty batches (nothing is launched).  Compared with the CPU reference on the same
bf16-rounded values.  The file sorts behind the rest of the GPU suite: these cases were added last."""
import pytest
import torch

from tolerances import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,fin,fout", [(4, 2, 8), (33, 18, 96), (33, 96, 2), (64, 256, 10), (5, 12, 1)])
def test_linear_layers_of_sizes_the_kernel_cannot_address_run_on_padded_copies(rows, fin, fout, cuda_status):
    """2 -> 8, 18 -> 96, 96 -> 2, 10 classes, a single output: row pitches that are not multiples of 16 bytes.  Forward
    and all three gradients through `ops.linear` equal the CPU reference on the same bf16-rounded values."""
    from rustral_b200 import ops
    g = torch.Generator().manual_seed(rows * 1000 + fin)
    x = (torch.randn(rows, fin, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(fout, fin, generator=g) * 0.2).to(torch.bfloat16)
    b = (torch.randn(fout, generator=g) * 0.1).to(torch.bfloat16)
    res = (torch.randn(rows, fout, generator=g) * 0.1).to(torch.bfloat16)
    outs = []
    for dev in ("cpu", "cuda"):
        xd, wd, bd = (t.detach().clone().to(dev).requires_grad_() for t in (x, w, b))
        y = ops.linear(xd, wd, bd, "gelu", res.to(dev))
        assert y.shape == (rows, fout) and y.is_contiguous()
        y.float().sum().backward()
        outs.append((y.detach().float().cpu(), xd.grad.float().cpu(), wd.grad.float().cpu(), bd.grad.float().cpu()))
    for name, c, got in zip(("y", "dx", "dw", "db"), *outs):
        assert_close(got, c, "gemm_act", what=f"{name} of linear {fin}->{fout}")


def test_empty_batches_run_through_the_gpu_wrappers_without_a_launch(cuda_status):
    """A batch of zero rows is legal input: forward, loss and backward give empty or zero results as on the CPU."""
    from rustral_b200 import ops
    w = (torch.randn(16, 8) * 0.1).to(torch.bfloat16).cuda().requires_grad_()
    b = torch.zeros(16, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    x = torch.zeros(0, 8, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    y = ops.linear(x, w, b, "gelu")
    assert y.shape == (0, 16)
    y.float().sum().backward()
    assert x.grad.shape == (0, 8) and float(w.grad.float().abs().sum()) == 0.0 and float(b.grad.float().abs().sum()) == 0.0
    assert ops.softmax(torch.zeros(0, 8, dtype=torch.bfloat16, device="cuda")).shape == (0, 8)
    g, bt = torch.ones(8, dtype=torch.bfloat16, device="cuda"), torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    assert ops.layer_norm(torch.zeros(0, 8, dtype=torch.bfloat16, device="cuda"), g, bt).shape == (0, 8)
    table = torch.zeros(10, 8, dtype=torch.bfloat16, device="cuda")
    assert ops.embedding(torch.zeros(0, dtype=torch.int64, device="cuda"), table).shape == (0, 8)
    assert ops.sum_dim0(torch.zeros(0, 8, dtype=torch.bfloat16, device="cuda")).tolist() == [0.0] * 8
