"""Softmax cross-entropy (fused forward + backward) and row softmax / log-softmax."""
from __future__ import annotations

import torch

from .. import _native as N


def cross_entropy_fwd_bwd(logits2: torch.Tensor, targets: torch.Tensor, n_valid: int | None = None,
                          grad_scale: float = 1.0, ignore_index: int = -100, dlogits=None, want_grad: bool = True,
                          loss_out=None):
    """Per-row loss (fp32 [rows]) and, when `want_grad`, ``(softmax - onehot) * grad_scale``.

    ``logits2`` is [rows, n_pad]; only the first ``n_valid`` columns take part (a padded vocabulary).
    ``dlogits`` may alias ``logits2`` to overwrite the logits in place.  ``loss_out`` (fp32 [rows], optional)
    receives the per-row loss instead of a new tensor.
    """
    rows, n_pad = logits2.shape
    n_valid = n_pad if n_valid is None else n_valid
    if not logits2.is_cuda:
        lf = logits2.float()[:, :n_valid]
        lse = torch.logsumexp(lf, -1)
        valid = (targets != ignore_index) & (targets >= 0) & (targets < n_valid)
        safe_t = torch.where(valid, targets, torch.zeros_like(targets))
        loss = torch.where(valid, lse - lf.gather(1, safe_t[:, None])[:, 0], torch.zeros_like(lse))
        grad = None
        if want_grad:
            p = torch.softmax(lf, -1)
            p.scatter_add_(1, safe_t[:, None], -torch.ones(rows, 1))
            p = p * (grad_scale * valid.float())[:, None]
            grad = dlogits if dlogits is not None else torch.empty_like(logits2)
            full = torch.zeros(rows, n_pad)
            full[:, :n_valid] = p
            grad.copy_(full.to(grad.dtype))
        if loss_out is not None:
            loss_out.copy_(loss)
            loss = loss_out
        return loss, lse, grad
    if logits2.dtype != torch.bfloat16:
        raise TypeError("cross_entropy: CUDA logits must be bf16")
    if logits2.stride(1) != 1:
        raise ValueError("cross_entropy: logits need a contiguous last dimension")
    targets = targets.to(torch.int64)
    loss = loss_out if loss_out is not None else torch.empty(rows, dtype=torch.float32, device=logits2.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits2.device)
    grad = None
    if want_grad:
        grad = dlogits if dlogits is not None else torch.empty_like(logits2)
    if rows == 0:
        return loss, lse, grad
    N.check(N.kernels().rb_cross_entropy(logits2.data_ptr(), logits2.stride(0), targets.data_ptr(), loss.data_ptr(),
                                         lse.data_ptr(), N.ptr(grad), grad.stride(0) if grad is not None else 0, rows,
                                         n_valid, n_pad, grad_scale, ignore_index, N.stream_ptr()),
            "rb_cross_entropy")
    return loss, lse, grad


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, n_valid, ignore_index):
        l2 = logits.reshape(-1, logits.shape[-1])
        t = targets.reshape(-1)
        count = max(int((t != ignore_index).sum()), 1)   # host value: the kernel folds 1/count into the gradient
        loss, _, grad = cross_entropy_fwd_bwd(l2, t, n_valid, 1.0 / count, ignore_index,
                                              want_grad=logits.requires_grad)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        from .elementwise import sum_all
        return sum_all(loss) / count

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad * g.to(grad.dtype)).reshape(ctx.shape), None, None, None


def cross_entropy(logits, targets, n_valid: int | None = None, ignore_index: int = -100):
    """Mean cross-entropy over rows whose target is not `ignore_index`; per-row softmax (the eager loss of the
    reference soft-maxes over the whole tensor, crates/nn/src/loss.rs:95, which is only right for one row)."""
    if logits.is_cuda and logits.dtype == torch.float32:
        # fp32 logits on the GPU (a head evaluated in full precision): the row log-softmax kernel with its exact
        # gradient, then the target column of every row; the fused kernel below is the bf16 path
        l2 = logits.reshape(-1, logits.shape[-1])
        if n_valid is not None and n_valid < l2.shape[1]:
            l2 = l2[:, :n_valid]
        lp = log_softmax(l2.contiguous())
        t = targets.reshape(-1).to(torch.int64)
        valid = (t != ignore_index) & (t >= 0) & (t < l2.shape[1])
        picked = lp.gather(1, torch.where(valid, t, torch.zeros_like(t))[:, None])[:, 0]
        return -(picked * valid).sum() / valid.sum().clamp_min(1)
    return _CrossEntropyFn.apply(logits, targets, n_valid, ignore_index)


def _softmax_impl(x, log_mode: bool):
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])      # a reshape, even as a no-op view, costs about 2 us
    if not x.is_cuda:
        f = torch.log_softmax if log_mode else torch.softmax
        return f(x2.float(), -1).to(x.dtype).reshape(x.shape)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if x2.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("softmax: fp32 or bf16 only")
    y = torch.empty_like(x2)
    if x2.numel() == 0:
        return y if x.dim() == 2 else y.reshape(x.shape)
    N.check(N.kernels().rb_softmax_rows(x2.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1], x2.stride(0),
                                        y.stride(0), int(log_mode), int(x2.dtype == torch.bfloat16), N.stream_ptr()),
            "rb_softmax_rows")
    return y if x.dim() == 2 else y.reshape(x.shape)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, log_mode):
        y = _softmax_impl(x, log_mode)
        ctx.save_for_backward(y)
        ctx.log_mode = log_mode
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        y2 = y.reshape(-1, y.shape[-1]).float().contiguous()
        g2 = dy.reshape(-1, y.shape[-1]).float().contiguous()
        if not y.is_cuda:
            if ctx.log_mode:
                dx = g2 - torch.exp(y2) * g2.sum(-1, keepdim=True)
            else:
                dx = y2 * (g2 - (g2 * y2).sum(-1, keepdim=True))
        else:
            dx = torch.empty_like(y2)
            N.check(N.kernels().rb_softmax_rows_bwd(y2.data_ptr(), g2.data_ptr(), dx.data_ptr(), y2.shape[0],
                                                    y2.shape[1], int(ctx.log_mode), N.stream_ptr()),
                    "rb_softmax_rows_bwd")
        return dx.to(y.dtype).reshape(y.shape), None


def softmax(x):
    """Softmax over the last dimension."""
    if not N.wants_grad(x):
        return _softmax_impl(x, False)
    return _SoftmaxFn.apply(x, False)


def log_softmax(x):
    """Log-softmax over the last dimension with the exact gradient (the reference's tape op uses a
    placeholder backward, crates/autodiff/src/lib.rs:611-626)."""
    if not N.wants_grad(x):
        return _softmax_impl(x, True)
    return _SoftmaxFn.apply(x, True)
