"""Python face of the C++ f32 reference backend (csrc/cpu): the oracle the tests hold the CUDA kernels and the
torch CPU path to, and the timed CPU baseline.  All functions take and return contiguous fp32 CPU tensors."""
from __future__ import annotations

import torch

from .. import _native as N


def _f(t):
    return t.detach().to(torch.float32).contiguous()


def matmul(a, b):
    a, b = _f(a), _f(b)
    c = torch.empty(a.shape[0], b.shape[1])
    N.cpu().rb_cpu_matmul(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0], a.shape[1], b.shape[1])
    return c


def linear(x, w, bias=None, act: str = "none"):
    x, w = _f(x), _f(w)
    bias = None if bias is None else _f(bias)
    y = torch.empty(x.shape[0], w.shape[0])
    N.cpu().rb_cpu_linear(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(), y.data_ptr(), x.shape[0],
                          x.shape[1], w.shape[0], {"none": 0, "gelu": 1, "relu": 2, "silu": 3}[act])
    return y


def softmax_rows(x, log_mode: bool = False):
    x = _f(x)
    y = torch.empty_like(x)
    N.cpu().rb_cpu_softmax_rows(x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], int(log_mode))
    return y


def layer_norm(x, gamma=None, beta=None, eps: float = 1e-5, rms: bool = False):
    x = _f(x)
    g = None if gamma is None else _f(gamma)
    b = None if beta is None else _f(beta)
    y = torch.empty_like(x)
    mean, rstd = torch.empty(x.shape[0]), torch.empty(x.shape[0])
    N.cpu().rb_cpu_layer_norm(x.data_ptr(), None if g is None else g.data_ptr(), None if b is None else b.data_ptr(),
                              y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), x.shape[0], x.shape[1], eps, int(rms))
    return y, mean, rstd


def layer_norm_bwd(dy, x, gamma, mean, rstd, rms: bool = False):
    dy, x, g, mean, rstd = _f(dy), _f(x), _f(gamma), _f(mean), _f(rstd)
    dx, dg, db = torch.empty_like(x), torch.empty(x.shape[1]), torch.empty(x.shape[1])
    N.cpu().rb_cpu_layer_norm_bwd(dy.data_ptr(), x.data_ptr(), g.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                  dx.data_ptr(), dg.data_ptr(), db.data_ptr(), x.shape[0], x.shape[1], int(rms))
    return dx, dg, db


def unary(op: str, x):
    from .elementwise import UNARY
    x = _f(x)
    y = torch.empty_like(x)
    N.cpu().rb_cpu_unary(UNARY[op], x.data_ptr(), y.data_ptr(), x.numel())
    return y


def cross_entropy(logits, targets, scale: float = 1.0, ignore_index: int = -100):
    x = _f(logits)
    t = targets.to(torch.int64).contiguous()
    loss, d = torch.empty(x.shape[0]), torch.empty_like(x)
    N.cpu().rb_cpu_cross_entropy(x.data_ptr(), t.data_ptr(), loss.data_ptr(), d.data_ptr(), x.shape[0], x.shape[1], scale,
                                 ignore_index)
    return loss, d


def adam(p, m, v, g, lr, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, step=1, decoupled=False):
    N.cpu().rb_cpu_adam(p.data_ptr(), m.data_ptr(), v.data_ptr(), _f(g).data_ptr(), p.numel(), lr, b1, b2, eps, wd, step,
                        int(decoupled))


def attention(q, k, v, causal: bool, scale: float):
    q, k, v = _f(q), _f(k), _f(v)
    B, Sq, H, Dh = q.shape
    o = torch.empty_like(q)
    N.cpu().rb_cpu_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, Sq, k.shape[1], H, k.shape[2], Dh,
                             int(causal), scale)
    return o


def moe_route(logits, k: int, renorm: bool = True):
    x = _f(logits)
    T, E = x.shape
    idx = torch.empty(T, k, dtype=torch.int32)
    w = torch.empty(T, k)
    aux = torch.zeros(1)
    N.cpu().rb_cpu_moe_route(x.data_ptr(), T, E, k, int(renorm), idx.data_ptr(), w.data_ptr(), aux.data_ptr())
    return idx, w, float(aux)
