"""bf16 GEMM with fused epilogues on the tcgen05 kernel; fp32 torch math for CPU tensors.

``gemm(a, b)`` computes ``D[M,N] = epilogue(alpha * A[M,K] @ B[N,K]^T)``.  ``a_mn`` / ``b_mn`` say that
the operand is handed over transposed (``[K,M]`` / ``[K,N]``), which is how the backward GEMMs of a
linear layer read activations and weights without a transpose in memory.

Epilogue order: ``+ bias`` -> activation (or multiply by ``act'(aux_in)``) -> ``+ residual`` ->
``+ D`` when ``accumulate``.  ``aux_out`` receives the pre-activation for the backward pass.
"""
from __future__ import annotations

import math
import threading

import torch

from .. import _native as N

_ACT_FWD = {"gelu", "relu", "silu"}
_ACT_BWD = {"dgelu", "drelu", "dsilu", "mul"}


def _gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def _gelu_tanh_grad(x):
    k0, k1 = math.sqrt(2.0 / math.pi), 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def act_reference(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "gelu":
        return _gelu_tanh(x)
    if name == "relu":
        return torch.relu(x)
    if name == "silu":
        return x * torch.sigmoid(x)
    return x


def act_grad_reference(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "gelu":
        return _gelu_tanh_grad(x)
    if name == "relu":
        return (x > 0).to(x.dtype)
    if name == "silu":
        s = torch.sigmoid(x)
        return s * (1 + x * (1 - s))
    return torch.ones_like(x)


def _gemm_cpu(a, b, a_mn, b_mn, bias, act, residual, aux_in, aux_out, out, out_dtype, accumulate, alpha):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    v = A @ B.t()
    if alpha != 1.0:
        v = v * alpha
    if bias is not None:
        v = v + bias.float()
    if act in _ACT_FWD:
        if aux_out is not None:
            aux_out.copy_(v.to(aux_out.dtype))
            v = aux_out.float()
        v = act_reference(act, v)
    elif act in _ACT_BWD:
        ax = aux_in.float()
        v = v * (ax if act == "mul" else act_grad_reference(act[1:], ax))
    if residual is not None:
        v = v + residual.float()
    if out is None:
        return v if v.dtype == out_dtype else v.to(out_dtype)      # v is a fresh tensor: no second buffer, no copy
    if accumulate:
        out.copy_((out.float() + v).to(out.dtype))
    else:
        out.copy_(v.to(out.dtype))
    return out


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


def _row_aligned(t, mult: int = 8) -> bool:
    """A 2-D operand the kernel can address: 16-byte aligned base, row pitch a multiple of `mult` elements."""
    return t is None or (t.data_ptr() % 16 == 0 and (t.shape[0] == 1 or t.stride(0) % mult == 0) and t.stride(-1) == 1)


def _needs_padding(a, b, bias, residual, aux_in, aux_out, out, out_dtype, n: int) -> bool:
    """True when a tensor of the call does not meet the kernel's addressing rules (TMA operands and vector stores want
    16-byte aligned bases and row pitches): layer sizes such as 2 -> 8 or 10 classes."""
    out_mult = 4 if out_dtype == torch.float32 else 8
    if out is None:
        if n % out_mult:
            return True
    elif not _row_aligned(out, out_mult):
        return True
    if not (_row_aligned(a) and _row_aligned(b) and _row_aligned(residual) and _row_aligned(aux_in) and _row_aligned(aux_out)):
        return True
    if (a.shape[0] == 1 and a.shape[1] % 8) or (b.shape[0] == 1 and b.shape[1] % 8):
        return True
    return bias is not None and bias.data_ptr() % 16 != 0


def _gemm_padded(a, b, *, a_mn, b_mn, bias, act, residual, aux_in, aux_out, out, out_dtype, accumulate, alpha, row_scale,
                 col_scale, call=None):
    """The same product with every dimension the kernel addresses by rows rounded up to a multiple of 8: operands are
    copied into zero-filled buffers, the kernel runs on those, and the live corner of the result is copied back.  Zeros
    in the contraction add nothing; padded rows and columns of the output are discarded.  This is the path of small or
    odd layer sizes, where two extra copies do not matter; aligned shapes never come here."""
    call = call or gemm
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    Nn = b.shape[1] if b_mn else b.shape[0]
    M8 = _round8(M) if a_mn else M
    N8 = _round8(Nn)
    K8 = _round8(K)

    def pad(t, rows, cols):
        if t is None:
            return None
        z = torch.zeros((rows, cols), dtype=t.dtype, device=t.device)
        z[:t.shape[0], :t.shape[1]] = t
        return z

    def padv(v, n):
        if v is None:
            return None
        z = torch.zeros(n, dtype=v.dtype, device=v.device)
        z[:v.numel()] = v.reshape(-1)
        return z
    ap = pad(a, K8, M8) if a_mn else pad(a, M8, K8)
    bp = pad(b, K8, N8) if b_mn else pad(b, N8, K8)
    outp = torch.zeros((M8, N8), dtype=out_dtype, device=a.device)
    acc = bool(accumulate and out is not None)
    if acc:
        outp[:M, :Nn] = out
    auxp = torch.zeros((M8, N8), dtype=aux_out.dtype, device=a.device) if aux_out is not None else None
    call(ap, bp, a_mn=a_mn, b_mn=b_mn, bias=padv(bias, N8), act=act, residual=pad(residual, M8, N8), aux_in=pad(aux_in, M8, N8),
         aux_out=auxp, out=outp, accumulate=acc, alpha=alpha, row_scale=padv(row_scale, M8), col_scale=padv(col_scale, N8))
    if aux_out is not None:
        aux_out.copy_(auxp[:M, :Nn])
    if out is not None:
        out.copy_(outp[:M, :Nn])
        return out
    return outp[:M, :Nn].contiguous() if (M8 != M or N8 != Nn) else outp


_workspaces: dict = {}
WORKSPACE_BYTES = 128 << 20


def _workspace(device) -> torch.Tensor:
    """Split-K scratch, one per device and stream, allocated on first use."""
    key = N.stream_key(device)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_plain_tls = threading.local()


def _plain_args() -> dict:
    """Per-thread cache of filled argument blocks (autograd runs backward GEMMs on its own thread)."""
    d = getattr(_plain_tls, "args", None)
    if d is None:
        d = _plain_tls.args = {}
    return d


# Optional tile-plan table: fn(M, N, K, a_mn, b_mn, out_is_f32) -> {"block_n", "splits", "group_m"} or None.  Installed by
# tune.GemmTuningTable.apply(); consulted only for plain calls that leave the plan to the kernel's own cost model.
_PLAN_HOOK = None


def set_plan_hook(fn) -> None:
    global _PLAN_HOOK
    _PLAN_HOOK = fn


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias=None, act: str = "none",
         residual=None, aux_in=None, aux_out=None, out=None, out_dtype=None, accumulate: bool = False,
         alpha: float = 1.0, block_n: int = 0, group_m: int = 0, max_ctas: int = 0, splits: int = 0,
         peer: dict | None = None, row_scale=None, col_scale=None) -> torch.Tensor:
    """`row_scale` (fp32 [M]) / `col_scale` (fp32 [N]) multiply the accumulator's rows / columns before the bias (weight
    scales of quantised layers).  `peer` selects the tensor-parallel modes of the kernel (see parallel/fused_tp.py): a dict with `mode`
    (1: remote row blocks of A are pulled from the peers' shards inside the kernel; 2: output row blocks are
    stored into their owner's receive slot), `world`, `rank`, `rows_per_rank`, `epoch`, `ready_flags` (pointer,
    mode 1) and `peer_ptrs` (one device address per rank)."""
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    Nn, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: contraction sizes differ ({K} vs {Kb})")
    if out is not None:
        out_dtype = out.dtype
    elif out_dtype is None:
        out_dtype = a.dtype if a.dtype in (torch.bfloat16, torch.float32) else torch.float32
    if act not in N.ACT:
        raise ValueError(f"gemm: unknown epilogue activation {act!r}")
    if not a.is_cuda:
        if row_scale is not None or col_scale is not None:
            a = a.float().t() if a_mn else a.float()
            a_mn = False
            if row_scale is not None:
                a = a * row_scale.float()[:, None]
            if col_scale is not None:
                b = (b.float().t() if b_mn else b.float()) * col_scale.float()[:, None]
                b_mn = False
        return _gemm_cpu(a, b, a_mn, b_mn, bias, act, residual, aux_in, aux_out, out, out_dtype, accumulate, alpha)

    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm: CUDA operands must be bf16 (accumulation is fp32)")
    if M == 0 or Nn == 0:
        # an empty batch (or an empty layer): nothing to launch; a given output is left as it is
        if aux_out is not None and aux_out.numel():
            aux_out.zero_()
        return out if out is not None else torch.empty((M, Nn), dtype=out_dtype, device=a.device)
    if K == 0 and peer is None and row_scale is None and col_scale is None:
        # an empty contraction (the weight gradient of an empty batch): the product is zero and only the epilogue is left;
        # the reference formula does that with tensor ops on the operands' device
        return _gemm_cpu(a, b, a_mn, b_mn, bias, act, residual, aux_in, aux_out, out, out_dtype, accumulate, alpha)
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm: operands must have a contiguous last dimension")
    # the cheap integer test settles the common aligned call; the full check runs only when it fails or optional tensors exist
    suspect = (((a.stride(0) | b.stride(0)) & 7) or (Nn & (3 if out_dtype == torch.float32 else 7))
               or ((a.data_ptr() | b.data_ptr()) & 15) or out is not None or bias is not None or residual is not None
               or aux_in is not None or aux_out is not None)
    if suspect and peer is None and _needs_padding(a, b, bias, residual, aux_in, aux_out, out, out_dtype, Nn):
        return _gemm_padded(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act=act, residual=residual, aux_in=aux_in, aux_out=aux_out,
                            out=out, out_dtype=out_dtype, accumulate=accumulate, alpha=alpha, row_scale=row_scale,
                            col_scale=col_scale)
    if out is None:
        out = torch.empty((M, Nn), dtype=out_dtype, device=a.device)
        accumulate = False
    if out.stride(1) != 1 or out.shape != (M, Nn):
        raise ValueError("gemm: bad output tensor")
    if _PLAN_HOOK is not None and block_n == 0 and splits == 0 and group_m == 0 and peer is None and max_ctas == 0:
        plan = _PLAN_HOOK(M, Nn, K, a_mn, b_mn, out.dtype == torch.float32)
        if plan:
            block_n, splits, group_m = int(plan.get("block_n", 0)), int(plan.get("splits", 0)), int(plan.get("group_m", 0))
    if (bias is None and residual is None and aux_in is None and aux_out is None and row_scale is None
            and col_scale is None and peer is None):
        # Plain product: the argument block of a (shape, strides, plan) is filled once and kept; a call only writes the
        # three addresses (and the split-K workspace), which halves the Python time of a small launch.
        cache = _plain_args()
        key = (M, Nn, K, a_mn, b_mn, act, out.dtype, accumulate, alpha, block_n, group_m, max_ctas, splits,
               a.stride(0), b.stride(0), out.stride(0))
        g = cache.get(key)
        if g is None:
            if len(cache) > 4096:
                cache.clear()
            g = N.RbGemmArgs()
            g.lda, g.ldb, g.ldd = a.stride(0), b.stride(0), out.stride(0)
            g.M, g.N, g.K = M, Nn, K
            g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
            g.act = N.ACT[act]
            g.out_f32 = int(out.dtype == torch.float32)
            g.accumulate = int(accumulate)
            g.alpha = alpha
            g.block_n, g.group_m, g.max_ctas, g.splits = block_n, group_m, max_ctas, splits
            cache[key] = g
        g.a, g.b, g.d = a.data_ptr(), b.data_ptr(), out.data_ptr()
        if splits != 1 and K >= 2048 and act == "none":
            ws = _workspace(a.device)
            g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
        N.check(N.kernels().rb_gemm_bf16(g, N.stream_ptr()), "rb_gemm_bf16")
        return out
    for t, nm in ((bias, "bias"), (residual, "residual"), (aux_in, "aux_in"), (aux_out, "aux_out")):
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"gemm: {nm} must be bf16")
    g = N.RbGemmArgs()
    g.a, g.b, g.d = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.bias = N.ptr(bias)
    g.residual = N.ptr(residual)
    g.aux_in = N.ptr(aux_in)
    g.aux_out = N.ptr(aux_out)
    g.lda, g.ldb, g.ldd = a.stride(0), b.stride(0), out.stride(0)
    g.ldr = residual.stride(0) if residual is not None else 0
    g.ld_aux_in = aux_in.stride(0) if aux_in is not None else 0
    g.ld_aux_out = aux_out.stride(0) if aux_out is not None else 0
    g.M, g.N, g.K = M, Nn, K
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.act = N.ACT[act]
    g.out_f32 = int(out.dtype == torch.float32)
    g.accumulate = int(accumulate)
    g.alpha = alpha
    g.block_n, g.group_m, g.max_ctas, g.splits = block_n, group_m, max_ctas, splits
    for t, n_, nm in ((row_scale, M, "row_scale"), (col_scale, Nn, "col_scale")):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n_ or not t.is_contiguous() or t.device != a.device):
            raise TypeError(f"gemm: {nm} must be a contiguous fp32 vector of {n_} elements on the operands' device")
    g.a_scale, g.b_scale = N.ptr(row_scale), N.ptr(col_scale)
    if row_scale is not None or col_scale is not None:
        splits = g.splits = 1                    # the scales are applied by the GEMM's own epilogue
    if peer is not None:
        g.peer_mode, g.peer_world, g.peer_rank = peer["mode"], peer["world"], peer["rank"]
        g.rows_per_rank, g.peer_epoch = peer["rows_per_rank"], peer["epoch"] & 0xFFFFFFFF
        g.ready_flags = peer.get("ready_flags")
        for r, pp in enumerate(peer["peer_ptrs"]):
            g.peer_ptrs[r] = pp
        g.splits = 1
    elif splits != 1 and K >= 2048 and act == "none":
        ws = _workspace(a.device)
        g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
    N.check(N.kernels().rb_gemm_bf16(g, N.stream_ptr()), "rb_gemm_bf16")
    return out


class WeightGradStore:
    """Deferred weight-gradient work of `linear` layers.

    Inside ``with WeightGradStore.defer() as queue:`` the backward pass of every `linear` computes only the gradient
    of its input (the part the previous pipeline stage is waiting for); the weight and bias gradient GEMMs are pushed
    onto `queue` and run later with ``WeightGradStore.run(queue)``, which accumulates them into ``.grad`` of the leaf
    tensors exactly as autograd would have.  This is what the zero-bubble pipeline schedule is built from (the
    reference only names that schedule: crates/distributed/src/pipeline_parallel.rs:55-62)."""
    # The queue is looked up per thread first (CPU tensors: autograd runs the backward pass on the calling thread, and
    # ranks may be threads of one process), then process-wide (CUDA tensors: autograd runs their backward functions on
    # a worker thread of the device; one rank per process).
    _tls = __import__("threading").local()
    _process_queue = None

    class _Defer:
        def __enter__(self):
            self.q = []
            WeightGradStore._tls.queue = self.q
            WeightGradStore._process_queue = self.q
            return self.q

        def __exit__(self, *exc):
            WeightGradStore._tls.queue = None
            if WeightGradStore._process_queue is self.q:       # another thread's deferral may have replaced it
                WeightGradStore._process_queue = None
            return False

    @classmethod
    def current(cls):
        q = getattr(cls._tls, "queue", None)
        return q if q is not None else cls._process_queue

    @classmethod
    def defer(cls):
        return cls._Defer()

    @staticmethod
    def run(queue) -> None:
        with torch.no_grad():
            for fn in queue:
                fn()
        queue.clear()

    @staticmethod
    def _accumulate(leaf: torch.Tensor, g: torch.Tensor) -> None:
        leaf.grad = g if leaf.grad is None else leaf.grad.add_(g)


class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b) (+ residual); W is [out, in] as in the reference's Linear (crates/nn/src/linear.rs:21)."""

    @staticmethod
    def forward(ctx, x, w, bias, act, residual):
        x2 = x.reshape(-1, x.shape[-1])
        need_pre = act in _ACT_FWD and (x.requires_grad or w.requires_grad)
        pre = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device) if need_pre else None
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = gemm(x2, w, bias=bias, act=act, residual=res2, aux_out=pre, out_dtype=x.dtype)
        ctx.save_for_backward(x2, w, pre)
        ctx.w_leaf = w if w.is_leaf else None                      # where a deferred weight gradient is accumulated
        ctx.b_leaf = bias if (bias is not None and bias.is_leaf) else None
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        if ctx.act in _ACT_FWD:
            from .elementwise import unary_bwd
            dz = unary_bwd(ctx.act, pre, dy2)
        else:
            dz = dy2
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dz, w, b_mn=True, out_dtype=x2.dtype).reshape(ctx.x_shape)
        queue = WeightGradStore.current()
        want_b = ctx.has_bias and ctx.needs_input_grad[2]
        if queue is not None and ctx.w_leaf is not None and (not want_b or ctx.b_leaf is not None):
            w_leaf, b_leaf, want_w = ctx.w_leaf, ctx.b_leaf, ctx.needs_input_grad[1]

            def later():
                if want_w:
                    WeightGradStore._accumulate(w_leaf, gemm(dz, x2, a_mn=True, b_mn=True, out_dtype=w_leaf.dtype))
                if want_b:
                    from .elementwise import sum_dim0
                    WeightGradStore._accumulate(b_leaf, sum_dim0(dz).to(b_leaf.dtype))
            queue.append(later)
            return dx, None, None, None, dres
        if ctx.needs_input_grad[1]:
            dw = gemm(dz, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if want_b:
            from .elementwise import sum_dim0
            db = sum_dim0(dz).to(w.dtype)
        return dx, dw, db, None, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias=None, act: str = "none", residual=None) -> torch.Tensor:
    """Differentiable fused linear: ``act(x @ w.T + bias) + residual``."""
    if not N.wants_grad(x, w, bias, residual):
        if x.dim() == 2:
            return gemm(x, w, bias=bias, act=act, residual=residual, out_dtype=x.dtype)
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = gemm(x.reshape(-1, x.shape[-1]), w, bias=bias, act=act, residual=res2, out_dtype=x.dtype)
        return y.reshape(*x.shape[:-1], w.shape[0])
    return _LinearFn.apply(x, w, bias, act, residual)
