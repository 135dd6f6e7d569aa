"""Tape: the reference's reverse-mode interface (crates/autodiff/src/lib.rs:119-1310) as a facade over torch.autograd.

Values are addressed by `TensorId`; every recorded op runs the framework's differentiable op (CUDA kernels on the
B200 backend, reference math on CPU) and stores the result.  `backward(output)` seeds ones, walks the graph
and returns a `GradientStore`; parameters watched twice share one leaf, so their gradients accumulate
(lib.rs:150-163).  log_softmax has its exact gradient (the reference's is a placeholder, :611-626).
"""
from __future__ import annotations

import itertools
import time

import torch

from .. import ops
from ..core import ForwardCtx, Parameter
from ..core.errors import InvalidArgument, ShapeMismatch

_ids = itertools.count(1)


class TensorId(int):
    @staticmethod
    def fresh() -> "TensorId":
        return TensorId(next(_ids))


class GradientStore:
    def __init__(self, grads: dict, param_map: dict):
        self._g = grads                  # TensorId -> tensor
        self._param_map = param_map      # ParameterId -> TensorId

    def get(self, tid: TensorId):
        return self._g.get(tid)

    def param_gradient(self, p: Parameter):
        tid = self._param_map.get(p.id)
        return None if tid is None else self._g.get(tid)

    def by_parameter_id(self) -> dict:
        return {pid: self._g[tid] for pid, tid in self._param_map.items() if tid in self._g}

    def __contains__(self, tid):
        return tid in self._g

    def __len__(self):
        return len(self._g)


class Tape:
    def __init__(self, ctx: ForwardCtx | None = None):
        self.ctx = ctx
        self.values: dict = {}
        self.param_map: dict = {}
        self._leaves: list = []
        self.num_ops = 0
        self.last_gradients = None       # GradientStore of the most recent backward()

    # ---- leaves ----------------------------------------------------------------------------------------------------
    def watch(self, t: torch.Tensor) -> TensorId:
        tid = TensorId.fresh()
        leaf = t.detach().clone().requires_grad_(t.is_floating_point())
        self.values[tid] = leaf
        if leaf.requires_grad:
            self._leaves.append(tid)
        return tid

    def constant(self, t: torch.Tensor) -> TensorId:
        tid = TensorId.fresh()
        self.values[tid] = t.detach()
        return tid

    def watch_parameter(self, p: Parameter) -> TensorId:
        tid = self.param_map.get(p.id)
        if tid is not None:
            return tid
        tid = TensorId.fresh()
        leaf = p.tensor.detach().requires_grad_(True)
        self.values[tid] = leaf
        self.param_map[p.id] = tid
        self._leaves.append(tid)
        return tid

    def value(self, tid: TensorId) -> torch.Tensor:
        return self.values[tid]

    def _record(self, name: str, out: torch.Tensor, t0: float) -> TensorId:
        tid = TensorId.fresh()
        self.values[tid] = out
        self.num_ops += 1
        if self.ctx is not None and self.ctx.profiler is not None:
            from ..core.operation_profiler import DeviceType, shape_bucket
            self.ctx.profiler.record(name, (time.perf_counter() - t0) * 1e3,
                                     DeviceType.CUDA if out.is_cuda else DeviceType.CPU, shape_bucket(out.shape))
        return tid

    def _op(self, name, fn, *tids):
        t0 = time.perf_counter()
        return self._record(name, fn(*[self.values[t] for t in tids]), t0)

    def apply(self, name: str, fn) -> TensorId:
        """Records the result of `fn()` (a differentiable computation over parameters and earlier tape values, e.g. a
        whole module forward) as one tape op."""
        t0 = time.perf_counter()
        return self._record(name, fn(), t0)

    # ---- recorded ops -----------------------------------------------------------------------------------------------
    def add(self, a, b): return self._op("add", lambda x, y: x + y, a, b)
    def sub(self, a, b): return self._op("sub", lambda x, y: x - y, a, b)
    def mul(self, a, b): return self._op("mul", lambda x, y: x * y, a, b)
    def mul_scalar(self, a, s: float): return self._op("mul_scalar", lambda x: x * s, a)
    def add_scalar(self, a, s: float): return self._op("add_scalar", lambda x: x + s, a)
    def relu(self, a): return self._op("relu", ops.relu, a)
    def gelu(self, a): return self._op("gelu", ops.gelu, a)
    def sigmoid(self, a): return self._op("sigmoid", torch.sigmoid, a)
    def tanh(self, a): return self._op("tanh", torch.tanh, a)
    def transpose_tape(self, a): return self._op("transpose", lambda x: x.t().contiguous(), a)
    def sum_all_tape(self, a): return self._op("sum_all", lambda x: x.float().sum(), a)
    def softmax(self, a): return self._op("softmax", ops.softmax, a)
    def log_softmax(self, a): return self._op("log_softmax", ops.log_softmax, a)
    def reshape_tape(self, a, shape): return self._op("reshape", lambda x: x.reshape(tuple(shape)), a)

    def matmul(self, a, b):
        def f(x, y):
            if x.dim() != 2 or y.dim() != 2 or x.shape[1] != y.shape[0]:
                raise ShapeMismatch((x.shape[0], "k"), y.shape, "Tape.matmul")
            return ops.linear(x, y.t().contiguous())
        return self._op("matmul", f, a, b)

    def add_row_vector_tape(self, a, row): return self._op("add_row_vector", lambda x, r: x + r, a, row)

    def linear_tape(self, x, w, b=None):
        if b is None:
            return self._op("linear", lambda xx, ww: ops.linear(xx, ww), x, w)
        return self._op("linear", lambda xx, ww, bb: ops.linear(xx, ww, bb), x, w, b)

    def fused_linear_bias_relu_tape(self, x, w, b):
        return self._op("fused_linear_bias_relu", lambda xx, ww, bb: ops.linear(xx, ww, bb, "relu"), x, w, b)

    def fused_linear_bias_gelu_tape(self, x, w, b):
        return self._op("fused_linear_bias_gelu", lambda xx, ww, bb: ops.linear(xx, ww, bb, "gelu"), x, w, b)

    def layer_norm_tape(self, x, gamma, beta, eps: float = 1e-5):
        return self._op("layer_norm", lambda xx, g, bt: ops.layer_norm(xx, g, bt, eps), x, gamma, beta)

    def gather_rows_tape(self, table, ids):
        ids_t = torch.as_tensor(ids, dtype=torch.int64)
        return self._op("gather_rows", lambda t: ops.embedding(ids_t.to(t.device), t), table)

    def concat_tape(self, tids, dim: int = 0):
        return self._op("concat", lambda *xs: torch.cat(xs, dim), *tids)

    def slice_tape(self, a, start: int, end: int, dim: int = 0):
        def f(x):
            if not (0 <= start <= end <= x.shape[dim]):
                raise InvalidArgument("slice out of range")
            return x.narrow(dim, start, end - start)
        return self._op("slice", f, a)

    def cross_entropy_loss(self, logits, targets):
        """logits [B, C]; targets: class indices (list / int64 tensor) or a one-hot [B, C] tensor.  Mean over the batch."""
        def f(lg):
            t = targets if isinstance(targets, torch.Tensor) else torch.as_tensor(targets)
            t = t.to(lg.device)
            if t.dim() == 2:
                t = t.argmax(-1)
            return ops.cross_entropy(lg, t.to(torch.int64))
        return self._op("cross_entropy_loss", f, logits)

    def mse_loss(self, pred, target):
        return self._op("mse_loss", lambda p, t: ((p.float() - t.float()) ** 2).mean(), pred, target)

    def attention(self, q, k, v, causal: bool = False):
        return self._op("attention", lambda a, b, c: ops.flash_attention(a, b, c, causal), q, k, v)

    # ---- backward ----------------------------------------------------------------------------------------------------
    def backward(self, output: TensorId, make_ones=None, ops_table=None) -> GradientStore:
        out = self.values[output]
        seed = torch.ones_like(out) if make_ones is None else make_ones(out.shape)
        leaves = [t for t in self._leaves if self.values[t].requires_grad]
        grads = torch.autograd.grad(out, [self.values[t] for t in leaves], grad_outputs=seed, allow_unused=True)
        store = {t: g for t, g in zip(leaves, grads) if g is not None}
        self.last_gradients = GradientStore(store, dict(self.param_map))
        return self.last_gradients


class GradExt:
    """Gradient lookup for a `Parameter` (crates/autodiff/src/lib.rs:1280-1310): from a tape whose backward has run
    (`gradient`), or from a `GradientStore` plus the tape's parameter map (`gradient_from_store`)."""

    @staticmethod
    def gradient(param: Parameter, tape: "Tape"):
        store = getattr(tape, "last_gradients", None)
        return None if store is None else store.param_gradient(param)

    @staticmethod
    def gradient_from_store(param: Parameter, grads: GradientStore, param_map: dict | None = None):
        if param_map is None:
            return grads.param_gradient(param)
        tid = param_map.get(param.id)
        return None if tid is None else grads.get(tid)


class GradExtFromStore:
    """The store-based half of `GradExt` under its own name (crates/autodiff/src/lib.rs:1293-1310): look a parameter's
    gradient up in a `GradientStore` through a parameter map, without the tape at hand."""

    gradient_from_store = staticmethod(GradExt.gradient_from_store)


class TapeModule:
    """Mixin: `forward_tape(input_id, tape, ctx) -> TensorId` in terms of a module's ordinary differentiable forward."""

    def forward_tape(self, x: TensorId, tape: Tape, ctx: ForwardCtx) -> TensorId:
        pids = {}
        for _, p in self.named_parameters():
            tid = tape.watch_parameter(p)
            pids[p.id] = tid
        # run the module on the tape's leaves so that gradients land in the tape
        saved = {}
        for _, p in self.named_parameters():
            saved[p.id] = p.tensor
            p.tensor = tape.values[pids[p.id]]
        try:
            import time as _t
            t0 = _t.perf_counter()
            out = self.forward(tape.values[x], ctx)
        finally:
            for _, p in self.named_parameters():
                p.tensor = saved[p.id]
        return tape._record(type(self).__name__, out, t0)
