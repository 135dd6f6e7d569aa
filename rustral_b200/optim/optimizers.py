"""Optimizers over named Parameters (crates/optim/src/lib.rs:22-604).

Every step is one fused kernel per parameter (or per flat buffer): m, v, p and the optional bf16 working copy are
read and written once.  "AdamW" is really decoupled here; `Adam(weight_decay=...)` keeps the reference's coupled
L2 behaviour (crates/optim/src/lib.rs:464-470).  `Sgd.momentum` is used (the reference stores and ignores it).
Checkpoints key state by parameter NAME (the reference keys by process-local id, which does not survive a restart).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from ..core import NamedParameters, Parameter
from ..core.errors import CoreError, ShapeMismatch


class OptimError(CoreError):
    pass


class MissingState(OptimError):
    pass


@dataclass
class Gradient:
    param_id: int
    tensor: torch.Tensor


@dataclass
class AdamState:
    m: torch.Tensor
    v: torch.Tensor
    t: int = 0


@dataclass
class AdamCheckpoint:
    lr: float
    beta1: float
    beta2: float
    eps: float
    weight_decay: float
    decoupled: bool
    state: dict = field(default_factory=dict)      # name -> {"m": list, "v": list, "t": int, "shape": list}

    def to_json(self) -> dict:
        return {"lr": self.lr, "beta1": self.beta1, "beta2": self.beta2, "eps": self.eps,
                "weight_decay": self.weight_decay, "decoupled": self.decoupled, "state": self.state}

    @classmethod
    def from_json(cls, d: dict) -> "AdamCheckpoint":
        return cls(d["lr"], d["beta1"], d["beta2"], d["eps"], d["weight_decay"], d.get("decoupled", False), d["state"])


class Optimizer:
    """step(params, gradients) updates parameters in place; step_named_parameters walks a model."""

    lr: float

    def step(self, params, gradients=None, ctx=None) -> None:
        raise NotImplementedError

    def _grad_of(self, p: Parameter, gradients):
        if gradients is None:
            return p.tensor.grad
        if isinstance(gradients, dict):
            return gradients.get(p.id, gradients.get(p.name))
        for g in gradients:
            if g.param_id == p.id:
                return g.tensor
        return None

    def step_named_parameters(self, model: NamedParameters, grads: dict | None = None, ctx=None) -> None:
        self.step([p for _, p in model.named_parameters()], grads, ctx)

    def zero_grad(self, params) -> None:
        for p in params:
            p.zero_grad()

    def set_lr(self, lr: float) -> None:
        self.lr = lr


class Sgd(Optimizer):
    def __init__(self, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0):
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self._mom: dict = {}

    def step(self, params, gradients=None, ctx=None) -> None:
        with torch.no_grad():
            for p in params:
                g = self._grad_of(p, gradients)
                if g is None:
                    continue
                if tuple(g.shape) != p.shape:
                    raise ShapeMismatch(p.shape, g.shape, f"gradient of {p.name}")
                mom = None
                if self.momentum != 0.0:
                    mom = self._mom.get(p.id)
                    if mom is None:
                        mom = self._mom[p.id] = torch.zeros(p.shape, dtype=torch.float32, device=p.tensor.device)
                if p.tensor.dtype == torch.float32:
                    ops.sgd_step(p.tensor.view(-1), g.contiguous().view(-1), lr=self.lr, momentum=self.momentum,
                                 weight_decay=self.weight_decay, mom=None if mom is None else mom.view(-1))
                else:   # low-precision parameter: update an fp32 shadow and round
                    shadow = p.tensor.float().view(-1)
                    ops.sgd_step(shadow, g.contiguous().view(-1), lr=self.lr, momentum=self.momentum,
                                 weight_decay=self.weight_decay, mom=None if mom is None else mom.view(-1))
                    p.tensor.copy_(shadow.view(p.shape).to(p.tensor.dtype))


class Adam(Optimizer):
    """Adam with optional coupled L2 (`weight_decay`) or decoupled decay (`decoupled=True`, i.e. AdamW)."""

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 0.0, decoupled: bool = False, max_grad_norm: float = 0.0):
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay, self.decoupled, self.max_grad_norm = weight_decay, decoupled, max_grad_norm
        self.state: dict = {}       # ParameterId -> AdamState
        self._master: dict = {}     # fp32 master copies of low-precision parameters
        self._master_seen: dict = {}  # ParameterId -> (data_ptr, tensor version) of the parameter after our last write
        self._names: dict = {}

    def with_betas(self, b1: float, b2: float):
        self.beta1, self.beta2 = b1, b2
        return self

    def with_weight_decay(self, wd: float):
        self.weight_decay = wd
        return self

    @classmethod
    def adamw(cls, lr: float = 1e-3, weight_decay: float = 0.01, **kw):
        return cls(lr=lr, weight_decay=weight_decay, decoupled=True, **kw)

    def _state(self, p: Parameter) -> AdamState:
        st = self.state.get(p.id)
        if st is None:
            z = lambda: torch.zeros(p.numel(), dtype=torch.float32, device=p.tensor.device)
            st = self.state[p.id] = AdamState(z(), z(), 0)
            self._names[p.id] = p.name
        return st

    def step(self, params, gradients=None, ctx=None) -> None:
        params = list(params)
        with torch.no_grad():
            grad_norm = None
            if self.max_grad_norm > 0:
                acc = None
                for p in params:
                    g = self._grad_of(p, gradients)
                    if g is not None:
                        acc = ops.sumsq(g, out=acc, accumulate=acc is not None)
                if acc is not None:
                    grad_norm = ops.optim.sqrt_scalar(acc)
            for p in params:
                g = self._grad_of(p, gradients)
                if g is None:
                    continue
                if tuple(g.shape) != p.shape:
                    raise ShapeMismatch(p.shape, g.shape, f"gradient of {p.name}")
                st = self._state(p)
                st.t += 1
                g = g.contiguous().view(-1)
                if g.dtype not in (torch.float32, torch.bfloat16):
                    g = g.float()
                if p.tensor.dtype == torch.float32:
                    master, lowp = p.tensor.view(-1), None
                else:
                    master = self._fresh_master(p)
                    lowp = p.tensor.view(-1) if p.tensor.dtype == torch.bfloat16 else None
                ops.adam_step(master, st.m, st.v, g, lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                              weight_decay=self.weight_decay, step=st.t, decoupled=self.decoupled, p_lowp=lowp,
                              max_grad_norm=self.max_grad_norm, grad_norm=grad_norm)
                if p.tensor.dtype not in (torch.float32, torch.bfloat16):
                    p.tensor.copy_(master.view(p.shape).to(p.tensor.dtype))
                if p.tensor.dtype != torch.float32:
                    self._master_seen[p.id] = (p.tensor.data_ptr(), p.tensor._version)

    def _fresh_master(self, p: Parameter) -> torch.Tensor:
        """The fp32 master copy of a low-precision parameter.  The copy is re-derived from the parameter whenever
        somebody else wrote the parameter since this optimizer's last step (a state-dict load, a re-initialisation, a
        tied-weight copy): such writes bump the tensor's version counter or replace its storage, the optimizer's own
        kernel write does neither."""
        master = self._master.get(p.id)
        seen = self._master_seen.get(p.id)
        now = (p.tensor.data_ptr(), p.tensor._version)
        if master is None or master.numel() != p.numel() or master.device != p.tensor.device or (seen is not None and seen != now):
            master = self._master[p.id] = p.tensor.detach().float().reshape(-1).clone()
        return master

    def reset_master(self, params=None) -> None:
        """Forgets the fp32 master copies (of `params`, or all): the next step re-derives them from the parameters."""
        ids = list(self._master) if params is None else [p.id for p in params]
        for pid in ids:
            self._master.pop(pid, None)
            self._master_seen.pop(pid, None)

    # ---- checkpoints ---------------------------------------------------------------------------------------------
    def save_checkpoint(self, params=None) -> AdamCheckpoint:
        names = dict(self._names)
        if params is not None:
            names.update({p.id: (n if isinstance(n, str) else p.name) for n, p in
                          ((getattr(x, "name", None), x) if isinstance(x, Parameter) else x for x in params)})
        state = {}
        for pid, st in self.state.items():
            entry = {"m": st.m.detach().cpu().tolist(), "v": st.v.detach().cpu().tolist(), "t": st.t,
                     "shape": [st.m.numel()]}
            if pid in self._master:      # low-precision parameter: the fp32 master copy is part of the state
                entry["master"] = self._master[pid].detach().cpu().tolist()
            state[names.get(pid, str(int(pid)))] = entry
        return AdamCheckpoint(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.decoupled, state)

    def load_checkpoint(self, ckpt: AdamCheckpoint, named_params) -> None:
        """named_params: iterable of (name, Parameter).  Missing names raise; sizes are checked."""
        self.lr, self.beta1, self.beta2, self.eps = ckpt.lr, ckpt.beta1, ckpt.beta2, ckpt.eps
        self.weight_decay, self.decoupled = ckpt.weight_decay, ckpt.decoupled
        staged = {}
        for name, p in named_params:
            if name not in ckpt.state:
                raise MissingState(f"no optimizer state for parameter {name!r}")
            s = ckpt.state[name]
            if len(s["m"]) != p.numel():
                raise ShapeMismatch((p.numel(),), (len(s["m"]),), f"optimizer state of {name}")
            dev = p.tensor.device
            master = None
            if "master" in s and p.tensor.dtype != torch.float32:
                if len(s["master"]) != p.numel():
                    raise ShapeMismatch((p.numel(),), (len(s["master"]),), f"master copy of {name}")
                master = torch.tensor(s["master"], dtype=torch.float32, device=dev)
            staged[p.id] = (name, AdamState(torch.tensor(s["m"], dtype=torch.float32, device=dev),
                                            torch.tensor(s["v"], dtype=torch.float32, device=dev), int(s["t"])), master, p)
        for pid, (name, st, master, p) in staged.items():
            self.state[pid] = st
            self._names[pid] = name
            self._master.pop(pid, None)
            self._master_seen.pop(pid, None)
            if master is not None:
                # the saved master copy continues the run exactly; the working copy is rounded from it
                self._master[pid] = master
                with torch.no_grad():
                    p.tensor.copy_(master.view(p.shape).to(p.tensor.dtype))
                self._master_seen[pid] = (p.tensor.data_ptr(), p.tensor._version)


def AdamW(lr: float = 1e-3, weight_decay: float = 0.01, **kw) -> Adam:
    """Adam with decoupled weight decay."""
    return Adam.adamw(lr, weight_decay, **kw)
