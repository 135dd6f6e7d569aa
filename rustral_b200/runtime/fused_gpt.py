"""Hand-scheduled training engine for decoder-only transformers on one B200 (per rank).

The engine owns flat parameter / gradient / optimizer-state buffers and a set of preallocated activation
buffers, and runs forward, backward and the optimizer as an explicit sequence of kernel launches:

* every matmul is the tcgen05 GEMM; bias, GELU, residual adds and the GELU derivative ride in its epilogues,
  weight gradients are accumulated straight into the fp32 gradient buffer by the GEMM epilogue;
* attention reads q, k, v in place from the packed QKV projection and writes packed gradients back;
* LayerNorm / RMSNorm backward folds the residual-branch gradient in the same pass;
* the loss kernel overwrites the logits with their gradient;
* AdamW updates fp32 master weights and writes the bf16 working copy in the same pass, with global-norm
  clipping decided on the device.

This is the hot path the training entry points (`Trainer`, `bench.py`) use.  It replaces the per-example tape loop
of the reference's trainer (crates/runtime/src/tape_trainer.rs:310-485) and its per-parameter optimizer ops
(crates/optim/src/lib.rs:433-514).  Parameter names follow crates/nn/src/tape_transformer.rs:261-274 and
crates/runtime/examples/wikitext2_lm.rs:120-137.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from .. import ops
from ..models.config import GPTConfig
from ..ops import attention as attn_ops
from ..ops import norm as norm_ops
from ..ops import rotary as rope_ops
from ..ops.matmul import gemm

ALIGN = 128   # elements; keeps every parameter 256-byte aligned in bf16 and 512-byte aligned in fp32


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    decay: bool
    init: str        # "normal", "ones", "zeros", "normal_scaled" (residual projections)
    offset: int = 0

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


def param_specs(cfg: GPTConfig) -> list:
    d, f, V = cfg.d_model, cfg.ffn_dim, cfg.vocab_padded
    specs = [ParamSpec("tok_embed.embed", (V, d), True, "normal")]
    if cfg.arch == "gpt2":
        specs.append(ParamSpec("pos_embed.embed", (cfg.seq_len, d), True, "normal"))
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        if cfg.arch == "gpt2":
            specs += [
                ParamSpec(p + "ln1.weight", (d,), False, "ones"), ParamSpec(p + "ln1.bias", (d,), False, "zeros"),
                ParamSpec(p + "attn.wqkv.weight", (cfg.qkv_dim, d), True, "normal"),
                ParamSpec(p + "attn.wqkv.bias", (cfg.qkv_dim,), False, "zeros"),
                ParamSpec(p + "attn.wo.weight", (d, d), True, "normal_scaled"),
                ParamSpec(p + "attn.wo.bias", (d,), False, "zeros"),
                ParamSpec(p + "ln2.weight", (d,), False, "ones"), ParamSpec(p + "ln2.bias", (d,), False, "zeros"),
                ParamSpec(p + "ffn.fc1.weight", (f, d), True, "normal"), ParamSpec(p + "ffn.fc1.bias", (f,), False, "zeros"),
                ParamSpec(p + "ffn.fc2.weight", (d, f), True, "normal_scaled"),
                ParamSpec(p + "ffn.fc2.bias", (d,), False, "zeros"),
            ]
        else:
            specs += [
                ParamSpec(p + "ln1.weight", (d,), False, "ones"),
                ParamSpec(p + "attn.wqkv.weight", (cfg.qkv_dim, d), True, "normal"),
                ParamSpec(p + "attn.wo.weight", (d, d), True, "normal_scaled"),
                ParamSpec(p + "ln2.weight", (d,), False, "ones"),
                ParamSpec(p + "ffn.gate_up.weight", (2 * f, d), True, "normal"),
                ParamSpec(p + "ffn.down.weight", (d, f), True, "normal_scaled"),
            ]
    specs.append(ParamSpec("final_norm.weight", (d,), False, "ones"))
    if cfg.arch == "gpt2":
        specs.append(ParamSpec("final_norm.bias", (d,), False, "zeros"))
    if not cfg.tie_embeddings:
        specs.append(ParamSpec("head.weight", (V, d), True, "normal"))
    # decayed parameters first, so each optimizer group is one contiguous range of the flat buffers
    specs.sort(key=lambda s: (not s.decay,))
    off = 0
    for s in specs:
        s.offset = off
        off += (s.numel + ALIGN - 1) // ALIGN * ALIGN
    return specs


class FlatParams:
    """Flat bf16 working copy, fp32 master copy, fp32 gradients and Adam moments, with named views."""

    def __init__(self, cfg: GPTConfig, device, seed: int = 0, pad_to: int = ALIGN):
        self.cfg = cfg
        self.specs = param_specs(cfg)
        last = self.specs[-1]
        total = last.offset + (last.numel + ALIGN - 1) // ALIGN * ALIGN
        self.total = (total + pad_to - 1) // pad_to * pad_to
        self.decay_end = next((s.offset for s in self.specs if not s.decay), self.total)
        self.device = torch.device(device)
        lowp = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.master = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.lowp = torch.zeros(self.total, dtype=lowp, device=self.device)
        self.grad = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.m = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.by_name = {s.name: s for s in self.specs}
        self._init(seed)

    def _init(self, seed: int) -> None:
        self.master.copy_(init_flat_host(self.cfg, self.specs, self.total, seed))
        self.sync_lowp()

    def sync_lowp(self) -> None:
        if self.lowp.dtype == torch.float32:
            self.lowp.copy_(self.master)
        else:
            ops.cast_f32_to_bf16(self.master, self.lowp)

    def view(self, buf: torch.Tensor, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return buf[s.offset:s.offset + s.numel].view(s.shape)

    def w(self, name):
        return self.view(self.lowp, name)

    def g(self, name):
        return self.view(self.grad, name)

    # ---- hooks of the sharded store (parallel/zero3.py): nothing to do when every rank holds everything ---------
    per_micro_reduce = False

    def begin_micro(self, first_micro: bool) -> None:
        pass

    def acquire(self, bucket: int, prefetch=None) -> None:
        pass

    def begin_grads(self, bucket: int) -> None:
        pass

    def grads_done(self, bucket: int) -> None:
        pass

    def end_micro(self) -> None:
        pass

    def state_key(self):
        return ()

    def get_state(self):
        return None

    def set_state(self, st) -> None:
        pass

    # ---- checkpoint views ---------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        """fp32 tensors keyed by parameter name, vocabulary padding removed; fused projections are split into the
        per-matrix names of the reference (attn.wq / wk / wv)."""
        return flat_to_state(self.cfg, self.specs, self.master.detach().float().cpu())

    def load_state_dict(self, state: dict) -> None:
        """Strict: every expected key present, no extra keys, shapes equal; nothing is written before all checks pass."""
        host = self.master.detach().cpu().clone()
        state_to_flat(self.cfg, self.specs, state, host)
        self.master.copy_(host)
        self.sync_lowp()


def init_flat_host(cfg: GPTConfig, specs: list, total: int, seed: int) -> torch.Tensor:
    """Host fp32 image of freshly initialised parameters in the flat layout of `specs` (same values for every way of
    distributing them afterwards: one generator, parameters drawn in `specs` order)."""
    gen = torch.Generator().manual_seed(seed)
    host = torch.zeros(total, dtype=torch.float32)
    for s in specs:
        v = host[s.offset:s.offset + s.numel].view(s.shape)
        if s.init == "ones":
            v.fill_(1.0)
        elif s.init == "normal":
            v.normal_(0.0, cfg.init_std, generator=gen)
        elif s.init == "normal_scaled":
            v.normal_(0.0, cfg.init_std / math.sqrt(2 * cfg.n_layer), generator=gen)
        if s.name in ("tok_embed.embed", "head.weight") and cfg.vocab_padded > cfg.vocab_size:
            v[cfg.vocab_size:].zero_()     # padded vocabulary rows stay inert
    return host


def flat_to_state(cfg: GPTConfig, specs: list, host: torch.Tensor) -> dict:
    """Named fp32 tensors from a host image in the flat layout: vocabulary padding removed, the fused QKV projection
    split into the per-matrix names of the reference (attn.wq / wk / wv)."""
    out = {}
    hd = cfg.head_dim
    for s in specs:
        t = host[s.offset:s.offset + s.numel].view(s.shape).clone()
        if s.name in ("tok_embed.embed", "head.weight"):
            t = t[:cfg.vocab_size].clone()
        if ".attn.wqkv." in s.name:
            q_end, k_end = cfg.n_head * hd, (cfg.n_head + cfg.n_kv_head) * hd
            for nm, sl in (("wq", slice(0, q_end)), ("wk", slice(q_end, k_end)), ("wv", slice(k_end, None))):
                out[s.name.replace("wqkv", nm)] = t[sl].clone()
        else:
            out[s.name] = t
    return out


def state_to_flat(cfg: GPTConfig, specs: list, state: dict, host: torch.Tensor) -> None:
    """Writes named tensors into a host image in the flat layout.  Strict: every expected key present, no extra keys,
    shapes equal; `host` is only written after all checks have passed."""
    from ..core.errors import SerializationError, ShapeMismatch
    expected = flat_to_state(cfg, specs, host)
    missing = [k for k in expected if k not in state]
    extra = [k for k in state if k not in expected]
    if missing:
        raise SerializationError(f"missing keys: {missing}")
    if extra:
        raise SerializationError(f"unexpected keys: {extra}")
    for k, t in expected.items():
        if tuple(state[k].shape) != tuple(t.shape):
            raise ShapeMismatch(t.shape, state[k].shape, k)
    for s in specs:
        v = host[s.offset:s.offset + s.numel].view(s.shape)
        if ".attn.wqkv." in s.name:
            parts = [state[s.name.replace("wqkv", nm)].float() for nm in ("wq", "wk", "wv")]
            v.copy_(torch.cat(parts, 0))
        elif s.name in ("tok_embed.embed", "head.weight"):
            v[:cfg.vocab_size].copy_(state[s.name].float())
        else:
            v.copy_(state[s.name].float())


class FusedGPTEngine:
    """Forward / backward / optimizer for one model replica (or one data-parallel rank)."""

    def __init__(self, cfg: GPTConfig, device=None, micro_batch: int = 8, seed: int = 0, lr: float = 3e-4,
                 betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, max_grad_norm: float = 1.0,
                 flat_pad_to: int = ALIGN, params=None):
        """`params`: a parameter store to use instead of a `FlatParams` built here (the sharded store of ZeRO-3,
        `parallel.zero3.ShardedParams`)."""
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.cfg = cfg
        self.device = torch.device(device)
        self.micro_batch = micro_batch
        self.params = params if params is not None else FlatParams(cfg, self.device, seed, pad_to=flat_pad_to)
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        self.act_dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self._acts = None
        self._acts_tokens = 0
        self.loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        # CUDA-graph replay of the micro-batch forward + backward (about 380 launches): RUSTRAL_TRAIN_GRAPHS=0 disables it
        self.use_graphs = self.device.type == "cuda" and os.environ.get("RUSTRAL_TRAIN_GRAPHS", "1") != "0"
        self._fb_graphs: dict = {}
        self.grad_norm_sq = torch.zeros((), dtype=torch.float32, device=self.device)
        self.grad_norm = torch.zeros((), dtype=torch.float32, device=self.device)
        self.kernel_launches = 0

    # ------------------------------------------------------------------------------------------ buffers
    def _buffers(self, T: int):
        if self._acts is not None and self._acts_tokens == T:
            return self._acts
        cfg, dev, dt = self.cfg, self.device, self.act_dtype
        d, f = cfg.d_model, cfg.ffn_dim
        e = lambda *shape, dtype=dt: torch.empty(shape, dtype=dtype, device=dev)
        layers = []
        for _ in range(cfg.n_layer):
            L = dict(x=e(T, d), ln1=e(T, d), rstd1=e(T, dtype=torch.float32), qkv=e(T, cfg.qkv_dim), attn=e(T, d),
                     lse=e(T // cfg.seq_len if T >= cfg.seq_len else 1, cfg.n_head, min(T, cfg.seq_len), dtype=torch.float32),
                     x1=e(T, d), ln2=e(T, d), rstd2=e(T, dtype=torch.float32))
            if cfg.arch == "gpt2":
                L.update(mean1=e(T, dtype=torch.float32), mean2=e(T, dtype=torch.float32), hpre=e(T, f), h=e(T, f))
            else:
                L.update(gu=e(T, 2 * f), h=e(T, f))
            layers.append(L)
        acts = dict(layers=layers, xf_in=e(T, d), xf=e(T, d), rstdf=e(T, dtype=torch.float32),
                    meanf=e(T, dtype=torch.float32), logits=e(T, cfg.vocab_padded),
                    row_loss=e(T, dtype=torch.float32))
        self._acts, self._acts_tokens = acts, T
        return acts

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, ids: torch.Tensor, want_logits: bool = True):
        """ids: int64 [B, S] on the device.  Fills the activation buffers; returns logits [B*S, vocab_padded]."""
        cfg, P = self.cfg, self.params
        B, S = ids.shape
        T = B * S
        A = self._buffers(T)
        rms = cfg.arch == "llama"
        H, Hk, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        scale = 1.0 / math.sqrt(D)
        x = A["layers"][0]["x"]
        # bucket 0 (embeddings, final norm, head) stays usable for the whole pass; block l is bucket 1 + l, gathered
        # one block ahead when the parameters are sharded (no-ops otherwise)
        P.acquire(0, prefetch=1)
        ops.embedding_forward(ids.reshape(-1), P.w("tok_embed.embed"),
                              P.w("pos_embed.embed") if cfg.arch == "gpt2" else None, S, out=x)
        for l, L in enumerate(A["layers"]):
            p = f"layers.{l}."
            x = L["x"]
            P.acquire(1 + l, prefetch=(2 + l) if l + 1 < cfg.n_layer else None)
            _, m1, r1 = norm_ops.norm_forward(x, P.w(p + "ln1.weight"), None if rms else P.w(p + "ln1.bias"),
                                              cfg.norm_eps, rms, out=L["ln1"])
            L["rstd1"] = r1
            if not rms:
                L["mean1"] = m1
            gemm(L["ln1"], P.w(p + "attn.wqkv.weight"), bias=None if rms else P.w(p + "attn.wqkv.bias"), out=L["qkv"])
            qkv = L["qkv"]
            if rms:
                rope_ops.rope_(qkv, H + Hk, D, S, theta=cfg.rope_theta)     # q and k heads are adjacent columns
            q = qkv[:, :H * D].view(B, S, H, D)
            k = qkv[:, H * D:(H + Hk) * D].view(B, S, Hk, D)
            v = qkv[:, (H + Hk) * D:].view(B, S, Hk, D)
            if self.device.type == "cuda":
                _, L["lse"] = attn_ops.attention_forward(q, k, v, True, scale, out=L["attn"].view(B, S, H, D))
            else:
                L["attn"].copy_(attn_ops.attention_reference(q, k, v, True, scale).reshape(T, H * D))
            gemm(L["attn"], P.w(p + "attn.wo.weight"), bias=None if rms else P.w(p + "attn.wo.bias"), residual=x,
                 out=L["x1"])
            _, m2, r2 = norm_ops.norm_forward(L["x1"], P.w(p + "ln2.weight"), None if rms else P.w(p + "ln2.bias"),
                                              cfg.norm_eps, rms, out=L["ln2"])
            L["rstd2"] = r2
            if not rms:
                L["mean2"] = m2
            nxt = A["layers"][l + 1]["x"] if l + 1 < cfg.n_layer else A["xf_in"]
            if rms:
                gemm(L["ln2"], P.w(p + "ffn.gate_up.weight"), out=L["gu"])
                rope_ops.swiglu_forward(L["gu"], out=L["h"])
                gemm(L["h"], P.w(p + "ffn.down.weight"), residual=L["x1"], out=nxt)
            else:
                gemm(L["ln2"], P.w(p + "ffn.fc1.weight"), bias=P.w(p + "ffn.fc1.bias"), act="gelu", aux_out=L["hpre"],
                     out=L["h"])
                gemm(L["h"], P.w(p + "ffn.fc2.weight"), bias=P.w(p + "ffn.fc2.bias"), residual=L["x1"], out=nxt)
        _, mf, rf = norm_ops.norm_forward(A["xf_in"], P.w("final_norm.weight"), None if rms else P.w("final_norm.bias"),
                                          cfg.norm_eps, rms, out=A["xf"])
        A["meanf"], A["rstdf"] = mf, rf
        if want_logits:
            head = P.w("tok_embed.embed" if cfg.tie_embeddings else "head.weight")
            gemm(A["xf"], head, out=A["logits"])
        return A["logits"]

    # ------------------------------------------------------------------------------------------ backward
    def forward_backward(self, ids: torch.Tensor, targets: torch.Tensor, grad_scale: float, first_micro: bool):
        """One micro-batch: forward, loss, backward.  Gradients accumulate into the flat fp32 buffer (written, not
        added, when `first_micro`).  The summed token loss is added to ``self.loss_acc``."""
        cfg, P = self.cfg, self.params
        B, S = ids.shape
        T = B * S
        rms = cfg.arch == "llama"
        H, Hk, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        scale = 1.0 / math.sqrt(D)
        P.begin_micro(first_micro)
        # a sharded store reduces every micro-batch's gradients into its shard: the local buffers are written afresh
        fresh = first_micro or P.per_micro_reduce
        acc = not fresh
        head_name = "tok_embed.embed" if cfg.tie_embeddings else "head.weight"
        logits = self.forward(ids)
        A = self._acts
        loss_rows, _, dlogits = ops.cross_entropy_fwd_bwd(logits, targets.reshape(-1), cfg.vocab_size, grad_scale,
                                                          dlogits=logits)
        ops.binary("add", self.loss_acc.view(1), ops.sum_all(loss_rows).view(1), out=self.loss_acc.view(1))

        P.begin_grads(0)
        gemm(dlogits, A["xf"], a_mn=True, b_mn=True, out=P.g(head_name), accumulate=acc)
        dxf = gemm(dlogits, P.w(head_name), b_mn=True, out_dtype=self.act_dtype)
        dx, _, _ = norm_ops.norm_backward(dxf, A["xf_in"], P.w("final_norm.weight"), A["meanf"], A["rstdf"], rms,
                                          dgamma=P.g("final_norm.weight"),
                                          dbeta=None if rms else P.g("final_norm.bias"), accumulate=acc)
        for l in range(cfg.n_layer - 1, -1, -1):
            L = A["layers"][l]
            p = f"layers.{l}."
            P.acquire(1 + l, prefetch=l if l > 0 else None)
            P.begin_grads(1 + l)
            if rms:
                gemm(dx, L["h"], a_mn=True, b_mn=True, out=P.g(p + "ffn.down.weight"), accumulate=acc)
                dh = gemm(dx, P.w(p + "ffn.down.weight"), b_mn=True, out_dtype=self.act_dtype)
                dgu = rope_ops.swiglu_backward(dh, L["gu"])
                gemm(dgu, L["ln2"], a_mn=True, b_mn=True, out=P.g(p + "ffn.gate_up.weight"), accumulate=acc)
                dln2 = gemm(dgu, P.w(p + "ffn.gate_up.weight"), b_mn=True, out_dtype=self.act_dtype)
            else:
                gemm(dx, L["h"], a_mn=True, b_mn=True, out=P.g(p + "ffn.fc2.weight"), accumulate=acc)
                ops.sum_dim0(dx, out=P.g(p + "ffn.fc2.bias"), accumulate=acc)
                dhp = gemm(dx, P.w(p + "ffn.fc2.weight"), b_mn=True, act="dgelu", aux_in=L["hpre"],
                           out_dtype=self.act_dtype)
                gemm(dhp, L["ln2"], a_mn=True, b_mn=True, out=P.g(p + "ffn.fc1.weight"), accumulate=acc)
                ops.sum_dim0(dhp, out=P.g(p + "ffn.fc1.bias"), accumulate=acc)
                dln2 = gemm(dhp, P.w(p + "ffn.fc1.weight"), b_mn=True, out_dtype=self.act_dtype)
            dx1, _, _ = norm_ops.norm_backward(dln2, L["x1"], P.w(p + "ln2.weight"), None if rms else L["mean2"],
                                               L["rstd2"], rms, dres=dx, dgamma=P.g(p + "ln2.weight"),
                                               dbeta=None if rms else P.g(p + "ln2.bias"), accumulate=acc)
            gemm(dx1, L["attn"], a_mn=True, b_mn=True, out=P.g(p + "attn.wo.weight"), accumulate=acc)
            if not rms:
                ops.sum_dim0(dx1, out=P.g(p + "attn.wo.bias"), accumulate=acc)
            dattn = gemm(dx1, P.w(p + "attn.wo.weight"), b_mn=True, out_dtype=self.act_dtype)
            qkv = L["qkv"]
            q = qkv[:, :H * D].view(B, S, H, D)
            k = qkv[:, H * D:(H + Hk) * D].view(B, S, Hk, D)
            v = qkv[:, (H + Hk) * D:].view(B, S, Hk, D)
            dqkv = torch.empty_like(qkv)
            dq = dqkv[:, :H * D].view(B, S, H, D)
            dk = dqkv[:, H * D:(H + Hk) * D].view(B, S, Hk, D)
            dv = dqkv[:, (H + Hk) * D:].view(B, S, Hk, D)
            if self.device.type == "cuda":
                attn_ops.attention_backward(dattn.view(B, S, H, D), q, k, v, L["attn"].view(B, S, H, D), L["lse"], True,
                                            scale, dq=dq, dk=dk, dv=dv)
            else:
                self._attention_backward_cpu(dattn.view(B, S, H, D), q, k, v, scale, dq, dk, dv)
            if rms:
                rope_ops.rope_(dqkv, H + Hk, D, S, theta=cfg.rope_theta, inverse=True)
            gemm(dqkv, L["ln1"], a_mn=True, b_mn=True, out=P.g(p + "attn.wqkv.weight"), accumulate=acc)
            if not rms:
                ops.sum_dim0(dqkv, out=P.g(p + "attn.wqkv.bias"), accumulate=acc)
            dln1 = gemm(dqkv, P.w(p + "attn.wqkv.weight"), b_mn=True, out_dtype=self.act_dtype)
            dx, _, _ = norm_ops.norm_backward(dln1, L["x"], P.w(p + "ln1.weight"), None if rms else L["mean1"],
                                              L["rstd1"], rms, dres=dx1, dgamma=P.g(p + "ln1.weight"),
                                              dbeta=None if rms else P.g(p + "ln1.bias"), accumulate=acc)
            P.grads_done(1 + l)
        # embeddings
        if fresh:
            if cfg.arch == "gpt2":
                ops.scalar_op("fill", P.g("pos_embed.embed").view(-1), 0.0, out=P.g("pos_embed.embed").view(-1))
            if not cfg.tie_embeddings:
                ops.scalar_op("fill", P.g("tok_embed.embed").view(-1), 0.0, out=P.g("tok_embed.embed").view(-1))
        ops.embedding_backward(ids.reshape(-1), dx, P.g("tok_embed.embed"),
                               P.g("pos_embed.embed") if cfg.arch == "gpt2" else None, S)
        P.grads_done(0)
        P.end_micro()

    def _forward_backward_graphed(self, ids, targets, grad_scale: float, first_micro: bool) -> None:
        """`forward_backward` replayed from a CUDA graph.  One graph per (shape, first_micro, grad_scale); the first
        two calls of a key run eagerly (lazy kernel configuration, scratch allocation, tensor-map cache), the third
        is captured and every later one is a copy of the token ids into static buffers plus one graph launch."""
        key = (tuple(ids.shape), bool(first_micro), float(grad_scale), self.params.state_key())
        g = self._fb_graphs.get(key)
        if g is None:
            g = {"calls": 0, "graph": None, "ids": torch.empty_like(ids, memory_format=torch.contiguous_format),
                 "tgt": torch.empty_like(targets, memory_format=torch.contiguous_format)}
            self._fb_graphs[key] = g
        if g["graph"] is None and g["calls"] < 2:
            g["calls"] += 1
            self.forward_backward(ids, targets, grad_scale, first_micro)
            return
        g["ids"].copy_(ids)
        g["tgt"].copy_(targets)
        from .. import _native
        if g["graph"] is None:
            torch.cuda.current_stream(self.device).synchronize()
            graph = torch.cuda.CUDAGraph()
            before = _native.launch_count
            with torch.cuda.graph(graph):
                self.forward_backward(g["ids"], g["tgt"], grad_scale, first_micro)
            g["launches"] = _native.launch_count - before      # kernels recorded in the graph
            _native.launch_count = before                      # nothing ran during capture
            g["graph"] = graph
            g["store_state"] = self.params.get_state()         # host-side bookkeeping of the store after this pass
        g["graph"].replay()
        self.params.set_state(g["store_state"])
        _native.launch_count += g["launches"]                  # a replay launches every recorded kernel

    @staticmethod
    def _attention_backward_cpu(do, q, k, v, scale, dq, dk, dv):
        qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
        o = attn_ops.attention_reference(qf, kf, vf, True, scale)
        o.backward(do.float())
        dq.copy_(qf.grad)
        dk.copy_(kf.grad)
        dv.copy_(vf.grad)

    # ------------------------------------------------------------------------------------------ optimizer
    def compute_grad_norm(self):
        """Global L2 norm of the accumulated gradient as a device scalar."""
        ops.sumsq(self.params.grad, out=self.grad_norm_sq)
        ops.optim.sqrt_scalar(self.grad_norm_sq, out=self.grad_norm)
        return self.grad_norm

    def optimizer_step(self, lr: float | None = None, shard: slice | None = None, grad_norm=None):
        """AdamW on the flat buffers (optionally only on `shard`, a range of the flat index space)."""
        P = self.params
        self.step_count += 1
        lr = self.lr if lr is None else lr
        if grad_norm is None and self.max_grad_norm > 0:
            grad_norm = self.compute_grad_norm()
        lo, hi = (0, P.total) if shard is None else (shard.start, shard.stop)
        for a, b, wd in ((lo, min(hi, P.decay_end), self.weight_decay), (max(lo, P.decay_end), hi, 0.0)):
            if b <= a:
                continue
            ops.adam_step(P.master[a:b], P.m[a:b], P.v[a:b], P.grad[a:b], lr=lr, beta1=self.betas[0],
                          beta2=self.betas[1], eps=self.eps, weight_decay=wd, step=self.step_count, decoupled=True,
                          p_lowp=P.lowp[a:b] if P.lowp.dtype != torch.float32 else None,
                          max_grad_norm=self.max_grad_norm, grad_norm=grad_norm)
        if P.lowp.dtype == torch.float32:
            P.lowp[lo:hi].copy_(P.master[lo:hi])

    # ------------------------------------------------------------------------------------------ one step
    def train_step(self, ids: torch.Tensor, targets: torch.Tensor, total_tokens: int | None = None,
                   lr: float | None = None, do_step: bool = True) -> torch.Tensor:
        """ids / targets: int64 [N, S] on the device, N a multiple of micro_batch.  Returns the mean loss as a device
        scalar (sum over this rank's tokens / total_tokens)."""
        N = ids.shape[0]
        mb = min(self.micro_batch, N)
        assert N % mb == 0, "batch must be a multiple of the micro-batch"
        total_tokens = total_tokens or ids.numel()
        self.loss_acc.zero_()
        for i in range(0, N, mb):
            if self.use_graphs:
                self._forward_backward_graphed(ids[i:i + mb], targets[i:i + mb], 1.0 / total_tokens, i == 0)
            else:
                self.forward_backward(ids[i:i + mb], targets[i:i + mb], 1.0 / total_tokens, first_micro=(i == 0))
        if do_step:
            self.optimizer_step(lr)
        return ops.scalar_op("mul_scalar", self.loss_acc.view(1), 1.0 / total_tokens).view(())

    @torch.no_grad()
    def logits(self, ids: torch.Tensor) -> torch.Tensor:
        """Logits [B, S, vocab] (padding columns removed) for evaluation."""
        B, S = ids.shape
        return self.forward(ids)[:, :self.cfg.vocab_size].reshape(B, S, self.cfg.vocab_size)
