"""Recurrent cells (crates/nn/src/lstm.rs:10-470): LSTM (gate order i, f, o, g), GRU (standard equations: the reset gate
is used, which the reference computes and ignores, lstm.rs:203-300), stacked and bidirectional wrappers.

On the GPU (bf16) a step is the two projection GEMMs plus one fused gate kernel, in training as in inference: the gate
kernels of csrc/kernels/rnn.cu have backward counterparts, wrapped as autograd functions here, so the backward pass of
a step is one gate kernel plus the GEMMs' own dgrad / wgrad kernels.  CPU tensors use the tensor-op form."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N_
from .. import ops
from ..core import ForwardCtx, Module, Parameter, Saveable, StatefulModule, Trainable


_P, _LL, _I = N_.c_void_p, N_.c_ll, N_.c_int
N_.optional_sig("rb_lstm_gates_fwd", [_P, _LL, _P, _P, _P, _I, _I, _P])
N_.optional_sig("rb_lstm_gates_bwd", [_P, _LL, _P, _P, _P, _P, _P, _LL, _P, _I, _I, _P])
N_.optional_sig("rb_gru_gates_fwd", [_P, _LL, _P, _LL, _P, _P, _I, _I, _P])
N_.optional_sig("rb_gru_gates_bwd", [_P, _LL, _P, _LL, _P, _P, _P, _P, _P, _I, _I, _P])


_SEQ_GRAPHS = __import__("os").environ.get("RUSTRAL_RNN_GRAPHS", "1") != "0"


def _native_cell_ok(t: torch.Tensor, hidden: int) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and hidden % 2 == 0


class _LstmGatesFn(torch.autograd.Function):
    """(h, c) = cell update from the pre-activations [B, 4H] (order i | f | o | g) and c_prev, one kernel each way
    (`rb_lstm_gates_fwd` / `rb_lstm_gates_bwd`; the backward recomputes the activations from the saved pre-activations)."""

    @staticmethod
    def forward(ctx, gates, c_prev):
        gates, c_prev = gates.contiguous(), c_prev.contiguous()
        B, H = c_prev.shape
        h, c = torch.empty_like(c_prev), torch.empty_like(c_prev)
        N_.check(N_.kernels().rb_lstm_gates_fwd(gates.data_ptr(), gates.stride(0), c_prev.data_ptr(), h.data_ptr(), c.data_ptr(),
                                                B, H, N_.stream_ptr()), "rb_lstm_gates_fwd")
        ctx.save_for_backward(gates, c_prev, c)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        gates, c_prev, c = ctx.saved_tensors
        B, H = c_prev.shape
        dh = torch.zeros_like(c) if dh is None else dh.contiguous()
        dc = None if dc is None else dc.contiguous()
        dgates, dc_prev = torch.empty_like(gates), torch.empty_like(c_prev)
        N_.check(N_.kernels().rb_lstm_gates_bwd(gates.data_ptr(), gates.stride(0), c_prev.data_ptr(), c.data_ptr(), dh.data_ptr(),
                                                N_.ptr(dc), dgates.data_ptr(), dgates.stride(0), dc_prev.data_ptr(), B, H,
                                                N_.stream_ptr()), "rb_lstm_gates_bwd")
        return dgates, dc_prev


class _GruGatesFn(torch.autograd.Function):
    """h = GRU cell update from gx = x W_x^T + b, gh = h_prev W_h^T ([B, 3H], order r | z | n) and h_prev."""

    @staticmethod
    def forward(ctx, gx, gh, h_prev):
        gx, gh, h_prev = gx.contiguous(), gh.contiguous(), h_prev.contiguous()
        B, H = h_prev.shape
        h = torch.empty_like(h_prev)
        N_.check(N_.kernels().rb_gru_gates_fwd(gx.data_ptr(), gx.stride(0), gh.data_ptr(), gh.stride(0), h_prev.data_ptr(),
                                               h.data_ptr(), B, H, N_.stream_ptr()), "rb_gru_gates_fwd")
        ctx.save_for_backward(gx, gh, h_prev)
        return h

    @staticmethod
    def backward(ctx, dh):
        gx, gh, h_prev = ctx.saved_tensors
        B, H = h_prev.shape
        dgx, dgh, dhp = torch.empty((B, 3 * H), dtype=gx.dtype, device=gx.device), torch.empty((B, 3 * H), dtype=gx.dtype, device=gx.device), \
            torch.empty_like(h_prev)
        N_.check(N_.kernels().rb_gru_gates_bwd(gx.data_ptr(), gx.stride(0), gh.data_ptr(), gh.stride(0), h_prev.data_ptr(),
                                               dh.contiguous().data_ptr(), dgx.data_ptr(), dgh.data_ptr(), dhp.data_ptr(), B, H,
                                               N_.stream_ptr()), "rb_gru_gates_bwd")
        return dgx, dgh, dhp


@dataclass
class LstmConfig:
    input_size: int
    hidden_size: int


GruConfig = LstmConfig          # a GRU cell is configured by the same two sizes (crates/nn/src/lstm.rs:218-223)


class LstmState(tuple):
    """(hidden, cell) of an LSTM: what `LstmCell.step` returns and takes, with the reference's field names
    (crates/nn/src/lstm.rs:33-38).  It is a plain 2-tuple, so `h, c = state` keeps working."""

    def __new__(cls, hidden, cell):
        return super().__new__(cls, (hidden, cell))

    @property
    def hidden(self):
        return self[0]

    @property
    def cell(self):
        return self[1]


@dataclass
class GruState:
    """The hidden state of a GRU under the reference's name (crates/nn/src/lstm.rs:227-230); `GruCell` itself passes the
    bare tensor, `GruState(h).hidden` wraps and unwraps it."""
    hidden: torch.Tensor


@dataclass
class BidirectionalOutput:
    """Both directions of a bidirectional pass, time-aligned, and their concatenation (crates/nn/src/lstm.rs:417-424)."""
    forward: torch.Tensor
    backward: torch.Tensor
    concatenated: torch.Tensor


class RnnCell(Module, Trainable, Saveable, StatefulModule):
    hidden_size: int

    def step(self, x, state, ctx):
        raise NotImplementedError

    def hidden_of(self, state):
        return state

    def forward_sequence(self, xs, ctx: ForwardCtx, state=None):
        """xs: [T, B, I].  Returns (outputs [T, B, H], final state)."""
        if state is None:
            state = self.initial_state(xs.shape[1], ctx, xs)
        outs = []
        for t in range(xs.shape[0]):
            state = self.step(xs[t], state, ctx)
            outs.append(self.hidden_of(state))
        return torch.stack(outs), state


class LstmCell(RnnCell):
    """Parameters wx [4H, I], wh [4H, H], b [4H]; the two gate matmuls are one fused GEMM each."""

    def __init__(self, config: LstmConfig, wx: Parameter, wh: Parameter, b: Parameter):
        self.config, self.wx, self.wh, self.b = config, wx, wh, b
        self.hidden_size = config.hidden_size

    @classmethod
    def new(cls, backend, input_size: int, hidden_size: int, seed: int = 42):
        s = hidden_size ** -0.5
        return cls(LstmConfig(input_size, hidden_size), backend.uniform_parameter("wx", (4 * hidden_size, input_size), seed, s),
                   backend.uniform_parameter("wh", (4 * hidden_size, hidden_size), seed + 1, s),
                   backend.constant_parameter("b", (4 * hidden_size,), 0.0))

    def initial_state(self, batch: int, ctx=None, like=None):
        dev = self.wx.tensor.device
        z = torch.zeros(batch, self.hidden_size, dtype=self.wx.tensor.dtype, device=dev)
        return z, z.clone()

    def hidden_of(self, state):
        return state[0]

    def step(self, x, state, ctx=None):
        h, c = state
        H = self.hidden_size
        if _native_cell_ok(x, H):
            # training and inference on the GPU: two GEMMs (the second adds the first as its residual) and the gate kernel
            gates = ops.linear(h, self.wh.tensor, None, "none", ops.linear(x, self.wx.tensor, self.b.tensor))
            return _LstmGatesFn.apply(gates, c)
        gates = ops.linear(x, self.wx.tensor, self.b.tensor) + ops.linear(h, self.wh.tensor)
        gf = gates.float()
        i, f, o, g = torch.sigmoid(gf[:, :H]), torch.sigmoid(gf[:, H:2 * H]), torch.sigmoid(gf[:, 2 * H:3 * H]), torch.tanh(gf[:, 3 * H:])
        c2 = f * c.float() + i * g
        h2 = o * torch.tanh(c2)
        return h2.to(x.dtype), c2.to(x.dtype)

    def forward(self, x_state, ctx=None):
        x, state = x_state
        return self.step(x, state, ctx)

    def forward_sequence(self, xs, ctx: ForwardCtx, state=None):
        """Inference on the GPU: the input projections of ALL steps are one GEMM, and a step is one GEMM (h W_h^T with
        that projection as its residual) plus the fused gate kernel.  With gradients, or on the CPU: the generic loop."""
        needs_grad = torch.is_grad_enabled() and (xs.requires_grad or (ctx is not None and ctx.is_training()))
        H = self.hidden_size
        if not xs.is_cuda or xs.dtype != torch.bfloat16 or needs_grad or H % 8:
            return super().forward_sequence(xs, ctx, state)
        T, B, I = xs.shape
        with torch.no_grad():
            h, c = state if state is not None else self.initial_state(B, ctx, xs)
            if T >= 4 and _SEQ_GRAPHS and not torch.cuda.is_current_stream_capturing():
                return self._graphed_sequence(xs, h, c)
            return self._sequence_body(xs, h.contiguous(), c.contiguous().clone())

    def _sequence_body(self, xs, h, c):
        """One input-projection GEMM for all steps, then per step one GEMM (with that projection as its residual) and the
        fused gate kernel; `c` is updated in place."""
        T, B, I = xs.shape
        H = self.hidden_size
        lib = N_.kernels()
        wx, wh, bias = self.wx.tensor.detach(), self.wh.tensor.detach(), self.b.tensor.detach()
        xproj = ops.linear(xs.reshape(T * B, I).contiguous(), wx, bias).view(T, B, 4 * H)
        outs = torch.empty((T, B, H), dtype=xs.dtype, device=xs.device)
        for t in range(T):
            gates = ops.linear(h, wh, None, "none", xproj[t])
            N_.check(lib.rb_lstm_gates_fwd(gates.data_ptr(), gates.stride(0), c.data_ptr(), outs[t].data_ptr(), c.data_ptr(),
                                           B, H, N_.stream_ptr()), "rb_lstm_gates_fwd")
            h = outs[t]
        return outs, (h, c)

    def _graphed_sequence(self, xs, h0, c0):
        """A sequence is 2 T + 1 small launches, each of which costs more on the host than on the device: the second call
        with the same shapes and weights captures them into a CUDA graph, later calls copy the inputs into the graph's
        static tensors and replay it (`RUSTRAL_RNN_GRAPHS=0` turns this off)."""
        key = (tuple(xs.shape), xs.device.index, self.wx.tensor.data_ptr(), self.wh.tensor.data_ptr(), self.b.tensor.data_ptr())
        graphs = self.__dict__.setdefault("_seq_graphs", {})
        g = graphs.get(key)
        if g is None:
            graphs[key] = {"graph": None}                     # first use: run eagerly (kernels configure themselves lazily)
            return self._sequence_body(xs, h0.contiguous(), c0.contiguous().clone())
        if g["graph"] is None:
            g["xs"], g["h0"], g["c0"] = torch.empty_like(xs), torch.empty_like(h0), torch.empty_like(c0)
            g["xs"].copy_(xs); g["h0"].copy_(h0); g["c0"].copy_(c0)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                c_work = g["c0"].clone()
                g["outs"], (g["h"], g["c"]) = self._sequence_body(g["xs"], g["h0"], c_work)
            g["graph"] = graph
        g["xs"].copy_(xs); g["h0"].copy_(h0); g["c0"].copy_(c0)
        g["graph"].replay()
        return g["outs"].clone(), (g["h"].clone(), g["c"].clone())


class GruCell(RnnCell):
    def __init__(self, config: LstmConfig, wx: Parameter, wh: Parameter, b: Parameter):
        self.config, self.wx, self.wh, self.b = config, wx, wh, b
        self.hidden_size = config.hidden_size

    @classmethod
    def new(cls, backend, input_size: int, hidden_size: int, seed: int = 42):
        s = hidden_size ** -0.5
        return cls(LstmConfig(input_size, hidden_size), backend.uniform_parameter("wx", (3 * hidden_size, input_size), seed, s),
                   backend.uniform_parameter("wh", (3 * hidden_size, hidden_size), seed + 1, s),
                   backend.constant_parameter("b", (3 * hidden_size,), 0.0))

    def initial_state(self, batch: int, ctx=None, like=None):
        return torch.zeros(batch, self.hidden_size, dtype=self.wx.tensor.dtype, device=self.wx.tensor.device)

    def step(self, x, h, ctx=None):
        H = self.hidden_size
        if _native_cell_ok(x, H):
            return _GruGatesFn.apply(ops.linear(x, self.wx.tensor, self.b.tensor), ops.linear(h, self.wh.tensor), h)
        gx = ops.linear(x, self.wx.tensor, self.b.tensor).float()
        gh = ops.linear(h, self.wh.tensor).float()
        r = torch.sigmoid(gx[:, :H] + gh[:, :H])
        z = torch.sigmoid(gx[:, H:2 * H] + gh[:, H:2 * H])
        n = torch.tanh(gx[:, 2 * H:] + r * gh[:, 2 * H:])
        return ((1 - z) * n + z * h.float()).to(x.dtype)

    def forward(self, x_state, ctx=None):
        x, h = x_state
        return self.step(x, h, ctx)

    def forward_sequence(self, xs, ctx: ForwardCtx, state=None):
        """Inference: the input projections of all steps are one GEMM, so a step is one GEMM plus the gate arithmetic
        (on the GPU: the fused gate kernel, and from the second call on a CUDA-graph replay of the whole sequence).
        With gradients: the generic loop."""
        needs_grad = torch.is_grad_enabled() and (xs.requires_grad or (ctx is not None and ctx.is_training()))
        if needs_grad:
            return super().forward_sequence(xs, ctx, state)
        T, B, I = xs.shape
        H = self.hidden_size
        with torch.no_grad():
            h = state if state is not None else self.initial_state(B, ctx, xs)
            if _native_cell_ok(xs, H) and H % 8 == 0:
                if T >= 4 and _SEQ_GRAPHS and not torch.cuda.is_current_stream_capturing():
                    return self._graphed_sequence(xs, h)
                return self._sequence_body(xs, h.contiguous())
            wx, wh, b = self.wx.tensor.detach(), self.wh.tensor.detach(), self.b.tensor.detach()
            gx_all = ops.linear(xs.reshape(T * B, I).contiguous(), wx, b).view(T, B, 3 * H).float()
            outs = torch.empty((T, B, H), dtype=xs.dtype, device=xs.device)
            for t in range(T):
                gx, gh = gx_all[t], ops.linear(h, wh).float()
                r = torch.sigmoid(gx[:, :H] + gh[:, :H])
                z = torch.sigmoid(gx[:, H:2 * H] + gh[:, H:2 * H])
                n = torch.tanh(gx[:, 2 * H:] + r * gh[:, 2 * H:])
                h = ((1 - z) * n + z * h.float()).to(xs.dtype)
                outs[t] = h
        return outs, h

    def _sequence_body(self, xs, h):
        """GPU inference: one input-projection GEMM for all steps, then per step the hidden projection GEMM and the fused
        gate kernel, which writes the new hidden state straight into the output sequence."""
        T, B, I = xs.shape
        H = self.hidden_size
        lib = N_.kernels()
        wx, wh, bias = self.wx.tensor.detach(), self.wh.tensor.detach(), self.b.tensor.detach()
        gx_all = ops.linear(xs.reshape(T * B, I).contiguous(), wx, bias).view(T, B, 3 * H)
        outs = torch.empty((T, B, H), dtype=xs.dtype, device=xs.device)
        for t in range(T):
            gh = ops.linear(h, wh)
            N_.check(lib.rb_gru_gates_fwd(gx_all[t].data_ptr(), gx_all[t].stride(0), gh.data_ptr(), gh.stride(0), h.data_ptr(),
                                          outs[t].data_ptr(), B, H, N_.stream_ptr()), "rb_gru_gates_fwd")
            h = outs[t]
        return outs, h

    def _graphed_sequence(self, xs, h0):
        """Same scheme as the LSTM's: eager on first use, captured on the second call with the same shapes and weights,
        replayed afterwards (`RUSTRAL_RNN_GRAPHS=0` turns it off)."""
        key = (tuple(xs.shape), xs.device.index, self.wx.tensor.data_ptr(), self.wh.tensor.data_ptr(), self.b.tensor.data_ptr())
        graphs = self.__dict__.setdefault("_seq_graphs", {})
        g = graphs.get(key)
        if g is None:
            graphs[key] = {"graph": None}
            return self._sequence_body(xs, h0.contiguous())
        if g["graph"] is None:
            g["xs"], g["h0"] = torch.empty_like(xs), torch.empty_like(h0.contiguous())
            g["xs"].copy_(xs); g["h0"].copy_(h0)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g["outs"], g["h"] = self._sequence_body(g["xs"], g["h0"])
            g["graph"] = graph
        g["xs"].copy_(xs); g["h0"].copy_(h0)
        g["graph"].replay()
        outs = g["outs"].clone()
        return outs, outs[-1]


class StackedLstm(Module, Trainable, Saveable):
    def __init__(self, cells: list):
        self.layers = cells

    @classmethod
    def new(cls, backend, input_size: int, hidden_size: int, num_layers: int, seed: int = 42):
        return cls([LstmCell.new(backend, input_size if i == 0 else hidden_size, hidden_size, seed + 10 * i)
                    for i in range(num_layers)])

    def forward_sequence(self, xs, ctx: ForwardCtx, states=None):
        finals = []
        for i, cell in enumerate(self.layers):
            xs, st = cell.forward_sequence(xs, ctx, None if states is None else states[i])
            finals.append(st)
        return xs, finals

    forward = forward_sequence


class BidirectionalRnn(Module, Trainable, Saveable):
    """Forward and backward passes over the sequence; outputs concatenated along the feature dimension."""

    def __init__(self, fwd: RnnCell, bwd: RnnCell):
        self.fwd, self.bwd = fwd, bwd

    def forward_sequence(self, xs, ctx: ForwardCtx):
        of, sf = self.fwd.forward_sequence(xs, ctx)
        ob, sb = self.bwd.forward_sequence(torch.flip(xs, (0,)), ctx)
        return torch.cat([of, torch.flip(ob, (0,))], -1), (sf, sb)

    forward = forward_sequence

    def forward_directions(self, xs, ctx: ForwardCtx) -> BidirectionalOutput:
        """The same pass with the two directions kept apart (the backward one re-aligned to the input's time order)."""
        of, _ = self.fwd.forward_sequence(xs, ctx)
        ob, _ = self.bwd.forward_sequence(torch.flip(xs, (0,)), ctx)
        ob = torch.flip(ob, (0,))
        return BidirectionalOutput(of, ob, torch.cat([of, ob], -1))

    def final_hidden(self, xs, ctx: ForwardCtx):
        _, (sf, sb) = self.forward_sequence(xs, ctx)
        return torch.cat([self.fwd.hidden_of(sf), self.bwd.hidden_of(sb)], -1)
