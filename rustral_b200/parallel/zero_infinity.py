"""ZeRO-Infinity style offload of optimizer state (crates/distributed/src/zero_infinity.rs).

Adam moments and fp32 master weights live in pinned host memory (optionally spilled to an NVMe-backed file) and
are streamed to the GPU one parameter at a time, with the next parameter's state prefetched on a side stream while
the current one is updated.  The update is the fused Adam kernel with the standard bias correction (the
reference's hand-rolled update multiplies sqrt(v) by sqrt(bc2), and its NVMe load discards what it reads)."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .. import ops


class StorageLocation:
    GPU, CPU, NVME = "gpu", "cpu", "nvme"


@dataclass
class ZeroInfinityConfig:
    cpu_offload: bool = True
    nvme_offload: bool = False
    nvme_path: str = "/tmp/rustral_b200_nvme"
    nvme_quota: int = 100 << 30
    prefetch_depth: int = 1
    pin_memory: bool = True


class _State:
    def __init__(self, p, cfg):
        n = p.numel()
        pin = cfg.pin_memory and torch.cuda.is_available()
        mk = lambda: torch.zeros(n, dtype=torch.float32, pin_memory=pin)
        self.m, self.v = mk(), mk()
        self.master = torch.empty(n, dtype=torch.float32, pin_memory=pin)
        self.master.copy_(p.tensor.detach().float().reshape(-1))
        self.t = 0
        self.location = StorageLocation.CPU
        self.nvme_offset = -1


class ZeroInfinity:
    def __init__(self, config: ZeroInfinityConfig | None = None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0):
        self.config = config or ZeroInfinityConfig()
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.states: dict = {}
        self._nvme_file = None
        self._nvme_used = 0

    def register_parameters(self, params) -> None:
        for p in params:
            self.states[p.id] = _State(p, self.config)

    # ---- NVMe spill -------------------------------------------------------------------------------------------------
    def _file(self):
        if self._nvme_file is None:
            os.makedirs(os.path.dirname(self.config.nvme_path) or ".", exist_ok=True)
            self._nvme_file = open(self.config.nvme_path, "w+b")
        return self._nvme_file

    def save_to_nvme(self, pid) -> None:
        st = self.states[pid]
        blob = torch.cat([st.m, st.v, st.master]).numpy().tobytes()
        if self._nvme_used + len(blob) > self.config.nvme_quota:
            raise RuntimeError("NVMe quota exceeded")
        f = self._file()
        if st.nvme_offset < 0:
            st.nvme_offset = self._nvme_used
            self._nvme_used += len(blob)
        f.seek(st.nvme_offset)
        f.write(blob)
        f.flush()
        n = st.m.numel()
        st.m = st.v = st.master = None
        st.location = StorageLocation.NVME
        st._n = n

    def load_from_nvme(self, pid) -> None:
        import numpy as np
        st = self.states[pid]
        if st.location != StorageLocation.NVME:
            return
        f = self._file()
        f.seek(st.nvme_offset)
        arr = np.frombuffer(f.read(st._n * 12), dtype=np.float32).copy()
        t = torch.from_numpy(arr)
        st.m, st.v, st.master = t[:st._n].clone(), t[st._n:2 * st._n].clone(), t[2 * st._n:].clone()
        st.location = StorageLocation.CPU

    # ---- step ----------------------------------------------------------------------------------------------------------
    def step(self, params) -> None:
        params = [p for p in params if p.tensor.grad is not None]
        cuda = bool(params) and params[0].tensor.is_cuda
        side = torch.cuda.Stream() if cuda else None

        def fetch(p):
            st = self.states[p.id]
            self.load_from_nvme(p.id)
            if not cuda:
                return st.m, st.v, st.master, None
            with torch.cuda.stream(side):
                bufs = [x.to(p.tensor.device, non_blocking=True) for x in (st.m, st.v, st.master)]
                ev = torch.cuda.Event()
                ev.record(side)
            return (*bufs, ev)

        nxt = fetch(params[0]) if params else None
        for i, p in enumerate(params):
            m, v, master, ev = nxt
            nxt = fetch(params[i + 1]) if i + 1 < len(params) else None     # prefetch overlaps this update
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            st = self.states[p.id]
            st.t += 1
            lowp = p.tensor.view(-1) if p.tensor.dtype == torch.bfloat16 else None
            ops.adam_step(master, m, v, p.tensor.grad.contiguous().view(-1), lr=self.lr, beta1=self.betas[0],
                          beta2=self.betas[1], eps=self.eps, weight_decay=self.weight_decay, step=st.t, decoupled=True,
                          p_lowp=lowp)
            with torch.no_grad():
                if lowp is None:
                    p.tensor.copy_(master.view(p.shape).to(p.tensor.dtype))
            if cuda:
                st.m.copy_(m, non_blocking=True)
                st.v.copy_(v, non_blocking=True)
                st.master.copy_(master, non_blocking=True)
            if self.config.nvme_offload:
                if cuda:
                    torch.cuda.current_stream().synchronize()
                self.save_to_nvme(p.id)
        if cuda:
            torch.cuda.current_stream().synchronize()

    def memory_stats(self) -> "ZeroInfinityStats":
        host = sum(3 * s.m.numel() * 4 for s in self.states.values() if s.location == StorageLocation.CPU)
        where = [s.location for s in self.states.values()]
        total = sum((s.m.numel() if s.m is not None else getattr(s, "_n", 0)) for s in self.states.values())
        return ZeroInfinityStats(total, where.count(StorageLocation.GPU), where.count(StorageLocation.CPU),
                                 where.count(StorageLocation.NVME), self._nvme_used, host)


@dataclass
class ZeroInfinityStats:
    """Where the optimizer states live (crates/distributed/src/zero_infinity.rs:504-527), plus the host bytes.  Compares
    equal to, and indexes like, the dictionary {"host_bytes", "nvme_bytes", "gpu_bytes"}."""
    total_params: int
    gpu_states: int
    cpu_states: int
    nvme_states: int
    nvme_bytes_used: int
    host_bytes: int = 0

    def as_dict(self) -> dict:
        return {"host_bytes": self.host_bytes, "nvme_bytes": self.nvme_bytes_used, "gpu_bytes": 0}

    def __getitem__(self, key):
        return self.as_dict()[key]

    def __eq__(self, other):
        if isinstance(other, dict):
            return self.as_dict() == other
        return isinstance(other, ZeroInfinityStats) and vars(self) == vars(other)


@dataclass
class ZeROMemoryEstimate:
    """crates/distributed/src/zero_infinity.rs:566-575 (bytes)."""
    model_memory: int
    optimizer_states: int
    gradient_memory: int
    gpu_memory: int
    cpu_memory: int
    nvme_memory: int
    total_memory: int


class ZeROInfinityEstimator:
    @staticmethod
    def estimate(num_params: int, world: int = 1) -> dict:
        return {"gpu_bytes": 2 * num_params + 4 * num_params, "host_bytes": 12 * num_params // world}

    @staticmethod
    def estimate_for(model_params: int, param_size_bytes: int, config: "ZeroInfinityConfig") -> ZeROMemoryEstimate:
        """The reference's estimate: parameters and gradients on the GPU, Adam's two moments on the host and / or on
        NVMe according to the configuration."""
        model = model_params * param_size_bytes
        opt = 2 * model
        gpu = 2 * model
        cpu = opt if config.cpu_offload else 0
        nvme = opt if config.nvme_offload else 0
        return ZeROMemoryEstimate(model, opt, model, gpu, cpu, nvme, gpu + cpu + nvme)
