"""DeviceMesh: n-dimensional rank layout with wildcard sub-group selection (crates/distributed/src/device_mesh.rs:32-287).

Row-major rank <-> coordinate mapping, last dimension fastest.  For 3-D parallelism the conventional shape is
[dp, pp, tp] with tensor parallelism innermost, so that a TP group is a run of adjacent ranks (on one node every
pair is one NVSwitch hop apart anyway; across nodes it keeps TP inside a node).  `for_3d_parallelism` builds that
order; the reference's [dp, tp, pp] order puts pipeline stages on adjacent ranks instead.
"""
from __future__ import annotations

from dataclasses import dataclass

from .process_group import DistributedError, ProcessGroup


class DeviceMesh:
    def __init__(self, shape, my_rank: int, dim_names=None):
        self.shape = tuple(int(s) for s in shape)
        if any(s <= 0 for s in self.shape):
            raise DistributedError("mesh dimensions must be positive")
        self.world_size = 1
        for s in self.shape:
            self.world_size *= s
        if not (0 <= my_rank < self.world_size):
            raise DistributedError(f"rank {my_rank} outside a mesh of {self.world_size}")
        self.my_rank = my_rank
        self.dim_names = tuple(dim_names) if dim_names else tuple(f"dim{i}" for i in range(len(self.shape)))
        self.my_coord = self.coord_of(my_rank)
        self._groups: dict = {}

    def coord_of(self, rank: int) -> tuple:
        c = []
        for s in reversed(self.shape):
            c.append(rank % s)
            rank //= s
        return tuple(reversed(c))

    def rank_of(self, coord) -> int:
        r = 0
        for c, s in zip(coord, self.shape):
            if not (0 <= c < s):
                raise DistributedError(f"coordinate {coord} outside mesh {self.shape}")
            r = r * s + c
        return r

    def matching_ranks(self, pattern) -> list:
        """Ranks whose coordinates match `pattern`; -1 is a wildcard."""
        if len(pattern) != len(self.shape):
            raise DistributedError("pattern rank differs from mesh rank")
        return [r for r in range(self.world_size)
                if all(p == -1 or p == c for p, c in zip(pattern, self.coord_of(r)))]

    def group_ranks_along(self, dim: int) -> list:
        """The ranks that differ from this one only in dimension `dim`."""
        pat = list(self.my_coord)
        pat[dim] = -1
        return self.matching_ranks(pat)

    def all_groups_along(self, dim: int) -> list:
        seen, out = set(), []
        for r in range(self.world_size):
            pat = list(self.coord_of(r))
            pat[dim] = -1
            key = tuple(pat)
            if key not in seen:
                seen.add(key)
                out.append(self.matching_ranks(pat))
        return out

    def get_process_group(self, dim, factory=None) -> ProcessGroup:
        """Sub-group along `dim` (index or name).  With torch.distributed every rank must call this for the same
        dimensions in the same order (new_group is collective); `factory(ranks) -> ProcessGroup` overrides creation."""
        if isinstance(dim, str):
            dim = self.dim_names.index(dim)
        if dim in self._groups:
            return self._groups[dim]
        mine = None
        for ranks in self.all_groups_along(dim):
            if factory is not None:
                g = factory(ranks) if self.my_rank in ranks else None
            elif len(ranks) == 1 and self.my_rank in ranks:
                g = ProcessGroup.new_single_process()
            else:
                g = ProcessGroup.new_torch_subgroup(ranks)
            if self.my_rank in ranks:
                mine = g
        self._groups[dim] = mine
        return mine

    @classmethod
    def for_3d_parallelism(cls, dp: int, tp: int, pp: int, rank: int) -> "DeviceMesh":
        return cls((dp, pp, tp), rank, ("dp", "pp", "tp"))

    def get_data_parallel_group(self, **kw):
        return self.get_process_group("dp", **kw)

    def get_tensor_parallel_group(self, **kw):
        return self.get_process_group("tp", **kw)

    def get_pipeline_parallel_group(self, **kw):
        return self.get_process_group("pp", **kw)


@dataclass
class ParallelismConfig:
    dp: int
    tp: int
    pp: int

    @classmethod
    def auto_select(cls, num_gpus: int, num_params: int) -> "ParallelismConfig":
        """tp = min(8, gpus/2) above 1B parameters, pp = min(8, rest/2) above 10B, dp = the rest
        (crates/distributed/src/device_mesh.rs:261-287)."""
        tp = pp = 1
        rem = num_gpus
        if num_params > 1_000_000_000 and rem >= 2:
            tp = max(1, min(8, rem // 2))
            while rem % tp:
                tp -= 1
            rem //= tp
        if num_params > 10_000_000_000 and rem >= 2:
            pp = max(1, min(8, rem // 2))
            while rem % pp:
                pp -= 1
            rem //= pp
        return cls(rem, tp, pp)

    def total_gpus(self) -> int:
        return self.dp * self.tp * self.pp
