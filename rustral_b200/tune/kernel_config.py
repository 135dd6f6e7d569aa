"""Structured kernel configurations (crates/autotuner/src/kernel_config.rs:9-420): dimension buckets, launch shape,
tile shape, algorithm choice, on-chip memory use, and `KernelConfig`, which bundles them with free integer parameters.

The defaults describe the sm_100a kernels of this package rather than the reference's WGSL ones: a GEMM CTA is 320
threads (one TMA warp, one MMA warp, eight epilogue warps) with 128 x 256 x 64 tiles in about 200 KB of shared memory;
attention CTAs hold two 128-row query tiles; reductions are two-pass so that results do not depend on scheduling.
`KernelConfig.to_gemm_plan()` turns a matmul configuration into the `block_n / splits / group_m` plan `ops.gemm` takes,
so a configuration found by a search over this space can be applied to the real kernel."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from . import ConvAlgorithm, MatmulAlgorithm, ReduceAlgorithm


class MatmulDimBucket(enum.Enum):
    """Tiny < 256, Small <= 512, Medium < 2048, Large < 8192, XLarge."""
    TINY = "Tiny"
    SMALL = "Small"
    MEDIUM = "Medium"
    LARGE = "Large"
    XLARGE = "XLarge"

    @classmethod
    def from_size(cls, size: int) -> "MatmulDimBucket":
        if size < 256:
            return cls.TINY
        if size <= 512:
            return cls.SMALL
        if size < 2048:
            return cls.MEDIUM
        if size < 8192:
            return cls.LARGE
        return cls.XLARGE

    def __str__(self) -> str:
        return self.value


@dataclass(frozen=True)
class WorkgroupConfig:
    """Threads of one CTA along x, y, z."""
    x: int = 256
    y: int = 1
    z: int = 1

    def total_threads(self) -> int:
        return self.x * self.y * self.z

    def is_valid(self) -> bool:
        return 0 < self.total_threads() <= 1024


@dataclass(frozen=True)
class BlockSize:
    """Tile of a GEMM-shaped kernel.  The tcgen05 path takes m in {128, 256 on a CTA pair}, n a multiple of 64 up to 256,
    k = 64 (one 128-byte swizzle row of bf16)."""
    m: int
    n: int
    k: int

    @classmethod
    def square(cls, size: int) -> "BlockSize":
        return cls(size, size, size)

    def is_valid(self) -> bool:
        return 0 < self.m <= 256 and 0 < self.n <= 256 and 0 < self.k <= 64

    def is_tcgen05_tile(self) -> bool:
        return self.m in (128, 256) and self.n in (64, 128, 192, 256) and self.k == 64


class CacheConfig(enum.Enum):
    DEFAULT = "default"
    PREFER_L1 = "prefer_l1"
    PREFER_SHARED = "prefer_shared"
    EQUAL = "equal"


@dataclass(frozen=True)
class MemoryConfig:
    use_shared: bool = True
    shared_size_bytes: int = 16384
    vector_width: int = 4
    cache_config: CacheConfig = CacheConfig.DEFAULT

    def fits_sm100(self) -> bool:
        """At most 227 KB of shared memory per CTA."""
        return self.shared_size_bytes <= 227 * 1024


@dataclass(frozen=True)
class AlgorithmConfig:
    """Tagged choice: kind is matmul / conv / reduce / elementwise / attention / custom; `value` is the algorithm
    member, the attention settings (use_flash, block_size_m, block_size_n) or the custom name."""
    kind: str
    value: object = None

    @classmethod
    def matmul(cls, a: MatmulAlgorithm):
        return cls("matmul", a)

    @classmethod
    def conv(cls, a: ConvAlgorithm):
        return cls("conv", a)

    @classmethod
    def reduce(cls, a: ReduceAlgorithm):
        return cls("reduce", a)

    @classmethod
    def elementwise(cls):
        return cls("elementwise")

    @classmethod
    def attention(cls, use_flash: bool = True, block_size_m: int = 128, block_size_n: int = 128):
        return cls("attention", (bool(use_flash), int(block_size_m), int(block_size_n)))

    @classmethod
    def custom(cls, name: str):
        return cls("custom", str(name))


@dataclass
class KernelConfig:
    workgroup: WorkgroupConfig = field(default_factory=WorkgroupConfig)
    algorithm: AlgorithmConfig = field(default_factory=AlgorithmConfig.elementwise)
    memory: MemoryConfig = field(default_factory=MemoryConfig)
    params: dict = field(default_factory=dict)

    @classmethod
    def default_for(cls, op: str) -> "KernelConfig":
        make = {"matmul": cls.default_matmul, "conv2d": cls.default_conv2d, "reduce": cls.default_reduce,
                "elementwise": cls.default_elementwise, "attention": cls.default_attention}.get(op)
        return make() if make else cls()

    @classmethod
    def default_matmul(cls):
        return cls(WorkgroupConfig(320, 1, 1), AlgorithmConfig.matmul(MatmulAlgorithm.TCGEN05_ONE_CTA),
                   MemoryConfig(True, 200 * 1024, 8, CacheConfig.PREFER_SHARED),
                   {"tile_m": 128, "tile_n": 256, "tile_k": 64, "stages": 4, "splits": 0, "group_m": 8})

    @classmethod
    def default_conv2d(cls):
        return cls(WorkgroupConfig(256, 1, 1), AlgorithmConfig.conv(ConvAlgorithm.IMPLICIT_GEMM),
                   MemoryConfig(True, 200 * 1024, 8, CacheConfig.PREFER_SHARED), {"tile_h": 4, "tile_w": 4, "tile_c": 32})

    @classmethod
    def default_reduce(cls):
        return cls(WorkgroupConfig(256, 1, 1), AlgorithmConfig.reduce(ReduceAlgorithm.TWO_PASS),
                   MemoryConfig(True, 4096, 8, CacheConfig.DEFAULT), {"items_per_thread": 8, "unroll": 1})

    @classmethod
    def default_elementwise(cls):
        return cls(WorkgroupConfig(256, 1, 1), AlgorithmConfig.elementwise(), MemoryConfig(False, 0, 8, CacheConfig.DEFAULT),
                   {"items_per_thread": 8, "vectorize": 1})

    @classmethod
    def default_attention(cls):
        return cls(WorkgroupConfig(384, 1, 1), AlgorithmConfig.attention(True, 128, 128),
                   MemoryConfig(True, 196 * 1024, 8, CacheConfig.PREFER_SHARED), {"softmax_scale": 1, "use_causal_mask": 1})

    def is_valid(self) -> bool:
        return self.workgroup.is_valid() and self.memory.fits_sm100()

    def block_size(self) -> BlockSize | None:
        p = self.params
        if {"tile_m", "tile_n", "tile_k"} <= set(p):
            return BlockSize(p["tile_m"], p["tile_n"], p["tile_k"])
        return None

    def to_gemm_plan(self) -> dict:
        """The plan `ops.gemm` takes (`block_n`, `splits`, `group_m`; 0 leaves a choice to the kernel's cost model).
        Tile widths the tcgen05 kernel does not have are rounded to the nearest one it has."""
        if self.algorithm.kind != "matmul":
            raise ValueError("to_gemm_plan: not a matmul configuration")
        want = int(self.params.get("tile_n", 0))
        bn = min((64, 128, 192, 256), key=lambda c: abs(c - want)) if want else 0
        return {"block_n": bn, "splits": int(self.params.get("splits", 0)), "group_m": int(self.params.get("group_m", 0))}

    def cache_key(self) -> str:
        alg = self.algorithm.value
        alg = alg.value if isinstance(alg, enum.Enum) else alg
        params = ",".join(f"{k}={v}" for k, v in sorted(self.params.items()))
        return f"{self.algorithm.kind}:{alg}|wg={self.workgroup.x}x{self.workgroup.y}x{self.workgroup.z}|smem={self.memory.shared_size_bytes}|{params}"
