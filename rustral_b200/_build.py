"""In-tree build of the native libraries.

Three shared objects are produced under ``rustral_b200/_lib``:

* ``librb200_kernels.so`` -- every ``csrc/kernels/*.cu`` and ``csrc/comm/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); plain ``extern "C"`` entry points.
* ``librb200_cpu.so``     -- the C++ f32 reference backend (``csrc/cpu/*.cpp``), the numerical oracle.
* ``librb200_runtime.so`` -- host runtime pieces in C++ (``csrc/runtime/*.cpp``): paged-KV block
  allocator, request scheduler core, tile-config search, data loader.

The libraries are bound with ctypes, so no torch headers are compiled and a full rebuild takes well
under a minute on a CPU-only machine (nvcc cross-compiles without a GPU).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v2", "-Wall", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _newer(target: Path, deps) -> bool:
    """True when `target` exists and is newer than every dependency."""
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), file=sys.stderr)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build command failed: {' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    return res


def _compile_group(sources, headers, out_lib: Path, compiler_cmd, link_cmd, verbose, force):
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    objs = []
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (out_lib.stem + "__" + src.stem + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src, *headers]):
            jobs.append(compiler_cmd(src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or not _newer(out_lib, objs):
        _run(link_cmd(objs, out_lib), verbose)
    return out_lib


def build_kernels(force: bool = False, verbose: bool = False, bounds: bool = False) -> Path:
    """`bounds`: the checking variant ``librb200_kernels_bounds.so`` (-DRB_BOUNDS: every kernel that reads indices from
    memory reports an out-of-range one through the status word; it never traps).  `RUSTRAL_BOUNDS=1` makes the package
    load that variant."""
    srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.h")) + sorted((CSRC / "kernels").glob("*.cuh")) + \
        sorted((CSRC / "comm").glob("*.h")) + sorted((CSRC / "comm").glob("*.cuh"))
    nvcc = _nvcc()
    inc = ["-I", str(CSRC / "kernels"), "-I", str(CSRC / "comm")]
    extra = ["-DRB_BOUNDS"] if bounds else []
    return _compile_group(
        srcs, hdrs, LIB_DIR / ("librb200_kernels_bounds.so" if bounds else "librb200_kernels.so"),
        lambda s, o: [nvcc, *NVCC_FLAGS, *extra, *inc, "-c", s, "-o", o],
        lambda objs, out: [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", out],
        verbose, force)


def _build_cxx(subdir: str, libname: str, force: bool, verbose: bool) -> Path:
    srcs = sorted((CSRC / subdir).glob("*.cpp"))
    hdrs = sorted((CSRC / subdir).glob("*.h")) + sorted((CSRC / subdir).glob("*.hpp"))
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    inc = ["-I", str(CSRC / subdir)]
    return _compile_group(
        srcs, hdrs, LIB_DIR / libname,
        lambda s, o: [cxx, *CXX_FLAGS, *inc, "-c", s, "-o", o],
        lambda objs, out: [cxx, "-shared", "-pthread", *objs, "-o", out],
        verbose, force)


def build_cpu(force: bool = False, verbose: bool = False) -> Path:
    return _build_cxx("cpu", "librb200_cpu.so", force, verbose)


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    return _build_cxx("runtime", "librb200_runtime.so", force, verbose)


def build_all(force: bool = False, verbose: bool = False) -> dict:
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = {}
    out["kernels"] = build_kernels(force, verbose)
    out["kernels_bounds"] = build_kernels(force, verbose, bounds=True)
    if any((CSRC / "cpu").glob("*.cpp")):
        out["cpu"] = build_cpu(force, verbose)
    if any((CSRC / "runtime").glob("*.cpp")):
        out["runtime"] = build_runtime(force, verbose)
    return out


if __name__ == "__main__":
    built = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in built.items():
        print(f"{k}: {v}")
