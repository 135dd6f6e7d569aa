"""ctypes bindings of the in-tree native libraries.

``kernels()`` returns the sm_100a kernel library.  It never falls back silently: when a CUDA device
is present and the library is missing or fails to load, the call raises, so a GPU run cannot pass on
an eager PyTorch path by accident.  ``cpu()`` / ``runtime()`` return the C++ reference backend and
the host runtime library (built on demand with g++ when absent, since they need no GPU toolchain).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

LIB_DIR = Path(__file__).resolve().parent / "_lib"
_lock = threading.Lock()
_libs: dict = {}

c_void_p, c_int, c_ll, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class RbGemmArgs(C.Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("d", c_void_p), ("bias", c_void_p), ("residual", c_void_p),
        ("aux_in", c_void_p), ("aux_out", c_void_p),
        ("lda", c_ll), ("ldb", c_ll), ("ldd", c_ll), ("ldr", c_ll), ("ld_aux_in", c_ll), ("ld_aux_out", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("a_mn_major", c_int), ("b_mn_major", c_int),
        ("act", c_int), ("out_f32", c_int), ("accumulate", c_int),
        ("alpha", c_float),
        ("block_n", c_int), ("group_m", c_int), ("max_ctas", c_int), ("splits", c_int),
        ("workspace", c_void_p), ("workspace_bytes", c_ll),
        ("group_mode", c_int), ("num_experts", c_int), ("tile_expert", c_void_p), ("num_m_tiles", c_void_p),
        ("expert_offsets", c_void_p), ("b_expert_rows", c_int), ("d_expert_stride", c_ll),
        ("peer_mode", c_int), ("peer_world", c_int), ("peer_rank", c_int), ("rows_per_rank", c_int),
        ("peer_epoch", C.c_uint), ("ready_flags", c_void_p), ("peer_ptrs", c_void_p * 8),
        ("tile_arrived", c_void_p), ("tile_expected", c_void_p),
        ("ab_fp8", c_int), ("a_scale", c_void_p), ("b_scale", c_void_p),
    ]


class RbAttnArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("d_o", c_void_p),
        ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("lse", c_void_p), ("delta", c_void_p),
        ("q_strides", c_ll * 3), ("k_strides", c_ll * 3), ("v_strides", c_ll * 3), ("o_strides", c_ll * 3),
        ("dq_strides", c_ll * 3), ("dk_strides", c_ll * 3), ("dv_strides", c_ll * 3),
        ("batch", c_int), ("heads", c_int), ("kv_heads", c_int), ("seq_q", c_int), ("seq_k", c_int),
        ("head_dim", c_int), ("causal", c_int), ("scale", c_float), ("kv_lens", c_void_p),
    ]


class RbAdamArgs(C.Structure):
    _fields_ = [
        ("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float), ("weight_decay", c_float),
        ("bias_correction1", c_float), ("bias_correction2", c_float), ("grad_scale", c_float),
        ("decoupled", c_int), ("max_grad_norm", c_float),
    ]


ACT = {"none": 0, "gelu": 1, "relu": 2, "silu": 3, "dgelu": 4, "drelu": 5, "dsilu": 6, "mul": 7}


class NativeError(RuntimeError):
    """A native entry point rejected its arguments or CUDA reported an error."""


# RUSTRAL_BOUNDS=1 selects the index-checking build of the kernel library (see _build.build_kernels).
# RUSTRAL_KERNEL_LIB names another build of the library (a file name inside the package's _lib folder or a path).
KERNEL_LIB = os.environ.get("RUSTRAL_KERNEL_LIB") or (
    "librb200_kernels_bounds.so" if os.environ.get("RUSTRAL_BOUNDS", "0") not in ("", "0") else "librb200_kernels.so")


def _load(name: str) -> C.CDLL:
    path = Path(name) if os.path.isabs(name) else LIB_DIR / name
    if not path.exists():
        raise FileNotFoundError(str(path))
    return C.CDLL(str(path))


def kernels() -> C.CDLL:
    """The sm_100a kernel library (``librb200_kernels.so``)."""
    lib = _libs.get("kernels")
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get("kernels")
        if lib is None:
            try:
                lib = _load(KERNEL_LIB)
            except (OSError, FileNotFoundError) as e:
                raise NativeError(
                    "librb200_kernels.so is not built or cannot be loaded; run "
                    "`python -m rustral_b200._build` (needs nvcc). CUDA tensors are only served by the "
                    f"native sm_100a kernels, there is no eager fallback. ({e})") from e
            _declare_kernels(lib)
            _libs["kernels"] = lib
    return lib


def have_kernels() -> bool:
    try:
        kernels()
        return True
    except NativeError:
        return False


def _ondemand(key: str, libname: str, builder: str, declare) -> C.CDLL:
    lib = _libs.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(key)
        if lib is None:
            if not (LIB_DIR / libname).exists():
                from . import _build
                getattr(_build, builder)()
            lib = _load(libname)
            declare(lib)
            _libs[key] = lib
    return lib


def cpu() -> C.CDLL:
    """The C++ f32 reference backend (``librb200_cpu.so``)."""
    from ._native_cpu import declare_cpu
    return _ondemand("cpu", "librb200_cpu.so", "build_cpu", declare_cpu)


def runtime() -> C.CDLL:
    """The host runtime library (``librb200_runtime.so``)."""
    from ._native_cpu import declare_runtime
    return _ondemand("runtime", "librb200_runtime.so", "build_runtime", declare_runtime)


def _declare_kernels(lib: C.CDLL) -> None:
    P = c_void_p

    def sig(name, args, res=c_int):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res

    sig("rb_init", [])
    sig("rb_sm_count", [])
    sig("rb_build_flags", [])
    sig("rb_status_read", [C.POINTER(C.c_uint), c_int])
    sig("rb_gemm_bf16", [C.POINTER(RbGemmArgs), P])
    sig("rb_norm_bwd_num_partials", [c_int, c_int])
    sig("rb_norm_fwd", [P, c_ll, P, P, P, c_ll, P, P, c_int, c_int, c_float, c_int, P])
    sig("rb_norm_bwd", [P, c_ll, P, c_ll, P, P, P, P, c_ll, P, c_ll, P, P, P, c_int, c_int, c_int, c_int, P])
    sig("rb_cross_entropy", [P, c_ll, P, P, P, P, c_ll, c_int, c_int, c_int, c_float, c_ll, P])
    sig("rb_softmax_rows", [P, P, c_int, c_int, c_ll, c_ll, c_int, c_int, P])
    sig("rb_softmax_rows_bwd", [P, P, P, c_int, c_int, c_int, P])
    sig("rb_adam_step", [P, P, P, P, c_int, P, c_ll, C.POINTER(RbAdamArgs), P, P, P])
    sig("rb_sgd_step", [P, P, P, c_int, P, c_ll, c_float, c_float, c_float, c_float, P])
    sig("rb_sumsq_scratch_floats", [])
    sig("rb_sumsq", [P, c_int, c_ll, P, P, P, c_int, P])
    sig("rb_sqrt_scalar", [P, P, P])
    sig("rb_cast_f32_to_bf16", [P, P, c_ll, P])
    sig("rb_cast_bf16_to_f32", [P, P, c_ll, P])
    sig("rb_embedding_fwd", [P, P, P, P, c_ll, c_int, c_int, c_ll, P])
    sig("rb_embedding_bwd_scratch_ints", [c_ll, c_ll], c_ll)
    sig("rb_embedding_bwd", [P, P, P, P, P, c_ll, c_int, c_int, c_ll, P])
    sig("rb_attention_fwd", [C.POINTER(RbAttnArgs), P])
    sig("rb_attention_bwd", [C.POINTER(RbAttnArgs), P])
    sig("rb_binary", [c_int, P, P, P, c_ll, c_int, P])
    sig("rb_unary", [c_int, P, P, c_ll, c_int, P])
    sig("rb_scalar", [c_int, P, c_float, P, c_ll, c_int, P])
    sig("rb_unary_bwd", [c_int, P, P, P, c_ll, c_int, P])
    sig("rb_add_row_vector", [P, P, P, c_ll, c_int, c_int, P])
    sig("rb_sum_dim0", [P, c_ll, P, c_ll, c_int, c_int, c_int, P])
    sig("rb_sum_dim0_slabs", [])
    sig("rb_sum_dim0_staged", [P, c_ll, P, P, c_ll, c_int, c_int, c_int, P])
    sig("rb_sum_all", [P, c_ll, c_int, P, P, P])
    sig("rb_transpose", [P, P, c_int, c_int, c_int, P])
    sig("rb_gather_rows", [P, P, P, c_ll, c_int, c_ll, c_int, P])
    sig("rb_scatter_rows", [P, P, P, c_ll, c_int, c_ll, c_int, P])
    sig("rb_broadcast_to", [P, P, c_ll, c_ll, c_ll, c_ll, c_int, P])
    sig("rb_strided_copy", [P, c_ll, P, c_ll, c_ll, c_ll, c_int, P])
    sig("rb_apply_mask", [P, P, c_float, P, c_ll, c_int, P])
    sig("rb_dropout", [P, P, P, c_ll, c_float, C.c_ulonglong, C.c_ulonglong, c_int, c_int, P])
    sig("rb_argmax_rows", [P, c_ll, P, c_ll, c_int, c_int, P])
    for name, args, res in _OPTIONAL_SIGS:
        if hasattr(lib, name):
            sig(name, args, res)


# Entry points added by later kernel files; declared when present in the loaded library.
_OPTIONAL_SIGS: list = []


def optional_sig(name: str, args, res=c_int) -> None:
    _OPTIONAL_SIGS.append((name, args, res))
    lib = _libs.get("kernels")
    if lib is not None and hasattr(lib, name):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res


# --------------------------------------------------------------------------------------------- helpers
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> int:
    """The current CUDA stream of the current device as an integer handle.  The two torch._C entry points answer in a
    fraction of a microsecond; `torch.cuda.current_stream()` builds a Stream object and costs about 3 us, a third of a
    small launch."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def stream_key(device) -> tuple:
    """(device, current stream handle of that device): the key of per-stream scratch buffers."""
    if _raw_stream is not None and device.index is not None:
        return (device, _raw_stream(device.index))
    return (device, torch.cuda.current_stream(device).cuda_stream)


def wants_grad(*tensors) -> bool:
    """True when autograd would record an op on these inputs; wrappers skip their autograd.Function otherwise (its
    `apply` alone costs several microseconds per call)."""
    if not torch.is_grad_enabled():
        return False
    for t in tensors:
        if t is not None and t.requires_grad:
            return True
    return False


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


# Kernel launches issued per native entry point (entries not listed launch one kernel).
_LAUNCHES = {"rb_norm_bwd": 2, "rb_sumsq": 2, "rb_sum_all": 2, "rb_sum_dim0_staged": 2, "rb_attention_bwd": 3,
             "rb_embedding_bwd": 5, "rb_status_read": 0}
launch_count = 0


def check(code: int, what: str) -> None:
    global launch_count
    launch_count += _LAUNCHES.get(what, 1)
    if code != 0:
        if code > 0:
            raise NativeError(f"{what}: CUDA error {code}")
        raise NativeError(f"{what}: rejected arguments (code {code})")


def read_status(clear: bool = True) -> tuple[int, int]:
    """(status bits, code of the wait that gave up) of the current device; synchronises."""
    out = (C.c_uint * 4)()
    check(kernels().rb_status_read(out, 1 if clear else 0), "rb_status_read")
    return int(out[0]), int(out[1])


def raise_on_status() -> None:
    bits, where = read_status(clear=True)
    if bits:
        raise NativeError(f"a device-side bounded wait gave up or a kernel flagged an error: bits={bits:#x} where={where}")
