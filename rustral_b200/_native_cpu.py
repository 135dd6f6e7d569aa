"""ctypes signatures of the C++ reference backend and the host runtime library."""
from __future__ import annotations

import ctypes as C

P, I, LL, F, D = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_double


def _sig(lib, name, args, res=None):
    fn = getattr(lib, name)
    fn.argtypes = args
    fn.restype = res


def declare_cpu(lib) -> None:
    _sig(lib, "rb_cpu_set_threads", [I])
    _sig(lib, "rb_cpu_matmul", [P, P, P, I, I, I])
    _sig(lib, "rb_cpu_linear", [P, P, P, P, I, I, I, I])
    _sig(lib, "rb_cpu_softmax_rows", [P, P, I, I, I])
    _sig(lib, "rb_cpu_layer_norm", [P, P, P, P, P, P, I, I, F, I])
    _sig(lib, "rb_cpu_layer_norm_bwd", [P, P, P, P, P, P, P, P, I, I, I])
    _sig(lib, "rb_cpu_unary", [I, P, P, LL])
    _sig(lib, "rb_cpu_cross_entropy", [P, P, P, P, I, I, F, LL])
    _sig(lib, "rb_cpu_adam", [P, P, P, P, LL, F, F, F, F, F, I, I])
    _sig(lib, "rb_cpu_attention", [P, P, P, P, I, I, I, I, I, I, I, F])
    _sig(lib, "rb_cpu_moe_route", [P, I, I, I, I, P, P, P])
    _sig(lib, "rb_cpu_gather_rows", [P, P, P, LL, I, LL])
    _sig(lib, "rb_cpu_scatter_add_rows", [P, P, P, LL, I, LL])


def declare_runtime(lib) -> None:
    _sig(lib, "rb_ba_create", [I, I], P)
    _sig(lib, "rb_ba_destroy", [P])
    for n in ("rb_ba_num_free", "rb_ba_num_blocks", "rb_ba_block_size", "rb_ba_num_sequences"):
        _sig(lib, n, [P], I)
    _sig(lib, "rb_ba_reserve", [P, LL, I], I)
    _sig(lib, "rb_ba_can_reserve", [P, LL, I], I)
    _sig(lib, "rb_ba_free", [P, LL], I)
    _sig(lib, "rb_ba_table_len", [P, LL], I)
    _sig(lib, "rb_ba_table", [P, LL, P, I], I)
    _sig(lib, "rb_ba_slot", [P, LL, I], LL)
    _sig(lib, "rb_search_create", [I, I, P, P, C.c_uint64, I], P)
    _sig(lib, "rb_search_destroy", [P])
    _sig(lib, "rb_search_next", [P, P], I)
    _sig(lib, "rb_search_report", [P, P, D])
    _sig(lib, "rb_search_best", [P, P, P], I)
    _sig(lib, "rb_search_num_evals", [P], I)
    _sig(lib, "rb_tokens_open", [C.c_char_p, I], P)
    _sig(lib, "rb_tokens_close", [P])
    _sig(lib, "rb_tokens_len", [P], LL)
    _sig(lib, "rb_tokens_gather", [P, P, I, I, P], I)
    _sig(lib, "rb_tokens_sample_offsets", [P, C.c_uint64, C.c_uint64, I, I, P])
    _sig(lib, "rb_prefetch_create", [P, C.c_uint64, C.c_uint64, I, I, I, P], P)
    _sig(lib, "rb_prefetch_next", [P, I, P], I)
    _sig(lib, "rb_prefetch_release", [P, I], I)
    _sig(lib, "rb_prefetch_destroy", [P])
    _sig(lib, "rb_sched_create", [P, I, I, D, I], P)
    _sig(lib, "rb_sched_destroy", [P])
    _sig(lib, "rb_sched_add", [P, I, I, I, I, LL], LL)
    _sig(lib, "rb_sched_has_work", [P], I)
    _sig(lib, "rb_sched_retire", [P])
    _sig(lib, "rb_sched_schedule", [P, P, P, P, I], I)
    _sig(lib, "rb_sched_take_retired", [P, P, I], I)
    _sig(lib, "rb_sched_update", [P, P, P, I, P], I)
    _sig(lib, "rb_sched_state", [P, LL], I)
    _sig(lib, "rb_sched_stats", [P, P])
    _sig(lib, "rb_sched_list", [P, I, P, I], I)
    _sig(lib, "rb_sched_forget", [P, LL])
    _sig(lib, "rb_sched_abort", [P, LL], C.c_int)
    _sig(lib, "rb_aw_create", [I], P)
    _sig(lib, "rb_aw_destroy", [P])
    _sig(lib, "rb_aw_submit_copy", [P, C.c_char_p, P, LL], LL)
    _sig(lib, "rb_aw_submit_borrowed", [P, C.c_char_p, P, LL], LL)
    _sig(lib, "rb_aw_wait", [P, LL, I], I)
    _sig(lib, "rb_aw_flush", [P, I], I)
    _sig(lib, "rb_aw_pending", [P], I)
    _sig(lib, "rb_aw_bytes_written", [P], LL)
    _sig(lib, "rb_aw_take_error", [P, C.c_char_p, I], I)
