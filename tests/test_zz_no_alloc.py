"""rb_norm_bwd_noalloc: the normalisation backward pass for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off limits: inside a serving loop that must not synchronise the
device, in a plugin that only receives input and output buffers, or in host code with no allocator of its own.  For
them the library exports one entry point whose scratch memory is a fixed device array inside the library.  This test
drives that entry point through its exported C symbol, exactly as such a caller would, and checks that it produces
what the ordinary entry point (which takes caller-provided scratch) produces, on two calls in a row, because the
built-in scratch is shared between calls and keeps the previous call's contents.

The file name sorts behind the regular suites on purpose: a run that stops at the first failure has by then run them.
"""
import ctypes as C

import pytest
import torch

from rustral_b200 import _native as N

pytestmark = pytest.mark.gpu

P, LL, I = C.c_void_p, C.c_longlong, C.c_int


def _symbols():
    lib = N.kernels()
    fn = lib.rb_norm_bwd_noalloc
    fn.argtypes = [P, LL, P, LL, P, P, P, P, LL, P, LL, P, P, I, I, I, I, P]
    fn.restype = I
    cap = lib.rb_norm_bwd_noalloc_capacity_floats
    cap.argtypes = []
    cap.restype = LL
    return lib, fn, cap


def _problem(rows, n, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    x, dy, dres = mk(rows, n), mk(rows, n), mk(rows, n)
    gamma = (torch.randn(n, generator=g) * 0.1 + 1).to(torch.bfloat16).cuda()
    xf = x.float()
    mean = xf.mean(-1).contiguous()
    rstd = torch.rsqrt(((xf - mean[:, None]) ** 2).mean(-1) + 1e-5).contiguous()
    return x, dy, dres, gamma, mean, rstd


def _run_reference(lib, x, dy, dres, gamma, mean, rstd, rms):
    rows, n = x.shape
    parts = lib.rb_norm_bwd_num_partials(rows, n)
    scratch = torch.empty(2 * parts * n, dtype=torch.float32, device="cuda")
    dx = torch.empty_like(x)
    dg = torch.empty(n, dtype=torch.float32, device="cuda")
    db = torch.empty(n, dtype=torch.float32, device="cuda")
    rc = lib.rb_norm_bwd(dy.data_ptr(), n, x.data_ptr(), n, gamma.data_ptr(), None if rms else mean.data_ptr(),
                         rstd.data_ptr(), dres.data_ptr(), n, dx.data_ptr(), n, dg.data_ptr(), None if rms else db.data_ptr(),
                         scratch.data_ptr(), rows, n, int(rms), 0, N.stream_ptr())
    assert rc == 0
    return dx, dg, db


def _run_noalloc(fn, x, dy, dres, gamma, mean, rstd, rms):
    rows, n = x.shape
    dx = torch.empty_like(x)
    dg = torch.empty(n, dtype=torch.float32, device="cuda")
    db = torch.empty(n, dtype=torch.float32, device="cuda")
    rc = fn(dy.data_ptr(), n, x.data_ptr(), n, gamma.data_ptr(), None if rms else mean.data_ptr(), rstd.data_ptr(),
            dres.data_ptr(), n, dx.data_ptr(), n, dg.data_ptr(), None if rms else db.data_ptr(), rows, n, int(rms), 0,
            N.stream_ptr())
    assert rc == 0, f"rb_norm_bwd_noalloc returned {rc}"
    return dx, dg, db


def _close(a, b):
    # both entry points run the same deterministic kernels (ordered partial sums, no atomics): the results are equal
    # bit for bit, not merely close
    assert torch.equal(a, b)


@pytest.mark.parametrize("rms", [False, True])
def test_noalloc_entry_matches_the_allocating_entry_twice_in_a_row(rms):
    lib, fn, cap = _symbols()
    lib.rb_init()
    N.read_status(clear=True)
    assert cap() == 2 * 296 * 4096
    # two different problems back to back: the second call finds the first call's partial sums in the shared scratch
    for rows, n, seed in ((1500, 768, 1), (333, 2048, 2)):
        args = _problem(rows, n, seed)
        got = _run_noalloc(fn, *args, rms)
        want = _run_reference(lib, *args, rms)
        torch.cuda.synchronize()
        _close(got[0], want[0])
        _close(got[1], want[1])
        if not rms:
            _close(got[2], want[2])
    assert N.read_status(clear=True)[0] == 0


def test_noalloc_entry_refuses_what_does_not_fit():
    lib, fn, cap = _symbols()
    rows, n = 4096, 8192                      # 2 * 296 * 8192 floats: twice the built-in scratch
    assert 2 * lib.rb_norm_bwd_num_partials(rows, n) * n > cap()
    x = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    s = torch.ones(rows, dtype=torch.float32, device="cuda")
    dg = torch.zeros(n, dtype=torch.float32, device="cuda")
    rc = fn(x.data_ptr(), n, x.data_ptr(), n, g.data_ptr(), s.data_ptr(), s.data_ptr(), None, 0, x.data_ptr(), n,
            dg.data_ptr(), dg.data_ptr(), rows, n, 0, 0, N.stream_ptr())
    assert rc == -22
