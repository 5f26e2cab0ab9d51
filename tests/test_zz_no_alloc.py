"""The allocation-free linear-backward entry point against the regular one.

Some embedders of the library own all device memory themselves and may not let a library call cudaMalloc; for them
``rtp_linear_bwd_noalloc`` keeps its scratch in a fixed array inside the shared library.  The test calls it through
its exported C symbol, twice in a row (the array keeps the previous call's contents, so the second call checks
that everything that must start at zero is cleared), and compares with the regular entry point on the same inputs.
This file is collected last on purpose: a run that stops at the first failure has then already run every other
test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_linear_backward_matches_regular_entry_point():
    from rtp_b200.ops import _lib
    from rtp_b200.parallel import engine as E
    from rtp_b200.parallel.context import get_context
    L = _lib.lib()
    fn = L.rtp_linear_bwd_noalloc
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                   C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    L.rtp_noalloc_last_error.restype = C.c_char_p
    L.rtp_noalloc_status.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong)]
    L.rtp_noalloc_status.restype = C.c_int
    torch.manual_seed(0)
    M, IN, OUT = 777, 512, 1024
    bias_off = OUT * IN
    nflat = bias_off + OUT
    eng = E.get_engine(get_context())
    for trial in range(2):
        flat = (torch.randn(nflat, device="cuda") * 0.05).to(BF)
        x = torch.randn(M, IN, device="cuda", dtype=BF)
        dy = torch.randn(M, OUT, device="cuda", dtype=BF)
        # regular entry point (scratch from torch's allocator and the engine workspace)
        dx_ref, g_ref = E.linear_bwd_raw(eng, flat, (True, bias_off, nflat * 2), x, dy, False, IN, OUT)
        torch.cuda.synchronize()
        # allocation-free entry point: outputs are allocated here, by the caller
        dx = torch.empty(M, IN, device="cuda", dtype=BF)
        g = torch.zeros(nflat, device="cuda", dtype=BF)
        # free bytes as the driver sees them: a cudaMalloc inside the library would show here, whereas torch's own
        # counters only see torch's caching allocator
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), IN, dy.data_ptr(), OUT, flat.data_ptr(), bias_off, M, IN, OUT, dx.data_ptr(), IN,
                g.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.rtp_noalloc_last_error()
        status = C.c_ulonglong(99)
        assert L.rtp_noalloc_status(torch.cuda.current_stream().cuda_stream, C.byref(status)) == 0
        assert status.value == 0, status.value        # no bounded wait ran out inside the kernel
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if trial == 1:     # the first call may still load the kernels' module lazily; the second must not take a byte
            assert torch.cuda.mem_get_info()[0] == free_before
        assert _rel(dx, dx_ref) < 1e-3, (trial, _rel(dx, dx_ref))
        assert _rel(g[:bias_off], g_ref[:bias_off]) < 1e-3, (trial, _rel(g[:bias_off], g_ref[:bias_off]))
        assert _rel(g[bias_off:], g_ref[bias_off:]) < 1e-3, (trial, _rel(g[bias_off:], g_ref[bias_off:]))
        # and against plain fp32 math, within the tolerance of the other GEMM tests
        w = flat[:bias_off].view(OUT, IN).float()
        assert _rel(dx, dy.float() @ w) < 1e-2
        assert _rel(g[:bias_off].view(OUT, IN), dy.float().t() @ x.float()) < 1e-2
        assert _rel(g[bias_off:], dy.float().sum(0)) < 1e-2


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    from rtp_b200.ops import _lib
    L = _lib.lib()
    fn = L.rtp_linear_bwd_noalloc
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                   C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    L.rtp_noalloc_last_error.restype = C.c_char_p
    rc = fn(None, 8, None, 8, None, -1, 8, 8, 65536 + 8, None, 8, None, None)
    assert rc != 0
    assert b"exceeds" in L.rtp_noalloc_last_error()
