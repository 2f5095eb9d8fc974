"""The allocation-free fp32 GEMM entry point against the regular dispatch / invoke pair.

`pmlb_gemm_f32_noalloc` serves hosts that have given all device memory to their own pool and
cannot let a library allocate behind their back; its scratch is a fixed array inside the
library.  The test calls it twice in a row through the C ABI -- the second call with another
shape, so that whatever the first call left in the shared array is in the way -- and compares
each result with what pmlb_gemm_dispatch + pmlb_gemm_invoke produce for the same operands.
Collected last (file name) so that a failure here cannot hide other tests in a -x run.
"""

import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from plaidml_b200 import kernels as K
from gpu_util import dev, empty, max_rel, ptr, rng

pytestmark = pytest.mark.gpu


def _noalloc():
    lib = K.load()
    fn = lib.pmlb_gemm_f32_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                   C.c_int64, C.c_int64, C.c_int32, C.c_int32]
    fn.restype = C.c_int
    return lib, fn


def _regular(a_t, b_t, m, n, k, b_is_nk):
    d = K.GemmDesc()
    d.in_dtype = d.out_dtype = K.F32
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.lda, d.ldb, d.ldc = k, (k if b_is_nk else n), n
    d.b_is_nk = int(b_is_nk)
    plan = K.Plan("gemm", d)
    c = empty((m, n), K.F32)
    plan.gemm(ptr(a_t), ptr(b_t), ptr(c))
    plan.check()
    return c.cpu().numpy()


def test_two_calls_in_a_row_match_the_allocating_path():
    lib, fn = _noalloc()
    g = rng(4242)
    for m, n, k, b_is_nk in [(256, 192, 320, False), (70, 50, 37, True)]:
        a = g.uniform(-1, 1, size=(m, k)).astype(np.float32)
        b = g.uniform(-1, 1, size=(n, k) if b_is_nk else (k, n)).astype(np.float32)
        a_t, b_t = dev(a), dev(b)
        c_t = empty((m, n), K.F32)
        c_t.fill_(float("nan"))
        rc = fn(None, ptr(a_t), ptr(b_t), ptr(c_t), m, n, k, k, (k if b_is_nk else n), n, int(b_is_nk), 1)
        assert rc == K.OK, lib.pmlb_last_error().decode()
        got = c_t.cpu().numpy()
        want = _regular(a_t, b_t, m, n, k, b_is_nk)
        # 1e-5 relative is the tolerance of the fp32 GEMM tests; the two paths run the same kernels
        assert max_rel(got, want) < 1e-5
        assert max_rel(got, oracle.gemm_f32_acc64(a, b, b_is_nk)) < 1e-5


def test_calls_leave_free_device_memory_unchanged_and_enqueued_launches_report_through_status():
    # the property the entry point exists for: once the first call on the device has happened (it is what brings
    # the static array into being under lazy module loading), further calls take no device memory at all
    lib, fn = _noalloc()
    status = lib.pmlb_gemm_f32_noalloc_status
    status.argtypes = [C.c_void_p]
    status.restype = C.c_int
    g = rng(4243)
    m, n, k = 192, 160, 96
    a = g.uniform(-1, 1, size=(m, k)).astype(np.float32)
    b = g.uniform(-1, 1, size=(k, n)).astype(np.float32)
    a_t, b_t = dev(a), dev(b)
    c_t = empty((m, n), K.F32)
    assert fn(None, ptr(a_t), ptr(b_t), ptr(c_t), m, n, k, k, n, n, 0, 1) == K.OK   # first call (or a later one)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        c_t.fill_(float("nan"))
        # enqueue only; the status query synchronises and would report a device-side time-out
        assert fn(None, ptr(a_t), ptr(b_t), ptr(c_t), m, n, k, k, n, n, 0, 0) == K.OK
        assert status(None) == K.OK, lib.pmlb_last_error().decode()
        assert max_rel(c_t.cpu().numpy(), oracle.gemm_f32_acc64(a, b, False)) < 1e-5
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_oversized_problem_is_refused_without_touching_the_device():
    lib, fn = _noalloc()
    t = empty((16,), K.F32)
    # 8 * (m + n) * k = 64 MiB of scratch: beyond the 32 MiB array
    rc = fn(None, ptr(t), ptr(t), ptr(t), 4096, 4096, 1024, 1024, 4096, 4096, 0, 1)
    assert rc == K.ERR_UNSUPPORTED
    msg = lib.pmlb_last_error().decode()
    assert "bytes of scratch" in msg and str(32 << 20) in msg
