"""The allocation-free linear layer (ncmb_linear_fwd_noalloc) against linear_fwd.

Some callers of this library cannot allocate device memory while they run (fixed
memory budgets, host callbacks, stream-capture regions, latency-critical serving
loops), so the library offers one GEMM entry point whose scratch lives in an
array compiled into the module.  This file is collected last on purpose: if it
fails, a run that stops at the first failure has already executed every other
test.  It must pass on its own in a fresh process and after the rest of the suite.
"""
import os

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    import capi
    lib = capi.NcmLib(helpers.CUDA_LIB)
    lib.ncmb_set_gemm_mode(2)          # linear_fwd then runs the same three-pass kernel
    return lib


def _free_device_bytes(lib):
    import ctypes as C
    free, total = C.c_ulonglong(0), C.c_ulonglong(0)
    lib.ncmb_mem_info(C.byref(free), C.byref(total))
    return free.value


def _pair(lib, rng, batch, M, K, with_bias, warmed):
    x = rng.standard_normal((batch, K)).astype(np.float32)
    W = (rng.standard_normal((M, K)) * 0.05).astype(np.float32)
    b = rng.standard_normal(M).astype(np.float32) if with_bias else None
    xd, Wd = lib.to_backend(x), lib.to_backend(W)
    bd = lib.to_backend(b) if with_bias else None
    y_ref, y_new = lib.alloc(batch * M), lib.alloc(batch * M)
    lib.linear_fwd(xd, Wd, bd, y_ref, batch, M, K)
    lib.ncmb_sync()
    assert lib.ncmb_gemm_tc_check() == 0
    free_before = _free_device_bytes(lib)
    rc = lib.ncmb_linear_fwd_noalloc(xd, Wd, bd, y_new, batch, M, K)
    assert rc == 0
    # the entry point's own status word (not the one linear_fwd's kernels write): 0 = no bounded wait ran out
    assert lib.ncmb_linear_fwd_noalloc_check() == 0
    if warmed:
        # "allocates nothing", pinned: the device's free memory is what it was before the call (the first call of
        # a process may still load the kernels' code, so the comparison starts with the second)
        assert _free_device_bytes(lib) == free_before
    want = x.astype(np.float64) @ W.astype(np.float64).T + (b if with_bias else 0.0)
    return lib.to_host(y_ref, (batch, M)), lib.to_host(y_new, (batch, M)), want


def test_two_calls_in_a_row_match_linear_fwd(cuda):
    rng = np.random.default_rng(123)
    # second call is smaller and uses different data: nothing of the first call's scratch may leak in
    for i, (batch, M, K, bias) in enumerate(((777, 520, 512, True), (130, 96, 100, False), (40, 64, 64, True))):
        ref, new, want = _pair(cuda, rng, batch, M, K, bias, warmed=i > 0)
        # same kernels, same operand splits: the two entry points agree to the last bit
        assert np.array_equal(ref, new)
        # and both are fp32-grade against a float64 product (tolerance of the kernel tests, scaled by |y|)
        assert np.abs(new - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


def test_sizes_beyond_the_built_in_scratch_are_refused(cuda):
    rng = np.random.default_rng(5)
    K, M = 1024, 64
    batch = (8 << 20) // (2 * K) + 64          # 2*batch*K alone exceeds the 8 Mi-float array
    x = cuda.alloc(batch * K)
    W = cuda.to_backend((rng.standard_normal((M, K)) * 0.05).astype(np.float32))
    y = cuda.alloc(batch * M)
    assert cuda.ncmb_linear_fwd_noalloc(x, W, None, y, batch, M, K) == -1
    # shapes the tensor-core kernel does not take are refused as well, not silently rerouted
    assert cuda.ncmb_linear_fwd_noalloc(x, W, None, y, 8, M, K) == -1
    assert cuda.ncmb_linear_fwd_noalloc(x, W, None, y, 16, M, K) == -1      # up to 16 rows: refused; 17 and more run
    assert cuda.ncmb_linear_fwd_noalloc(x, W, None, y, 17, M, K) == 0
    assert cuda.ncmb_linear_fwd_noalloc_check() == 0
