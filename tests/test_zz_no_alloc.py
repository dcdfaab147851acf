"""The allocation-free bias-gradient entry point against the regular one.

`rst_bias_grad_noalloc` serves hosts that may not call cudaMalloc where they need
db (a process whose own allocator has claimed the whole device and hands out raw
pointers, or a step under a hard latency bound, which an allocation's device-wide
synchronisation would break): it works on raw device pointers and keeps its partial
sums in a fixed array inside the library instead of scratch grown on demand.
This file is collected last on purpose, so a failure here cannot hide the result
of any other test in a run that stops at the first failure.
"""
import ctypes as C

import numpy as np
import pytest

import rstorch_b200 as rt
from conftest import REL_TOL, rel_err
from rstorch_b200 import _lib

pytestmark = pytest.mark.gpu


def regular_db(ctx, dY: np.ndarray, cin: int = 8) -> np.ndarray:
    """db as the existing entry point rst_linear_backward computes it."""
    B, cout = dY.shape
    x, w = ctx.zeros(B, cin), ctx.zeros(cout, cin)
    dw, db, grad = ctx.empty(cout, cin), ctx.empty(1, cout), ctx.tensor(dY)
    ctx._check(ctx._lib.rst_linear_backward(ctx.handle, grad.handle, x.handle, w.handle, None,
                                            dw.handle, db.handle, None))
    return db.numpy()


def noalloc_db(ctx, dY: np.ndarray) -> np.ndarray:
    """db through the new entry point: raw pointers and the caller's stream only."""
    B, cout = dY.shape
    src, dst = ctx.tensor(dY), ctx.empty(1, cout)
    dst.fill(np.nan)                               # the call must overwrite every element
    if not _warmed:
        # The first call on a device looks up the array's address, and the driver may load the
        # two kernels' code then; the memory comparison below starts after that one call.
        tiny = ctx.zeros(2, 2)
        _lib.check(ctx._lib.rst_bias_grad_noalloc(C.c_void_p(tiny.data_ptr()), 2, 2, C.c_void_p(tiny.data_ptr()),
                                                  C.c_void_p(ctx.stream_pointer())))
        _warmed.append(True)
    ctx.synchronize()
    before, free_before = ctx.memory_stats(), device_free_bytes()
    status = ctx._lib.rst_bias_grad_noalloc(C.c_void_p(src.data_ptr()), B, cout, C.c_void_p(dst.data_ptr()),
                                            C.c_void_p(ctx.stream_pointer()))
    _lib.check(status)
    ctx.synchronize()
    assert ctx.memory_stats() == before            # nothing was requested from the library's allocator
    assert device_free_bytes() == free_before      # and the driver handed out no device memory either
    return dst.numpy()


_warmed: list = []


def device_free_bytes() -> int:
    """Free device memory as the driver reports it (cudaMemGetInfo)."""
    import torch
    return torch.cuda.mem_get_info(0)[0]


def test_two_calls_in_a_row_match_the_regular_entry_point(ctx):
    rng = np.random.default_rng(42)
    # the second call is narrower and shorter than the first, so anything left in the shared
    # array by the first call would show up if the second one read it
    for rows, cols in [(4096, 1000), (333, 130)]:
        dY = rng.standard_normal((rows, cols))
        got, want = noalloc_db(ctx, dY), regular_db(ctx, dY)
        assert got.shape == want.shape == (1, cols)
        assert rel_err(got, want) < REL_TOL
        assert rel_err(got, dY.sum(axis=0, keepdims=True) / rows) < REL_TOL


def test_one_row_and_the_widest_input_that_fits(ctx):
    rng = np.random.default_rng(3)
    one_row = rng.standard_normal((1, 77))         # a single row: db is the row itself
    assert np.array_equal(noalloc_db(ctx, one_row), one_row)
    widest = rng.standard_normal((3, 262144))      # RST_BIAS_GRAD_NOALLOC_MAX_COLS: room for one row part only
    assert rel_err(noalloc_db(ctx, widest), widest.sum(axis=0, keepdims=True) / 3) < REL_TOL


def test_wide_input_uses_fewer_row_parts_than_fit(ctx):
    rng = np.random.default_rng(7)
    dY = rng.standard_normal((512, 20000))         # 20000 columns leave room for 13 row parts only
    assert rel_err(noalloc_db(ctx, dY), regular_db(ctx, dY)) < REL_TOL


def test_sizes_beyond_the_fixed_array_are_rejected(ctx):
    lib = ctx._lib
    one = ctx.empty(1, 1)
    too_wide = 262144 + 1                          # RST_BIAS_GRAD_NOALLOC_MAX_COLS + 1
    status = lib.rst_bias_grad_noalloc(C.c_void_p(one.data_ptr()), 1, too_wide, C.c_void_p(one.data_ptr()), None)
    assert status == _lib.RST_ERR_UNSUPPORTED
    assert b"262144" in lib.rst_last_error(None)
    assert lib.rst_bias_grad_noalloc(None, 4, 4, None, None) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_bias_grad_noalloc(None, 0, 0, None, None) == _lib.RST_OK
