"""GPU: the allocation-free column sum (mg_colsum_noalloc).

Collected last on purpose (file name), so that a run which stops at the first
failure has already exercised every other test.

Some callers cannot allocate device memory at the point where they need a bias
gradient — an allocation would stall a latency-critical loop, or all memory
already belongs to another component's pool.  mg_colsum_noalloc keeps its
partial sums in a fixed array inside the library image instead.  The test calls
it through the C ABI twice in a row on different inputs (the second, smaller
call finds the first call's partials still in the shared array) and compares
each result with the pooled entry point mg_add_row_bwd, within the reduction
tolerance used throughout the suite (1e-10 of the column's sum of magnitudes).
It also checks the documented size limit and that no pool memory is taken.
"""
import ctypes as C

import numpy as np
import pytest

from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu
TOL = 1e-10
LIMIT = 131072


def _pooled(abi, dg, M, N):
    out = abi.empty(N)
    abi.mg_add_row_bwd(dg.ptr, None, out.ptr, M, N, K.ACC_STORE_B)
    return out.numpy()


def test_two_calls_in_a_row_match_the_pooled_entry_point(abi):
    rng = np.random.default_rng(2024)
    first = rng.standard_normal((4096, 1024))
    second = rng.standard_normal((257, 10))          # smaller: stale partials lie beyond it
    d1, d2 = abi.array(first), abi.array(second)
    out1, out2 = abi.empty(1024), abi.array(np.full(10, 3.0))
    # Set-up call: the first call on a device resolves the static array's address
    # (and lets the driver load the module that holds it).  Documented to come first.
    abi.mg_colsum_noalloc(d2.ptr, out2.ptr, 1, 10, 1)
    threes = np.full(10, 3.0)
    abi.mg_upload(out2.ptr, threes.ctypes.data, 10)
    free0, total = C.c_size_t(), C.c_size_t()
    abi.mg_sync()
    abi.mg_mem_info(C.byref(free0), C.byref(total))
    abi.mg_colsum_noalloc(d1.ptr, out1.ptr, 4096, 1024, 0)
    abi.mg_colsum_noalloc(d2.ptr, out2.ptr, 257, 10, 1)      # accumulates onto 3.0
    abi.mg_sync()
    free1 = C.c_size_t()
    abi.mg_mem_info(C.byref(free1), C.byref(total))
    assert free1.value == free0.value                        # nothing was taken from the device
    got1, got2 = out1.numpy(), out2.numpy()
    ref1, ref2 = _pooled(abi, d1, 4096, 1024), _pooled(abi, d2, 257, 10)
    assert np.all(np.abs(got1 - ref1) <= TOL * np.abs(first).sum(axis=0))
    assert np.all(np.abs(got2 - (ref2 + 3.0)) <= TOL * (np.abs(second).sum(axis=0) + 3.0))
    # and against plain host arithmetic
    assert np.all(np.abs(got1 - first.sum(axis=0)) <= TOL * np.abs(first).sum(axis=0))
    # repeated call on the first input reproduces the same bits
    again = abi.empty(1024)
    abi.mg_colsum_noalloc(d1.ptr, again.ptr, 4096, 1024, 0)
    assert np.array_equal(again.numpy(), got1)


def test_odd_width_and_single_row(abi):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((33, 77))
    dx, out = abi.array(x), abi.empty(77)
    abi.mg_colsum_noalloc(dx.ptr, out.ptr, 33, 77, 0)
    assert np.all(np.abs(out.numpy() - _pooled(abi, dx, 33, 77)) <= TOL * np.abs(x).sum(axis=0))
    row = abi.array(x[:1])
    abi.mg_colsum_noalloc(row.ptr, out.ptr, 1, 77, 0)
    assert np.array_equal(out.numpy(), x[0])


def test_width_beyond_the_static_limit_is_rejected(abi):
    wide = abi.zeros(LIMIT + 2)
    out = abi.zeros(LIMIT + 2)
    with pytest.raises(K.MgError) as e:
        abi.mg_colsum_noalloc(wide.ptr, out.ptr, 1, LIMIT + 2, 0)
    assert e.value.code == K.ERR_INVALID and "static scratch limit" in str(e.value)
    abi.mg_colsum_noalloc(wide.ptr, out.ptr, 1, LIMIT, 0)    # exactly at the limit is fine
    abi.mg_sync()
    assert not out.numpy().any()
