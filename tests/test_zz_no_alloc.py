"""litnice_b200_gemv_noalloc: the few-row product for callers that may not
allocate device memory while they run (a host whose arenas already own all of
it, or a loop that cannot take the stall of an allocation). Its partial sums
live in an array built into the library, so this checks, through the C ABI,
that it returns what the existing projection entry of the plugin table returns
on the same operands (and what the oracle's product returns), on two calls in a
row that share that array, and that it refuses a shape whose partial sums would
not fit.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from litnicelm_b200.plugin import Backend
from abi_util import Buffer

pytestmark = pytest.mark.gpu

ETOOBIG, EINVAL = -6, -1


def device_sync():
    import torch
    torch.cuda.synchronize()


@pytest.fixture()
def be():
    b = Backend()
    fn = b.lib.litnice_b200_gemv_noalloc
    fn.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    yield b
    b.close()


def run_pair(be, m, k, n, seed, with_bias):
    """(no-alloc result, plugin-table result) for one shape."""
    rng = np.random.default_rng(seed)
    xb = Buffer(be, m * k * 4, rng)
    wb = Buffer(be, k * n * 4, rng)
    bb = Buffer(be, n * 4, rng)
    out_new = Buffer(be, m * n * 4, fill=-7.0)
    out_old = Buffer(be, m * n * 4, fill=-9.0)
    device_sync()
    rc = be.lib.litnice_b200_gemv_noalloc(xb.ptr, m, wb.ptr, k, n, bb.ptr if with_bias else None,
                                          out_new.ptr, None)
    assert rc == 0
    device_sync()
    # existing entry points: gemm_ranked_matrix_rhs (+ add_bias_rowwise) of the plugin table
    a = xb.view((1, m, k))
    o = out_old.view((1, m, n))
    be.call("gemm_ranked_matrix_rhs", a, wb.view((k, n)), o)
    if with_bias:
        be.call("add_bias_rowwise", o, bb.view((1, n)), o)
    got = out_new.pull().view(np.float32).reshape(m, n).copy()
    want = out_old.pull().view(np.float32).reshape(m, n).copy()
    # the oracle's product (device_backend.cpp:1112-1131 restated) on the same operands
    from oracle import binding as ob
    x = xb.host.view(np.float32).reshape(m, k)
    w = wb.host.view(np.float32).reshape(k, n)
    ref = ob.gemm(x, w)
    if with_bias:
        ref = ref + bb.host.view(np.float32)[None, :]
    np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-5 * np.sqrt(k) * float(np.abs(x).max() * np.abs(w).max()))
    return got, want


def test_two_calls_in_a_row_match_the_plugin_table(be):
    # both shapes split k across CTAs, so both go through the built-in array;
    # the second is smaller and must not see anything the first left behind
    for (m, k, n, bias) in [(8, 1024, 512, True), (1, 512, 96, False)]:
        got, want = run_pair(be, m, k, n, seed=m * 1000 + n, with_bias=bias)
        # tolerance of the projection parity tests (summation order differs)
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5 * np.sqrt(k))
        assert not np.any(got == -7.0)


@pytest.mark.parametrize("m,k,n", [(4, 300, 50), (2, 512, 98), (8, 192, 16384), (4, 256, 512)])
def test_other_paths_through_the_built_in_array(be, m, k, n):
    """Shapes that take the scalar-load kernel (n not a multiple of 4), four rows, and the
    largest shape the array holds (8 x 16384 columns in 3 splits = 393216 floats exactly)."""
    got, want = run_pair(be, m, k, n, seed=m + k + n, with_bias=(n % 2 == 0))
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5 * np.sqrt(k) * 4)


def test_wide_head_needs_no_scratch(be):
    got, want = run_pair(be, 2, 64, 32000, seed=5, with_bias=False)
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5 * np.sqrt(64))


def test_sizes_beyond_the_built_in_array_are_refused(be, capfd):
    buf = Buffer(be, 1024)
    # m=8, n=16512, k=256 would need 3*8*16512 floats of partial sums (> 393216)
    rc = be.lib.litnice_b200_gemv_noalloc(buf.ptr, 8, buf.ptr, 256, 16512, None, buf.ptr, None)
    assert rc == ETOOBIG
    assert "needs 396288 floats" in capfd.readouterr().err
    # the other refused range: 98 column blocks take 4 splits, 4*8*12544 floats
    rc = be.lib.litnice_b200_gemv_noalloc(buf.ptr, 8, buf.ptr, 256, 12544, None, buf.ptr, None)
    assert rc == ETOOBIG
    assert "needs 401408 floats" in capfd.readouterr().err
    assert be.lib.litnice_b200_gemv_noalloc(buf.ptr, 3, buf.ptr, 256, 128, None, buf.ptr, None) == EINVAL
    assert be.lib.litnice_b200_gemv_noalloc(None, 1, buf.ptr, 256, 128, None, buf.ptr, None) == EINVAL
