"""The tensor-core projection (tcgen05, three-product TF32 split) against the
fp32 SIMT kernel and the oracle, through litnice_b200_projection_host.

A single-pass TF32 product would miss these tolerances by more than an order of
magnitude (its error is ~5e-4 * sqrt(k) here), so passing them shows that the
split recovers fp32-grade accuracy.
"""
import ctypes as C

import numpy as np
import pytest

from litnicelm_b200 import plugin

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def project():
    lib = plugin.load_library()
    fn = lib.litnice_b200_projection_host
    f32p = C.POINTER(C.c_float)
    fn.argtypes = [C.c_int32, f32p, C.c_int32, C.c_int32, f32p, C.c_int32, f32p, f32p, C.c_int32, f32p]
    fn.restype = C.c_int

    def run(engine, a, w, bias=None, residual=None, relu=False):
        m, k = a.shape
        n = w.shape[1]
        out = np.empty((m, n), np.float32)
        p = lambda x: x.ctypes.data_as(f32p) if x is not None else None
        rc = fn(engine, p(a), m, k, p(w), n, p(bias), p(residual), 1 if relu else 0, p(out))
        assert rc == 0, f"projection_host engine {engine} failed: {rc}"
        return out

    return run


SHAPES = [(128, 32, 64), (128, 64, 128), (1, 64, 64), (129, 96, 192), (640, 512, 1536), (300, 2048, 512),
          (1000, 512, 2048), (4096, 256, 1024),
          # enough row tiles for the 256-column configuration
          (9600, 128, 1024), (19100, 96, 512)]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_tensor_core_projection_matches_simt_and_oracle(project, oracle, m, k, n):
    rng = np.random.default_rng(m * 7 + k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    want = oracle.gemm(a, w)
    simt = project(0, a, w)
    tc = project(1, a, w)
    atol = 2e-5 * np.sqrt(k)
    np.testing.assert_allclose(simt, want, rtol=2e-5, atol=atol)
    np.testing.assert_allclose(tc, want, rtol=2e-5, atol=atol)
    err_tc = float(np.abs(tc - want).max())
    err_simt = float(np.abs(simt - want).max())
    msg = f"{m}x{k}x{n}: max abs err TF32 pairs {err_tc:.2e}, simt {err_simt:.2e}"
    if k % 64 == 0:  # fp16 pairs with block scales
        f16 = project(2, a, w)
        np.testing.assert_allclose(f16, want, rtol=2e-5, atol=atol)
        msg += f", fp16 pairs {float(np.abs(f16 - want).max()):.2e}"
    print(msg)


@pytest.mark.parametrize("relu", [False, True])
def test_tensor_core_epilogue(project, relu):
    rng = np.random.default_rng(3)
    m, k, n = 200, 128, 256
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    want = a.astype(np.float64) @ w.astype(np.float64) + bias + res
    if relu:
        want = np.maximum(want, 0)
    for engine in (0, 1, 2):
        got = project(engine, a, w, bias, res, relu)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4)


# Few tiles and a long k: the CTAs of a tile form a cluster of 2..8 k ranges (how many depends on the
# tile count and on the operand type's k-block), each sends its partial sums of a row to the CTA that
# stores the row. The shapes give row shares of 64 down to 16 rows, even and uneven, and a ragged last tile.
CLUSTER_SHAPES = [(256, 512, 1024), (640, 2048, 512), (256, 1024, 512), (128, 1280, 640),
                  (300, 2048, 512), (128, 1792, 768), (200, 2048, 256), (77, 4096, 128)]


@pytest.mark.parametrize("m,k,n", CLUSTER_SHAPES)
def test_cluster_split_k_with_epilogue(project, m, k, n):
    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    want = np.maximum(a.astype(np.float64) @ w.astype(np.float64) + bias + res, 0)
    for engine in (1, 2):
        got = project(engine, a, w, bias, res, True)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-5 * np.sqrt(k), err_msg=f"engine {engine}")
        again = project(engine, a, w, bias, res, True)
        assert np.array_equal(got, again), "partial sums are added in rank order: bit-identical between runs"


def test_tensor_core_engine_rejects_unsupported_shapes(project):
    lib = plugin.load_library()
    a = np.zeros((4, 48), np.float32)
    w = np.zeros((48, 64), np.float32)
    out = np.zeros((4, 64), np.float32)
    f32p = C.POINTER(C.c_float)
    rc = lib.litnice_b200_projection_host(1, a.ctypes.data_as(f32p), 4, 48, w.ctypes.data_as(f32p), 64, None, None,
                                          0, out.ctypes.data_as(f32p))
    assert rc == -1  # k % 32 != 0


def test_fp16_pairs_follow_the_dynamic_range_of_each_block(project):
    """Rows and k-blocks of very different magnitude (2^-30 .. 2^20), a matrix far from
    unit scale, exact zeros: the per-block scales keep every block at full precision."""
    rng = np.random.default_rng(9)
    m, k, n = 300, 512, 256
    a = rng.standard_normal((m, k)).astype(np.float32)
    a *= np.exp2(rng.integers(-30, 21, size=(m, k // 64))).repeat(64, axis=1).astype(np.float32)
    a[5] = 0.0
    a[:, 64:128] = 0.0
    w = (rng.standard_normal((k, n)) * 3e-4).astype(np.float32)
    want = a.astype(np.float64) @ w.astype(np.float64)
    got = project(2, a, w)
    ref = project(1, a, w)
    scale = np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64) + 1e-30
    assert float((np.abs(got - want) / scale).max()) < 2e-6
    assert float((np.abs(ref - want) / scale).max()) < 2e-6
    assert np.all(got[5] == 0.0)
