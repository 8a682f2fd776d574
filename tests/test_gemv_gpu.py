"""Few-row products (the M <= 8 case of gemm_ranked_matrix_rhs,
device_backend.cpp:1112-1131, as the output head calls it on the last rows,
output_head.cpp:58-70) against the oracle, through the C ABI. Covers the
streaming kernel (TMA-staged ring) with both tile widths, with and without a
split of k, ragged ends of k and n, and the plain kernel that takes shapes TMA
cannot address.

Tolerance: the kernels add the k products in a different order than the
reference's sequential fp32 loop, so results agree to fp32 rounding of a sum of
k terms: |diff| <= 2e-5 * sqrt(k) * max|x| * max|w| per element.
"""
import numpy as np
import pytest

from litnicelm_b200.plugin import gemv_host

pytestmark = pytest.mark.gpu

SHAPES = [
    # m, k, n
    (1, 1024, 32000),   # config-4/5 head: 128-column tiles, no split
    (8, 1024, 32000),
    (1, 512, 1536),     # config-2 QKV as one row: 256-column tiles, k split
    (2, 2048, 512),     # config-2 W2
    (4, 512, 2048),
    (1, 4096, 1024),    # config-5 W2: long k
    (3, 1000, 512),     # k not a multiple of a stage, m padded to 4
    (1, 512, 1000),     # n not a multiple of the tile
    (8, 36, 132),       # one ragged stage, one ragged tile
    (1, 512, 96),       # config-2 head: narrower than a tile, plain kernel
    (5, 301, 50),       # nothing aligned: plain kernel, scalar loads
    (1, 64, 8),
]


@pytest.mark.parametrize("m,k,n", SHAPES)
@pytest.mark.parametrize("epilogue", ["none", "bias", "bias+residual+relu"])
def test_gemv_matches_oracle(oracle, m, k, n, epilogue):
    rng = np.random.default_rng(m * 7919 + k * 31 + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (rng.standard_normal((k, n), dtype=np.float32) * 0.02).astype(np.float32)
    b = rng.standard_normal(n, dtype=np.float32) if epilogue != "none" else None
    r = rng.standard_normal((m, n), dtype=np.float32) if "residual" in epilogue else None
    want = oracle.gemm(x, w)
    if b is not None:
        want = want + b[None, :]          # add_bias_rowwise
    if r is not None:
        want = np.maximum(want + r, 0)    # add, then relu
    got = gemv_host(x, w, b, r, relu=r is not None)
    tol = 2e-5 * np.sqrt(k) * float(np.abs(x).max()) * float(np.abs(w).max())
    assert got.shape == want.shape
    assert float(np.abs(got - want).max()) <= tol


def test_gemv_is_repeatable():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 1024), dtype=np.float32)
    w = rng.standard_normal((1024, 3072), dtype=np.float32)
    assert np.array_equal(gemv_host(x, w), gemv_host(x, w))


def test_a_wait_that_nothing_completes_gives_up_and_reports():
    """Every mbarrier wait of the library's kernels is bounded. The self-test kernel
    (one CTA, a barrier nobody arrives on, limit 500 microseconds) must return by
    itself with the wait-timeout code in the host-visible error word, and the
    device must still work afterwards."""
    import ctypes as C
    from litnicelm_b200.plugin import load_library
    lib = load_library()
    fn = lib.litnice_b200_selftest_wait_timeout
    fn.argtypes = [C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_double)]
    fn.restype = C.c_int
    code, detail, waited = C.c_int32(-1), C.c_int32(-1), C.c_double(0)
    assert fn(500, C.byref(code), C.byref(detail), C.byref(waited)) == 0
    assert code.value == 2 and detail.value == 99     # DEVERR_WAIT_TIMEOUT, the test's wait site
    assert 500.0 <= waited.value < 50000.0
    assert fn(5000, C.byref(code), C.byref(detail), C.byref(waited)) == -1   # limits above 1 ms are refused
    x = np.ones((1, 64), np.float32)
    assert np.array_equal(gemv_host(x, np.ones((64, 8), np.float32)), np.full((1, 8), 64.0, np.float32))


@pytest.mark.parametrize("m,k,n", [(1, 512, 1536), (1, 512, 2048), (8, 1024, 32000), (3, 1000, 512), (1, 1024, 4096)])
def test_layernorm_on_the_way_in_matches_oracle(oracle, m, k, n):
    """layernorm_forward followed by gemm_ranked_matrix_rhs + add_bias_rowwise + relu
    (transformer_layer.cpp:58-60,84 and the FFN) as one kernel: the statistics keep the
    reference's widths, so the normalised rows equal the stand-alone LayerNorm's and the
    product differs from the oracle's only by its summation order."""
    rng = np.random.default_rng(k + n)
    x = (rng.standard_normal((m, k)) * 2 + 0.5).astype(np.float32)
    w = (rng.standard_normal((k, n), dtype=np.float32) * 0.02).astype(np.float32)
    b = rng.standard_normal(n, dtype=np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(k)).astype(np.float32)
    xn = oracle.layernorm(x, gamma, beta)
    want = np.maximum(oracle.gemm(xn, w) + b[None, :], 0)
    got = gemv_host(x, w, b, relu=True, ln=(gamma, beta))
    tol = 2e-5 * np.sqrt(k) * float(np.abs(xn).max()) * float(np.abs(w).max())
    assert float(np.abs(got - want).max()) <= tol
    # and bit-identical to the same kernel fed the oracle's normalised rows
    assert np.array_equal(got, gemv_host(xn, w, b, relu=True))
