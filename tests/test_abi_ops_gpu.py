"""Per-operator parity of the plugin table against the oracle, through the C ABI.

Each test hands the B200 plugin the kinds of views the reference host builds in
inference (dense, prefix slices of max-size buffers, column slices of the qkv
buffer, in-place aliasing) and compares with the C restatement; where the
reference CPU plugin is available (oracle/_ref) it receives the identical views
too. Elementwise results must be bit-identical; reductions are compared within
a stated tolerance because the GPU sums in a different order.
"""
import os

import numpy as np
import pytest

from litnicelm_b200.plugin import Backend
from abi_util import Buffer, prefix_slice_view

pytestmark = pytest.mark.gpu

SEQ = [1, 5, 63, 64, 65]
S_MAX, D, H = 96, 64, 2
DH = D // H


@pytest.fixture(scope="module")
def be():
    b = Backend()
    assert b.device == 1
    yield b
    b.close()


@pytest.fixture(scope="module")
def cpu_plugin(oracle):
    if not oracle.have_ref():
        yield None
        return
    b = Backend(oracle.REF_CPU_PLUGIN, device_kinds=(0,))
    yield b
    b.close()


def both(be, cpu_plugin):
    return [p for p in (be, cpu_plugin) if p is not None]


@pytest.mark.parametrize("s", SEQ)
def test_elementwise_family_bit_exact(be, cpu_plugin, s):
    results = []
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(s)
        xb = Buffer(p, S_MAX * D * 4, rng)
        yb = Buffer(p, S_MAX * D * 4, rng)
        ob = Buffer(p, S_MAX * D * 4, fill=7.0)
        bias = Buffer(p, D * 4, rng)
        x = prefix_slice_view(xb, (1, S_MAX, D), s)
        y = prefix_slice_view(yb, (1, S_MAX, D), s)
        o = prefix_slice_view(ob, (1, S_MAX, D), s)
        bv = bias.view((1, D))
        xn, yn, bn = xb.np_view(x).copy(), yb.np_view(y).copy(), bias.np_view(bv).copy()
        out = {}
        p.call("add", x, y, o); ob.pull(); out["add"] = ob.np_view(o).copy()
        assert np.array_equal(out["add"], xn + yn)
        p.call("add_bias_rowwise", x, bv, o); ob.pull(); out["bias"] = ob.np_view(o).copy()
        assert np.array_equal(out["bias"], xn + bn)
        p.call("add_bias_relu_rowwise", x, bv, o); ob.pull(); out["bias_relu"] = ob.np_view(o).copy()
        assert np.array_equal(out["bias_relu"], np.maximum(xn + bn, 0))
        p.call("relu", x, o); ob.pull()
        assert np.array_equal(ob.np_view(o), np.maximum(xn, 0))
        p.call("mul_scalar", x, np.float32(0.125).item(), o); ob.pull()
        assert np.array_equal(ob.np_view(o), xn * np.float32(0.125))
        p.call("fill", o, 0.0); ob.pull()
        assert np.array_equal(ob.np_view(o), np.zeros_like(xn))
        # rows beyond the prefix are untouched
        assert np.all(ob.host.view(np.float32).reshape(S_MAX, D)[s:] == 7.0)
        # in place: add_bias_rowwise(out, b, out), add_bias_relu_rowwise_inplace
        p.call("add_bias_rowwise", x, bv, x); xb.pull()
        assert np.array_equal(xb.np_view(x), xn + bn)
        p.call("add_bias_relu_rowwise_inplace", y, bv); yb.pull()
        assert np.array_equal(yb.np_view(y), np.maximum(yn + bn, 0))
        results.append(out)
    if len(results) == 2:
        for k in results[0]:
            assert np.array_equal(results[0][k], results[1][k])


@pytest.mark.parametrize("s", SEQ)
def test_position_broadcast_add_and_embedding(be, cpu_plugin, s):
    V = 11
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(100 + s)
        table = Buffer(p, V * D * 4, rng)
        pos = Buffer(p, S_MAX * D * 4, rng)
        xb = Buffer(p, 2 * S_MAX * D * 4, fill=0.0)
        idb = Buffer(p, 2 * S_MAX * 4)
        ids = rng.integers(0, V, size=(2, s)).astype(np.int32)
        idv = idb.view((2, s), (S_MAX * 4, 4), dtype=1)
        idb.host.view(np.int32).reshape(2, S_MAX)[:, :s] = ids
        idb.push()
        x = prefix_slice_view(xb, (2, S_MAX, D), s)
        p.call("embedding_lookup", table.view((V, D)), idv, x)
        xb.pull()
        tn = table.host.view(np.float32).reshape(V, D)
        assert np.array_equal(xb.np_view(x), tn[ids])
        pv = pos.view((s, D))
        p.call("add", x, pv, x)  # X += pos[0:s] broadcast over the batch, in place
        xb.pull()
        assert np.array_equal(xb.np_view(x), tn[ids] + pos.host.view(np.float32).reshape(S_MAX, D)[:s][None])


@pytest.mark.parametrize("s", SEQ)
def test_layernorm(be, cpu_plugin, oracle, s):
    outs = []
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(200 + s)
        xb = Buffer(p, S_MAX * D * 4, rng)
        ob = Buffer(p, S_MAX * D * 4)
        g, b = Buffer(p, D * 4, rng), Buffer(p, D * 4, rng)
        x = prefix_slice_view(xb, (1, S_MAX, D), s)
        o = prefix_slice_view(ob, (1, S_MAX, D), s)
        p.call("layernorm_forward", x, g.view((1, D)), b.view((1, D)), o)
        ob.pull()
        want = oracle.layernorm(xb.np_view(x)[0], g.host.view(np.float32), b.host.view(np.float32))
        got = ob.np_view(o)[0]
        # double accumulation in both; only the summation order differs
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-6)
        outs.append(got.copy())
    if len(outs) == 2:
        np.testing.assert_allclose(outs[0], outs[1], rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("s", SEQ)
def test_softmax_variants(be, cpu_plugin, oracle, s):
    scale = np.float32(1.0 / np.sqrt(DH)).item()
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(300 + s)
        sb = Buffer(p, S_MAX * S_MAX * 4, rng)
        wb = Buffer(p, H * S_MAX * S_MAX * 4, fill=9.0)
        sc = sb.view((1, s, s), (S_MAX * S_MAX * 4, S_MAX * 4, 4))
        # weights_cache.select(0, h): [1, s, s] inside [H, 1, S, S]
        w = wb.view((1, s, s), (S_MAX * S_MAX * 4, S_MAX * 4, 4), offset=S_MAX * S_MAX * 4)
        x = sb.np_view(sc)[0].copy()
        p.call("scaled_causal_softmax_rows", sc, scale, w)
        wb.pull()
        got = wb.np_view(w)[0]
        want = oracle.scaled_causal_softmax_rows(x, scale)
        np.testing.assert_allclose(got, want, rtol=3e-6, atol=1e-7)
        assert np.all(np.triu(got, 1) == 0.0)
        np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-5)
        # reference attention: mul_scalar, mask(-1e9), softmax_rows, copy
        p.call("mul_scalar", sc, scale, sc)
        p.call("apply_causal_mask_inplace", sc, -1e9)
        sb.pull()
        masked = sb.np_view(sc)[0].copy()
        assert np.all(masked[np.triu_indices(s, 1)] == np.float32(-1e9))
        assert np.array_equal(np.tril(masked), np.tril(x * np.float32(scale)))
        p.call("softmax_rows", sc, w)
        wb.pull()
        got2 = wb.np_view(w)[0].copy()
        np.testing.assert_allclose(got2, oracle.softmax_rows(masked), rtol=3e-6, atol=1e-7)
        np.testing.assert_allclose(got2, want, rtol=3e-6, atol=1e-7)
        # in place, as the multistream variant does
        sb.host.view(np.float32).reshape(S_MAX, S_MAX)[:s, :s] = x
        sb.push()
        if p.device == 1:
            p.call("start_exec_context_iteration")
            p.call("start_exec_context_group")
            p.call("scaled_causal_softmax_rows_exec_context", sc, scale, sc)
            p.call("finish_exec_context_group")
            p.call("finish_exec_context_iteration")
        else:
            p.call("scaled_causal_softmax_rows", sc, scale, sc)
        sb.pull()
        np.testing.assert_allclose(sb.np_view(sc)[0], want, rtol=3e-6, atol=1e-7)


@pytest.mark.parametrize("s", SEQ)
def test_attention_gemms_on_qkv_slices(be, cpu_plugin, oracle, s):
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(400 + s)
        qkvb = Buffer(p, S_MAX * 3 * D * 4, rng)
        scb = Buffer(p, S_MAX * S_MAX * 4)
        ctxb = Buffer(p, S_MAX * D * 4, fill=0.0)
        st = (S_MAX * 3 * D * 4, 3 * D * 4, 4)
        h = 1
        q = qkvb.view((1, s, DH), st, offset=(0 * D + h * DH) * 4)
        k = qkvb.view((1, s, DH), st, offset=(1 * D + h * DH) * 4)
        v = qkvb.view((1, s, DH), st, offset=(2 * D + h * DH) * 4)
        sc = scb.view((1, s, s), (S_MAX * S_MAX * 4, S_MAX * 4, 4))
        ctx = ctxb.view((1, s, DH), (S_MAX * D * 4, D * 4, 4), offset=h * DH * 4)
        p.call("gemm_batched_rhs_t", q, k, sc)
        scb.pull()
        got = scb.np_view(sc)[0].copy()
        want = oracle.gemm_rhs_t(qkvb.np_view(q)[0], qkvb.np_view(k)[0])
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
        p.call("gemm_batched", sc, v, ctx)
        ctxb.pull()
        want2 = oracle.gemm(got, qkvb.np_view(v)[0])
        np.testing.assert_allclose(ctxb.np_view(ctx)[0], want2, rtol=1e-5, atol=1e-4)
        # the other head's columns of the context stay untouched
        assert np.all(ctxb.host.view(np.float32).reshape(S_MAX, D)[:, :DH] == 0.0)


@pytest.mark.parametrize("s,k,n", [(1, 64, 192), (5, 64, 96), (63, 256, 64), (64, 64, 8), (65, 100, 37),
                                    (300, 64, 256)])
def test_projection_gemm(be, cpu_plugin, oracle, s, k, n):
    smax = max(s, 8) + 3
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(500 + s)
        ab = Buffer(p, smax * k * 4, rng)
        wb = Buffer(p, k * n * 4, rng)
        ob = Buffer(p, smax * n * 4, fill=5.0)
        a = prefix_slice_view(ab, (1, smax, k), s)
        o = prefix_slice_view(ob, (1, smax, n), s)
        p.call("gemm_ranked_matrix_rhs", a, wb.view((k, n)), o)
        ob.pull()
        want = oracle.gemm(ab.np_view(a)[0], wb.host.view(np.float32).reshape(k, n))
        np.testing.assert_allclose(ob.np_view(o)[0], want, rtol=2e-5, atol=2e-5 * np.sqrt(k))
        assert np.all(ob.host.view(np.float32).reshape(smax, n)[s:] == 5.0)


def test_copy_dense_and_strided(be, cpu_plugin):
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(7)
        a = Buffer(p, 40 * 24 * 4, rng)
        b = Buffer(p, 40 * 24 * 4)
        p.call("copy", a.view((40, 24)), b.view((40, 24)))
        b.pull()
        assert np.array_equal(b.host, a.host)
        c = Buffer(p, 40 * 24 * 4, fill=1.0)
        src = a.view((10, 8), (24 * 4, 4), offset=4 * 4)
        dst = c.view((10, 8), (24 * 4, 4), offset=8 * 4)
        p.call("copy", src, dst)
        c.pull()
        assert np.array_equal(c.np_view(dst), a.np_view(src))


def test_rank3_strided_copy_is_superset_of_reference(be, cpu_plugin):
    """For a non-dense rank-3 view the CPU backend walks dims 0 and 1 only
    (device_backend.cpp:725-731); the plugin copies the whole logical view, so
    every element the reference writes must hold the same value."""
    s = 5
    outs = {}
    for p in both(be, cpu_plugin):
        rng = np.random.default_rng(8)
        a = Buffer(p, S_MAX * S_MAX * 4, rng)
        b = Buffer(p, S_MAX * S_MAX * 4, fill=-3.0)
        st = (S_MAX * S_MAX * 4, S_MAX * 4, 4)
        p.call("copy", a.view((1, s, s), st), b.view((1, s, s), st))
        b.pull()
        outs[p.device] = (b.host.view(np.float32).reshape(S_MAX, S_MAX).copy(),
                          a.host.view(np.float32).reshape(S_MAX, S_MAX).copy())
    got, src = outs[1]
    assert np.array_equal(got[:s, :s], src[:s, :s])
    assert np.all(got[s:] == -3.0) and np.all(got[:s, s:] == -3.0)
    if 0 in outs:
        ref, _ = outs[0]
        written = ref != -3.0
        assert np.array_equal(got[written], ref[written])


def test_memory_info_and_alloc(be):
    info = be.api.memory_info(be.h)
    assert info.available == 1 and 0 < info.free_bytes <= info.total_bytes
    assert info.total_bytes > 100 * 2**30  # a B200 carries 180 GB
    assert be.api.alloc(be.h, 0, 64) in (None, 0)
    p = be.alloc(1000, 1024)
    assert p % 1024 == 0
    assert be.api.supports_exec_context_iteration(be.h) == 1


def test_row_by_row_read_back_sees_every_device_write(be):
    """The reference reads logits one row per copy_device2host call
    (host_tensor_stage.hpp:101-125); the plugin answers such a walk from one
    read-ahead transfer. Every row must still be what the device holds at that
    moment: after a host upload, after a kernel wrote, walking to the very end
    of an allocation, and reading backwards."""
    rows, cols = 1024, 96
    rng = np.random.default_rng(11)
    buf = Buffer(be, rows * cols * 4, rng=rng)
    want = buf.host.view(np.float32).reshape(rows, cols).copy()

    def row(r):
        return be.download(buf.ptr, cols * 4, offset=r * cols * 4).view(np.float32)

    for r in range(300):  # forward walk: served from the read-ahead after the second call
        assert np.array_equal(row(r), want[r]), r
    # a host upload invalidates what was fetched ahead
    want[310:320] = rng.standard_normal((10, cols)).astype(np.float32)
    be.upload(buf.ptr, want[310:320], offset=310 * cols * 4)
    for r in range(300, 330):
        assert np.array_equal(row(r), want[r]), r
    # so does a kernel: fill rows 400..499 with a constant between two reads of the walk
    for r in range(330, 350):
        assert np.array_equal(row(r), want[r]), r
    t = buf.view((100, cols), offset=400 * cols * 4)
    be.call("fill", t, 2.5)
    want[400:500] = 2.5
    for r in range(350, 520):
        assert np.array_equal(row(r), want[r]), r
    # to the last row of the allocation, then backwards and at random
    for r in range(900, rows):
        assert np.array_equal(row(r), want[r]), r
    for r in [1023, 1000, 5, 700, 699, 698, 0]:
        assert np.array_equal(row(r), want[r]), r
    # a walk with a stride larger than the row (column slice of a wider tensor)
    for r in range(0, 1000, 7):
        got = be.download(buf.ptr, 16, offset=r * cols * 4 + 32).view(np.float32)
        assert np.array_equal(got, want[r, 8:12]), r
