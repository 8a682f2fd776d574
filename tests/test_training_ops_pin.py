"""Pins oracle/training_ops.py (the numpy restatement of the CPU backend's training
operators) to the reference's own CPU plugin, compiled under oracle/_ref, on the same
inputs through the plugin ABI. Runs on CPU."""
import numpy as np
import pytest

from litnicelm_b200.plugin import Backend
from oracle import training_ops as T
from training_util import dense, read


@pytest.fixture(scope="module")
def cpu(oracle):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not present")
    b = Backend(oracle.REF_CPU_PLUGIN, device_kinds=(0,))
    yield b
    b.close()


def test_restatement_matches_the_reference_cpu_plugin(cpu):
    rng = np.random.default_rng(11)
    B, S, D, V = 2, 9, 16, 13
    x = rng.standard_normal((B, S, D)).astype(np.float32)
    dy = rng.standard_normal((B, S, D)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal((1, D))).astype(np.float32)
    _, xv = dense(cpu, x)
    _, dv = dense(cpu, dy)
    _, gv = dense(cpu, gamma)
    ob, ov = dense(cpu, np.zeros_like(x))
    gb, gvv = dense(cpu, np.zeros((1, D), np.float32))
    bb, bvv = dense(cpu, np.zeros((1, D), np.float32))
    cpu.call("layernorm_backward", xv, gv, dv, ov, gvv, bvv)
    dx, dg, db = T.layernorm_backward(x, gamma, dy)
    np.testing.assert_allclose(read(ob, ov), dx, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(read(gb, gvv)[0], dg, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(read(bb, bvv)[0], db, rtol=1e-5, atol=1e-5)

    logits = (rng.standard_normal((B, S, V)) * 3).astype(np.float32)
    targets = rng.integers(0, V, size=(B, S)).astype(np.int32)
    lb, lv = dense(cpu, logits)
    _, tv = dense(cpu, targets, dtype=1)
    sb, sv = dense(cpu, np.zeros((1, 1), np.float32))
    cpu.call("cross_entropy_mean_backward_inplace", lv, tv, sv)
    assert abs(float(read(sb, sv)[0, 0]) - float(T.cross_entropy_mean(logits, targets))) < 1e-6
    np.testing.assert_allclose(read(lb, lv), T.backward_from_logits_targets(logits, targets), rtol=1e-5, atol=1e-8)

    ids = rng.integers(0, V, size=(B, S)).astype(np.int32)
    tok0 = rng.standard_normal((V, D)).astype(np.float32)
    pos0 = rng.standard_normal((S, D)).astype(np.float32)
    _, iv = dense(cpu, ids, dtype=1)
    tb, tvv = dense(cpu, tok0)
    pb, pvv = dense(cpu, pos0)
    cpu.call("accumulate_embedding_grads", iv, xv, tvv, pvv)
    tok_w, pos_w = T.accumulate_embedding_grads(ids, x, tok0, pos0)
    assert np.array_equal(read(tb, tvv), tok_w) and np.array_equal(read(pb, pvv), pos_w)

    z = rng.standard_normal((B, S, S))
    sm = np.exp(z - z.max(-1, keepdims=True))
    sm = (sm / sm.sum(-1, keepdims=True)).astype(np.float32)
    dout = rng.standard_normal((B, S, S)).astype(np.float32)
    for name, causal in (("softmax_backward_rows", False), ("softmax_backward_causal_rows", True)):
        _, smv = dense(cpu, sm)
        _, dov = dense(cpu, dout)
        rb, rv = dense(cpu, np.zeros_like(sm))
        cpu.call(name, smv, dov, rv)
        np.testing.assert_allclose(read(rb, rv), T.softmax_backward_rows(sm, dout, causal), rtol=1e-5, atol=1e-6)

    w = rng.standard_normal((D, 3 * D)).astype(np.float32)
    g = rng.standard_normal((B, S, 3 * D)).astype(np.float32)
    _, wv = dense(cpu, w)
    _, gv2 = dense(cpu, g)
    rb, rv = dense(cpu, np.zeros_like(x))
    cpu.call("gemm_ranked_matrix_rhs_t", gv2, wv, rv)
    np.testing.assert_allclose(read(rb, rv), T.gemm_ranked_matrix_rhs_t(g, w), rtol=1e-4, atol=1e-4)
    wb, wvv = dense(cpu, np.zeros_like(w))
    cpu.call("gemm_ranked_reduce_lhs_t", xv, gv2, wvv)
    np.testing.assert_allclose(read(wb, wvv), T.gemm_ranked_reduce_lhs_t(x, g), rtol=1e-4, atol=1e-4)
    rb, rv = dense(cpu, np.zeros((1, 3 * D), np.float32))
    cpu.call("row_sum", gv2, rv)
    np.testing.assert_allclose(read(rb, rv)[0], T.row_sum(g), rtol=1e-5, atol=1e-5)
    assert abs(cpu.call("sum_squares_f32", gv2) - T.sum_squares(g)) < 1e-3
    pre = rng.standard_normal((B, S, D)).astype(np.float32)
    _, pv = dense(cpu, pre)
    rb, rv = dense(cpu, np.zeros_like(pre))
    cpu.call("relu_backward", pv, dv, rv)
    assert np.array_equal(read(rb, rv), T.relu_backward(pre, dy))

    p0 = rng.standard_normal((7, 5)).astype(np.float32)
    gg = rng.standard_normal((7, 5)).astype(np.float32)
    m0 = np.zeros((7, 5), np.float32)
    v0 = np.zeros((7, 5), np.float32)
    pb, pv = dense(cpu, p0)
    _, ggv = dense(cpu, gg)
    mb, mv = dense(cpu, m0)
    vb, vv = dense(cpu, v0)
    cpu.call("adamw_step", pv, ggv, mv, vv, 1, 0.002, 0.9, 0.999, 0.01, 1)
    pw, mw, vw = T.adamw_step(p0, gg, m0, v0, 1, 0.002, 0.9, 0.999, 0.01, 1)
    np.testing.assert_allclose(read(pb, pv), pw, rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(read(mb, mv), mw, rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(read(vb, vv), vw, rtol=1e-6, atol=1e-12)
