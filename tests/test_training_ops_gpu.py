"""Training entries of the plugin table (the operators `litnicelm train` calls)
against the oracle's restatement of the CPU backend and, where oracle/_ref is
present, against the reference CPU plugin on identical views, through the C
ABI. Tolerances: elementwise operators and the optimiser step must be
bit-identical; the embedding-gradient scatter keeps the CPU order and must be
bit-identical; reductions (sums the CPU code runs as one sequential loop) are
compared within 2e-5 relative to the magnitude of the summed terms.
"""
import numpy as np
import pytest

from litnicelm_b200.plugin import Backend
from oracle import training_ops as T
from training_util import child_raises, dense, read, sliced

pytestmark = pytest.mark.gpu

B, S, S_MAX, D, V = 3, 20, 32, 48, 37


@pytest.fixture(scope="module")
def be():
    b = Backend()
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


def plugins(be, cpu_plugin):
    return [p for p in (be, cpu_plugin) if p is not None]


def close(got, want, terms=1.0, scale=None):
    scale = float(np.abs(want).max()) if scale is None else scale
    tol = 2e-5 * max(scale, 1e-6) * max(1.0, np.sqrt(terms))
    assert float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max()) <= tol


def test_sum_squares(be, cpu_plugin):
    x = np.random.default_rng(1).standard_normal((1, 70001)).astype(np.float32)
    want = T.sum_squares(x)
    for p in plugins(be, cpu_plugin):
        _, xv = dense(p, x)
        got = p.call("sum_squares_f32", xv)
        assert abs(got - want) <= 1e-6 * want


@pytest.mark.parametrize("slices", [False, True])
def test_relu_backward_bit_exact(be, cpu_plugin, slices):
    rng = np.random.default_rng(2)
    pre = rng.standard_normal((B, S, D)).astype(np.float32)
    dout = rng.standard_normal((B, S, D)).astype(np.float32)
    want = T.relu_backward(pre, dout)
    mk = (lambda p, a: sliced(p, a, S_MAX)) if slices else dense
    for p in plugins(be, cpu_plugin):
        (_, pv), (_, dv), (ob, ov) = mk(p, pre), mk(p, dout), mk(p, np.zeros_like(pre))
        p.call("relu_backward", pv, dv, ov)
        assert np.array_equal(read(ob, ov), want)
        db, dv2 = mk(p, dout)
        p.call("relu_backward_inplace", pv, dv2)
        assert np.array_equal(read(db, dv2), want)


@pytest.mark.parametrize("rows", [1, 7, 64, 1000])
def test_row_sum(be, cpu_plugin, rows):
    x = np.random.default_rng(rows).standard_normal((rows, D + 3)).astype(np.float32)
    want = T.row_sum(x)
    for p in plugins(be, cpu_plugin):
        _, xv = dense(p, x)
        ob, ov = dense(p, np.zeros((1, D + 3), np.float32))
        p.call("row_sum", xv, ov)
        close(read(ob, ov)[0], want, terms=rows, scale=1.0)
    xs = x[:B * S].reshape(B, S, D + 3) if rows >= B * S else None
    if xs is not None:
        _, xv = sliced(be, xs, S_MAX)
        ob, ov = dense(be, np.zeros((1, D + 3), np.float32))
        be.call("row_sum", xv, ov)
        close(read(ob, ov)[0], T.row_sum(xs), terms=B * S, scale=1.0)


def test_weight_gradient_products(be, cpu_plugin):
    rng = np.random.default_rng(4)
    a = rng.standard_normal((B, S, D)).astype(np.float32)       # activations
    g = rng.standard_normal((B, S, 2 * D)).astype(np.float32)   # upstream gradient
    w = rng.standard_normal((D, 2 * D)).astype(np.float32)      # weight [in, out]
    for p in plugins(be, cpu_plugin):
        _, av = sliced(p, a, S_MAX)
        _, gv = sliced(p, g, S_MAX)
        _, wv = dense(p, w)
        ob, ov = sliced(p, np.zeros_like(a), S_MAX)
        p.call("gemm_ranked_matrix_rhs_t", gv, wv, ov)          # dX = dY W^T
        close(read(ob, ov), T.gemm_ranked_matrix_rhs_t(g, w), terms=2 * D, scale=1.0)
        wb, wo = dense(p, np.zeros_like(w))
        p.call("gemm_ranked_reduce_lhs_t", av, gv, wo)          # dW = sum_b X^T dY
        close(read(wb, wo), T.gemm_ranked_reduce_lhs_t(a, g), terms=B * S, scale=1.0)
        q = rng.standard_normal((B, S, 16)).astype(np.float32)
        _, qv = sliced(p, q, S_MAX)
        sb, sv = dense(p, np.zeros((B, 16, D), np.float32))
        p.call("gemm_batched_lhs_t", qv, av, sv)                # per-batch Q^T X
        close(read(sb, sv), T.gemm_batched_lhs_t(q, a), terms=S, scale=1.0)


def test_layernorm_backward(be, cpu_plugin):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((B, S, D)) * 3 + 1).astype(np.float32)
    dy = rng.standard_normal((B, S, D)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal((1, D))).astype(np.float32)
    dx_w, dg_w, db_w = T.layernorm_backward(x, gamma, dy)
    for p in plugins(be, cpu_plugin):
        _, xv = sliced(p, x, S_MAX)
        _, dv = sliced(p, dy, S_MAX)
        _, gv = dense(p, gamma)
        ob, ov = sliced(p, np.zeros_like(x), S_MAX)
        gb, gvv = dense(p, np.full((1, D), 9.0, np.float32))
        bb, bvv = dense(p, np.full((1, D), 9.0, np.float32))
        p.call("layernorm_backward", xv, gv, dv, ov, gvv, bvv)
        close(read(ob, ov), dx_w, terms=1)
        close(read(gb, gvv)[0], dg_w, terms=B * S, scale=1.0)
        close(read(bb, bvv)[0], db_w, terms=B * S, scale=1.0)


@pytest.mark.parametrize("ids_dtype", [np.int32, np.float32])
def test_embedding_gradients_bit_exact(be, cpu_plugin, ids_dtype):
    rng = np.random.default_rng(6)
    ids = rng.integers(0, V, size=(B, S))
    ids[0, :5] = 3                       # repeats: the order of the additions matters
    d_cur = rng.standard_normal((B, S, D)).astype(np.float32)
    tok0 = rng.standard_normal((V, D)).astype(np.float32)
    pos0 = rng.standard_normal((S_MAX, D)).astype(np.float32)
    tok_w, pos_w = T.accumulate_embedding_grads(ids, d_cur, tok0, pos0)
    for p in plugins(be, cpu_plugin):
        _, iv = dense(p, ids.astype(ids_dtype), dtype=1 if ids_dtype == np.int32 else 0)
        _, cv = sliced(p, d_cur, S_MAX)
        tb, tv = dense(p, tok0)
        pb, pv = dense(p, pos0)
        p.call("accumulate_embedding_grads", iv, cv, tv, pv)
        assert np.array_equal(read(tb, tv), tok_w)
        assert np.array_equal(read(pb, pv), pos_w)


def test_cross_entropy_and_its_gradient(be, cpu_plugin):
    rng = np.random.default_rng(7)
    logits = (rng.standard_normal((B, S, V)) * 4).astype(np.float32)
    targets = rng.integers(0, V, size=(B, S)).astype(np.int32)
    loss_w = T.cross_entropy_mean(logits, targets)
    grad_w = T.backward_from_logits_targets(logits, targets)
    for p in plugins(be, cpu_plugin):
        _, tv = dense(p, targets, dtype=1)
        lb, lv = sliced(p, logits, S_MAX)
        ob, ov = dense(p, np.zeros((1, 1), np.float32))
        p.call("cross_entropy_mean", lv, tv, ov)
        assert abs(float(read(ob, ov)[0, 0]) - float(loss_w)) <= 2e-6 * abs(float(loss_w))
        assert abs(p.call("read_scalar_f32", ov) - float(loss_w)) <= 2e-6 * abs(float(loss_w))
        assert np.array_equal(read(lb, lv), logits)              # the loss alone leaves the logits
        p.call("backward_from_logits_targets", lv, tv)
        close(read(lb, lv), grad_w, terms=1, scale=1.0 / (B * S))
        lb2, lv2 = sliced(p, logits, S_MAX)
        ob2, ov2 = dense(p, np.zeros((1, 1), np.float32))
        p.call("cross_entropy_mean_backward_inplace", lv2, tv, ov2)
        assert abs(float(read(ob2, ov2)[0, 0]) - float(loss_w)) <= 2e-6 * abs(float(loss_w))
        close(read(lb2, lv2), grad_w, terms=1, scale=1.0 / (B * S))


def test_cross_entropy_target_out_of_range_is_reported():
    """The CPU backend throws at once; here the kernel records the bad target and the next
    synchronising call (read_scalar_f32, as the training loop issues every step) throws."""
    child_raises("""
logits = np.zeros((1, 4, 37), np.float32)
targets = np.array([[0, 1, 39, 3]], np.int32)
_, tv = dense(be, targets, dtype=1)
_, lv = dense(be, logits)
ob, ov = dense(be, np.zeros((1, 1), np.float32))
be.call("cross_entropy_mean", lv, tv, ov)
be.call("read_scalar_f32", ov)
""", "target out of range (target=39)")


def test_uniform_logits_give_log_vocab(be):
    logits = np.zeros((1, 4, V), np.float32)
    targets = np.array([[0, 1, 2, 3]], np.int32)
    _, tv = dense(be, targets, dtype=1)
    _, lv = dense(be, logits)
    ob, ov = dense(be, np.zeros((1, 1), np.float32))
    be.call("cross_entropy_mean", lv, tv, ov)
    assert abs(be.call("read_scalar_f32", ov) - np.log(V)) < 1e-5


@pytest.mark.parametrize("causal", [False, True])
def test_softmax_backward(be, cpu_plugin, causal):
    rng = np.random.default_rng(8)
    T_ = 24
    z = rng.standard_normal((B, T_, T_)).astype(np.float64)
    if causal:
        z = np.where(np.tril(np.ones((T_, T_), bool)), z, -np.inf)
    sm = np.exp(z - z.max(axis=-1, keepdims=True))
    sm = (sm / sm.sum(axis=-1, keepdims=True)).astype(np.float32)
    dout = rng.standard_normal((B, T_, T_)).astype(np.float32)
    want = T.softmax_backward_rows(sm, dout, causal)
    name = "softmax_backward_causal_rows" if causal else "softmax_backward_rows"
    for p in plugins(be, cpu_plugin):
        _, sv = dense(p, sm)
        _, dv = dense(p, dout)
        ob, ov = dense(p, np.full_like(sm, 3.0))
        p.call(name, sv, dv, ov)
        close(read(ob, ov), want, terms=T_, scale=1.0)
    if causal:  # the lane variant of the multistream attention, inside an open group
        _, sv = dense(be, sm)
        _, dv = dense(be, dout)
        ob, ov = dense(be, np.full_like(sm, 3.0))
        be.call("start_exec_context_iteration")
        be.call("start_exec_context_group")
        be.call("softmax_backward_causal_rows_exec_context", sv, dv, ov)
        q = rng.standard_normal((B, T_, 16)).astype(np.float32)
        _, qv = dense(be, q)
        gb, gv = dense(be, np.zeros((B, 16, T_), np.float32))
        be.call("gemm_batched_lhs_t_exec_context", qv, dv, gv)
        be.call("finish_exec_context_group")
        be.call("finish_exec_context_iteration")
        close(read(ob, ov), want, terms=T_, scale=1.0)
        close(read(gb, gv), T.gemm_batched_lhs_t(q, dout), terms=T_, scale=1.0)


@pytest.mark.parametrize("apply_decay", [0, 1])
def test_adamw_step_bit_exact(be, cpu_plugin, apply_decay):
    rng = np.random.default_rng(9)
    shape = (129, 77)
    p0 = rng.standard_normal(shape).astype(np.float32)
    g = (rng.standard_normal(shape) * 0.1).astype(np.float32)
    m0 = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    v0 = (rng.random(shape) * 0.001).astype(np.float32)
    results = []
    for p in plugins(be, cpu_plugin):
        pb, pv = dense(p, p0)
        _, gv = dense(p, g)
        mb, mv = dense(p, m0)
        vb, vv = dense(p, v0)
        for step in (1, 2, 3):
            p.call("adamw_step", pv, gv, mv, vv, step, 0.002, 0.9, 0.999, 0.01, apply_decay)
        results.append((read(pb, pv), read(mb, mv), read(vb, vv)))
    want = (p0, m0, v0)
    for step in (1, 2, 3):
        want = T.adamw_step(want[0], g, want[1], want[2], step, 0.002, 0.9, 0.999, 0.01, apply_decay)
    if len(results) == 2:  # the reference CPU plugin itself: bit for bit
        for a, b in zip(results[0], results[1]):
            assert np.array_equal(a, b)
    for a, b in zip(results[0], want):
        np.testing.assert_allclose(a, b, rtol=2e-6, atol=1e-9)


def test_misuse_is_refused_with_the_cpu_backends_messages():
    child_raises("""
_, pv = dense(be, np.ones((4, 4), np.float32))
be.call("adamw_step", pv, pv, pv, pv, 0, 0.002, 0.9, 0.999, 0.01, 0)
""", "adamw_step: step must be >= 1")
    child_raises("""
_, sv = dense(be, np.ones((1, 4, 4), np.float32))
be.call("softmax_backward_causal_rows_exec_context", sv, sv, sv)
""", "no exec context group is open")
