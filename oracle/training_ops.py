"""Test infrastructure, not product code.

numpy restatement of the training operators of litnicelm's CPU backend
(src/model/backend/device_backend.cpp; lines cited per function), used to check
the CUDA training entries of the plugin table. Widths follow the reference:
float64 where it accumulates in double, float32 where it accumulates in float
(sequential float32 sums are restated with float64 sums and compared within a
tolerance; where the order matters for bit-exactness the loop is kept).

Pin: tests/test_training_ops_pin.py runs the reference's own CPU plugin
(oracle/_ref/liblitnice_backend_cpu.so) on the same inputs and compares.
"""
from __future__ import annotations

import numpy as np


def sum_squares(x):  # :966-976
    return np.float32(np.sum(x.astype(np.float64) ** 2))


def relu_backward(preact, dout):  # :1003-1060
    return np.where(preact > 0, dout, np.float32(0)).astype(np.float32)


def row_sum(x):  # :1062-1094, float sums over every leading index
    return x.reshape(-1, x.shape[-1]).astype(np.float64).sum(axis=0).astype(np.float32)


def gemm_ranked_matrix_rhs_t(a, b):  # :1133-1152
    return np.einsum("...rk,ck->...rc", a.astype(np.float64), b.astype(np.float64)).astype(np.float32)


def gemm_ranked_reduce_lhs_t(a, b):  # :1154-1173
    k = a.shape[-2]
    return (a.reshape(-1, k, a.shape[-1]).astype(np.float64).transpose(0, 2, 1) @
            b.reshape(-1, k, b.shape[-1]).astype(np.float64)).sum(axis=0).astype(np.float32)


def gemm_batched_lhs_t(a, b):  # :1195-1214
    return (a.astype(np.float64).swapaxes(-1, -2) @ b.astype(np.float64)).astype(np.float32)


def layernorm_backward(x, gamma, dout):  # :1281-1343
    d = x.shape[-1]
    x2 = x.reshape(-1, d).astype(np.float64)
    dy = dout.reshape(-1, d).astype(np.float64)
    g = gamma.reshape(-1).astype(np.float64)
    mean = x2.mean(axis=1, keepdims=True)
    var = ((x2 - mean) ** 2).mean(axis=1, keepdims=True)
    inv_std = 1.0 / np.sqrt(var + np.float64(np.float32(1e-5)))
    xhat = (x2 - mean) * inv_std
    dxhat = dy * g
    s1 = dxhat.sum(axis=1, keepdims=True)
    s2 = (dxhat * xhat).sum(axis=1, keepdims=True)
    dx = (inv_std / d) * (d * dxhat - s1 - xhat * s2)
    dgamma = (dy * xhat).astype(np.float32).astype(np.float64).sum(axis=0)
    dbeta = dy.sum(axis=0)
    return dx.astype(np.float32).reshape(x.shape), dgamma.astype(np.float32), dbeta.astype(np.float32)


def accumulate_embedding_grads(ids, d_cur, d_tok, d_pos):  # :1368-1389, in token order, float32
    d_tok, d_pos = d_tok.copy(), d_pos.copy()
    flat = ids.reshape(-1)
    seq = ids.shape[-1]
    cur = d_cur.reshape(-1, d_cur.shape[-1])
    for t, idx in enumerate(flat):
        d_tok[int(idx)] = d_tok[int(idx)] + cur[t]
        d_pos[t % seq] = d_pos[t % seq] + cur[t]
    return d_tok, d_pos


def cross_entropy_mean(logits, targets):  # :1391-1417
    v = logits.shape[-1]
    lg = logits.reshape(-1, v)
    tg = targets.reshape(-1).astype(np.int64)
    m = lg.max(axis=1)
    lse = np.exp((lg - m[:, None]).astype(np.float64)).sum(axis=1)
    per = (m.astype(np.float64) + np.log(lse)) - lg[np.arange(len(tg)), tg].astype(np.float64)
    return np.float32(per.sum() / len(tg))


def backward_from_logits_targets(logits, targets):  # :1430-1464
    v = logits.shape[-1]
    lg = logits.reshape(-1, v)
    tg = targets.reshape(-1).astype(np.int64)
    m = lg.max(axis=1, keepdims=True)
    e = np.exp((lg - m).astype(np.float64))
    p = (e / e.sum(axis=1, keepdims=True)).astype(np.float32)
    p[np.arange(len(tg)), tg] -= np.float32(1.0)
    return (p * (np.float32(1.0) / np.float32(len(tg)))).astype(np.float32).reshape(logits.shape)


def softmax_backward_rows(sm, dout, causal=False):  # :1519-1552, :1649-1673
    cols = sm.shape[-1]
    s = sm.reshape(-1, cols).astype(np.float64)
    g = dout.reshape(-1, cols).astype(np.float64)
    if causal:
        live = np.arange(cols)[None, :] <= (np.arange(s.shape[0]) % cols)[:, None]
    else:
        live = np.ones_like(s, dtype=bool)
    dot = np.where(live, s * g, 0.0).sum(axis=1, keepdims=True)
    return np.where(live, s * (g - dot), 0.0).astype(np.float32).reshape(sm.shape)


def adamw_step(p, g, m, v, step, lr, beta1, beta2, weight_decay, apply_decay):  # :1699-1750, float32 throughout
    f = np.float32
    p, m, v = p.astype(f).copy(), m.astype(f).copy(), v.astype(f).copy()
    lr, beta1, beta2, weight_decay = f(lr), f(beta1), f(beta2), f(weight_decay)
    b1c = f(1.0) - f(np.float64(beta1) ** float(step))
    b2c = f(1.0) - f(np.float64(beta2) ** float(step))
    m[...] = beta1 * m + (f(1.0) - beta1) * g
    v[...] = beta2 * v + (f(1.0) - beta2) * g * g
    mhat = m / b1c
    vhat = v / b2c
    adam = mhat / (np.sqrt(vhat) + f(1e-8))
    decay = weight_decay * p if apply_decay else np.zeros_like(p)
    p[...] = p - lr * (adam + decay)
    return p, m, v
