"""The bound behind the fixed per-head scales of the fp16-pair attention operands.

The attention kernel (csrc/attention_tc16.cu) stores Q, K and V as fp16 pairs under one
power-of-two scale per head that is derived from the weights alone: for every input row,
    |LN(x) W[:, c] + b[c]| <= sqrt(D) * |gamma * W[:, c]|_2 + |beta . W[:, c] + b[c]|
because the normalised row xhat of layernorm_forward (device_backend.cpp:1247-1279: biased
variance, eps added to it) has |xhat|_2 <= sqrt(D). This test checks the inequality itself, in
numpy, on inputs chosen to stress it (constant rows, one huge element, tiny variance, aligned
with a weight column), and that the scale derived from it keeps every value inside fp16.
"""
import numpy as np

D, N = 64, 192


def layernorm(x, gamma, beta, eps=1e-5):
    mean = x.mean(axis=1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * gamma + beta


def bound(w, gamma, beta, bias):
    gw = gamma[:, None] * w
    return np.sqrt(D) * np.sqrt((gw * gw).sum(axis=0)) + np.abs(beta @ w + bias)


def head_scale(col_bounds):
    """Power of two that puts the largest bound of 64 columns into [2^14, 2^15)."""
    am = col_bounds.reshape(-1, 64).max(axis=1) * 1.001
    return 2.0 ** (14 - np.floor(np.log2(am)))


def test_bound_holds_for_adversarial_rows():
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.05, size=(D, N)) * np.repeat([40.0, 1e-3, 1.0], 64)[None, :]
    gamma = 1.0 + rng.normal(0, 0.5, size=D)
    beta = rng.normal(0, 2.0, size=D)
    bias = rng.normal(0, 0.3, size=N)
    rows = [rng.normal(0, s, size=(64, D)) for s in (1e-6, 1.0, 1e4)]
    spike = np.zeros((D, D))
    spike[np.arange(D), np.arange(D)] = 1e6                      # one huge element per row
    rows.append(spike)
    rows.append(np.full((4, D), 3.25) + rng.normal(0, 1e-7, size=(4, D)))   # nearly constant rows
    aligned = (gamma[:, None] * w).T[:32]                        # rows along the scaled weight columns
    rows.append(aligned * 1e3)
    x = np.concatenate(rows)
    y = layernorm(x, gamma, beta) @ w + bias
    b = bound(w, gamma, beta, bias)
    assert (np.abs(y) <= b[None, :] * (1 + 1e-9)).all()
    # the aligned rows come close to it: the bound is not vacuous
    assert (np.abs(y[-32:]) / b[None, :]).max() > 0.5


def test_scale_keeps_every_value_inside_fp16():
    rng = np.random.default_rng(12)
    w = rng.normal(0, 0.02, size=(D, N)) * np.repeat([1.0, 300.0, 1e-4], 64)[None, :]
    gamma, beta, bias = np.ones(D), rng.normal(0, 1.0, size=D), np.zeros(N)
    b = bound(w, gamma, beta, bias)
    s = head_scale(b)
    scaled_bound = (b.reshape(-1, 64).max(axis=1) * 1.001) * s
    assert ((scaled_bound >= 2.0 ** 14) & (scaled_bound < 2.0 ** 15)).all()
    x = rng.normal(0, 1.0, size=(256, D))
    y = (layernorm(x, gamma, beta) @ w + bias) * np.repeat(s, 64)[None, :]
    assert np.abs(y).max() < 65504.0
    # a pair of halves carries the usual values with 22 bits: relative error below 2^-21
    hi = y.astype(np.float16).astype(np.float64)
    lo = (y - hi).astype(np.float16).astype(np.float64)
    big = np.abs(y) >= 2.0 ** -3
    assert (np.abs(hi + lo - y)[big] / np.abs(y)[big]).max() < 2.0 ** -21
