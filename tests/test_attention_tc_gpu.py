"""Tensor-core attention (head dimension 64) against the oracle and against the
fp32 SIMT attention kernel, through the C ABI's native forward and token loop.

Shapes are chosen around the kernel's 128-row tiles and around its two
schedules: key ranges cut over several CTAs (few streams x heads) and one CTA
walking several key tiles (many streams x heads).
"""
import os

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import Session

pytestmark = pytest.mark.gpu

LOGIT_RTOL = 1e-3   # the path's stated tolerance against the oracle
KERNEL_RTOL = 1e-4  # two fp32-accurate kernels against each other
NEAR_TIE = 1e-4

DIMS = formats.ModelDims(2, 2, 128, 256, 96, 1024)  # L, H, D, F, V, S: head dimension 64


def rel_err(got, want):
    scale = np.maximum(np.abs(want).max(axis=-1, keepdims=True), 1e-6)
    return float((np.abs(got - want) / scale).max())


@pytest.fixture(scope="module")
def arena():
    return formats.make_param_arena(DIMS, 1234, bias_std=0.02)


class simt_attention:
    """Sessions created inside this block keep the SIMT attention kernel."""

    def __enter__(self):
        self.old = os.environ.get("LITNICE_B200_TC_ATTN")
        os.environ["LITNICE_B200_TC_ATTN"] = "0"

    def __exit__(self, *exc):
        if self.old is None:
            del os.environ["LITNICE_B200_TC_ATTN"]
        else:
            os.environ["LITNICE_B200_TC_ATTN"] = self.old


@pytest.mark.parametrize("seq", [1, 64, 127, 128, 129, 255, 256, 257, 300, 513, 640])
def test_split_key_schedule_matches_oracle(oracle, arena, seq):
    """One and three streams of two heads: every query tile's keys are cut over CTAs."""
    ids = formats.zipf_prompt(DIMS.vocab, seq, 9000 + seq)
    want = oracle.forward(DIMS, arena, ids)
    with Session(DIMS, 3) as s:
        s.load_params(arena)
        one = s.forward(ids, all_rows=True)[0]
        three = s.forward(np.stack([ids, ids[::-1].copy(), ids]), all_rows=True)
    assert rel_err(one, want) < LOGIT_RTOL
    assert rel_err(three[0], want) < LOGIT_RTOL
    assert np.array_equal(three[0], three[2])
    assert rel_err(three[1], oracle.forward(DIMS, arena, ids[::-1].copy())) < LOGIT_RTOL


@pytest.mark.parametrize("streams,seq", [(40, 200), (19, 512), (80, 130)])
def test_multi_tile_schedule_matches_simt_kernel_and_oracle(oracle, arena, streams, seq):
    """Enough (stream, head) pairs that one CTA walks all key tiles of its query tile."""
    ids = np.stack([formats.zipf_prompt(DIMS.vocab, seq, 500 + b) for b in range(streams)])
    with Session(DIMS, streams) as s:
        s.load_params(arena)
        got = s.forward(ids, all_rows=True)
    with simt_attention():
        with Session(DIMS, streams) as s:
            s.load_params(arena)
            ref = s.forward(ids, all_rows=True)
    assert rel_err(got, ref) < KERNEL_RTOL
    for b in (0, streams // 2, streams - 1):
        assert rel_err(got[b], oracle.forward(DIMS, arena, ids[b])) < LOGIT_RTOL


def test_token_loop_across_tile_boundaries(oracle, arena):
    """Graph replay with the context growing through 128 and 192: tokens and step logits."""
    prompt = formats.zipf_prompt(DIMS.vocab, 120, 77)
    ref_t, ref_l = oracle.generate(DIMS, arena, prompt, 80, want_logits=True)
    with Session(DIMS, 2) as s:
        s.load_params(arena)
        s.keep_step_logits(True)
        toks = s.generate(np.stack([prompt, prompt]), 80)
        lg = s.read_step_logits(toks.shape[1], 2)
    assert np.array_equal(toks[0], toks[1])
    n = len(ref_t)
    for i in range(n):
        if toks[0][i] != ref_t[i]:
            top2 = np.sort(ref_l[i])[-2:]
            assert top2[1] - top2[0] < NEAR_TIE, f"step {i}"
            n = i
            break
    assert n >= 8
    assert rel_err(lg[:n, 0, :], ref_l[:n]) < LOGIT_RTOL


def test_token_loop_graph_replay_equals_direct_launches(arena):
    """The replayed graphs (launches sized for a 64-token bucket, the length read on
    the device) give the same tokens as launching every kernel for the exact length."""
    prompts = np.stack([formats.zipf_prompt(DIMS.vocab, 100, 31 + b) for b in range(3)])
    with Session(DIMS, 3) as s:
        s.load_params(arena)
        a = s.generate(prompts, 70)
    old = os.environ.get("LITNICE_B200_GRAPHS")
    os.environ["LITNICE_B200_GRAPHS"] = "0"
    try:
        with Session(DIMS, 3) as s:
            s.load_params(arena)
            b = s.generate(prompts, 70)
    finally:
        if old is None:
            del os.environ["LITNICE_B200_GRAPHS"]
        else:
            os.environ["LITNICE_B200_GRAPHS"] = old
    assert np.array_equal(a, b)


@pytest.mark.parametrize("seq", [200, 384])
def test_fixed_head_scales_with_skewed_weights(oracle, seq):
    """The fp16-pair attention keeps Q, K and V under scales derived from the weights alone
    (a bound over every possible LayerNorm output). Weights whose heads and thirds differ by
    orders of magnitude, a wide LayerNorm scale and large shifts and biases must neither
    overflow fp16 nor lose accuracy: logits against the oracle at the path's tolerance."""
    arena = formats.make_param_arena(DIMS, 4321, bias_std=0.05, ln_std=0.3)
    lay = formats.ParamLayout.build(DIMS)
    D = DIMS.d_model
    rng = np.random.default_rng(5)
    for l in range(DIMS.n_layers):
        w = lay.view(arena, f"layer{l}.attn_qkv_w")
        b = lay.view(arena, f"layer{l}.attn_qkv_b")
        # Q of head 0 large, K of head 1 tiny, V thirds 30x apart; one outlier column per third
        col_scale = np.ones(3 * D, dtype=np.float32)
        col_scale[0:64] = 40.0
        col_scale[D + 64:D + 128] = 1e-3
        col_scale[2 * D:2 * D + 64] = 30.0
        col_scale[[5, D + 70, 2 * D + 100]] *= 25.0
        w *= col_scale[None, :]
        b *= col_scale[None, :]
        lay.view(arena, f"layer{l}.ln1_beta")[...] += rng.normal(0.0, 2.0, size=(1, D)).astype(np.float32)
    ids = formats.zipf_prompt(DIMS.vocab, seq, 600 + seq)
    want = oracle.forward(DIMS, arena, ids)
    assert np.isfinite(want).all()
    with Session(DIMS, 2) as s:
        s.load_params(arena)
        got = s.forward(np.stack([ids, ids]), all_rows=True)
    assert np.isfinite(got).all()
    assert rel_err(got[0], want) < LOGIT_RTOL
    assert np.array_equal(got[0], got[1])


class tf32_pair_attention:
    """Sessions created inside this block keep Q, K and V^T as TF32 pairs (attention_tc.cu)."""

    def __enter__(self):
        self.old = os.environ.get("LITNICE_B200_ATTN16")
        os.environ["LITNICE_B200_ATTN16"] = "0"

    def __exit__(self, *exc):
        if self.old is None:
            del os.environ["LITNICE_B200_ATTN16"]
        else:
            os.environ["LITNICE_B200_ATTN16"] = self.old


@pytest.mark.parametrize("streams,seq", [(1, 300), (19, 512)])
def test_tf32_pair_kernel_matches_oracle_and_fp16_pair_kernel(oracle, arena, streams, seq):
    """The kernel behind LITNICE_B200_ATTN16=0 (split-key and multi-tile schedules) against the
    oracle, and the default fp16-pair kernel against it."""
    ids = np.stack([formats.zipf_prompt(DIMS.vocab, seq, 800 + b) for b in range(streams)])
    with tf32_pair_attention():
        with Session(DIMS, streams) as s:
            s.load_params(arena)
            old = s.forward(ids, all_rows=True)
    with Session(DIMS, streams) as s:
        s.load_params(arena)
        new = s.forward(ids, all_rows=True)
    for b in (0, streams - 1):
        assert rel_err(old[b], oracle.forward(DIMS, arena, ids[b])) < LOGIT_RTOL
    assert rel_err(new, old) < KERNEL_RTOL
