"""Parity of the native GPU token loop with the oracle, through the C ABI.

Tolerances are the ones the task states for this floating-point path: logits
within 1e-3 relative (measured against the largest |logit| of the row), greedy
token sequences identical except at logged near-ties (top-2 gap < 1e-4 in the
oracle's logits), argmax/top-k indices identical on identical logits.
"""
import hashlib
import os

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import Session
from conftest import GOLDEN, load_small

pytestmark = pytest.mark.gpu

LOGIT_RTOL = 1e-3
NEAR_TIE = 1e-4


def rel_err(got, want):
    scale = np.maximum(np.abs(want).max(axis=-1, keepdims=True), 1e-6)
    return float((np.abs(got - want) / scale).max())


def assert_greedy_identity(tokens, ref_tokens, ref_step_logits):
    """Identical sequences, except that a first mismatch is accepted when the
    oracle's own top-2 gap at that step is a near-tie (the streams then diverge
    legitimately, so the comparison stops there)."""
    n = min(len(tokens), len(ref_tokens))
    assert len(tokens) == len(ref_tokens)
    for i in range(n):
        if tokens[i] != ref_tokens[i]:
            top2 = np.sort(ref_step_logits[i])[-2:]
            gap = float(top2[1] - top2[0])
            assert gap < NEAR_TIE, f"step {i}: token {tokens[i]} != {ref_tokens[i]} with top-2 gap {gap}"
            print(f"near-tie at step {i}: gap {gap:.3e}; comparison stops here")
            return i
    return n


@pytest.fixture(scope="module", params=["c1", "abcdef"])
def small(request):
    d, z = load_small(request.param)
    s = Session(d, max_streams=4)
    s.load_params(z["arena"])
    yield request.param, d, z, s
    s.close()


def test_forward_all_rows_matches_reference_fixture(small):
    name, d, z, s = small
    got = s.forward(z["prompt"], all_rows=True)[0]
    assert rel_err(got, z["logits"]) < LOGIT_RTOL
    last = s.forward(z["prompt"], all_rows=False)[0]
    assert rel_err(last[None], z["logits"][-1:]) < LOGIT_RTOL


def test_greedy_tokens_match_reference_fixture(small):
    name, d, z, s = small
    s.keep_step_logits(True)
    toks = s.generate(z["prompt"], 128)[0]
    n = assert_greedy_identity(toks, z["greedy_tokens"], z["greedy_step_logits"])
    lg = s.read_step_logits(len(toks), 1)[:, 0, :]
    s.keep_step_logits(False)
    assert rel_err(lg[:n], z["greedy_step_logits"][:n]) < LOGIT_RTOL
    # loop guard of inference.cpp:278
    assert len(toks) == min(128, d.max_seq - len(z["prompt"]))


def test_sampled_tokens_match_reference_fixture(small):
    """The fused sampler follows libstdc++'s draw rule, so with the generator
    seed of the fixture the sampled stream is reproduced token for token as long
    as the logits agree closely enough not to move a top-p cut."""
    name, d, z, s = small
    temp, top_k, top_p, seed = z["sampled_params"]
    toks = s.generate(z["prompt"], 128, temp=float(temp), top_k=int(top_k), top_p=float(top_p),
                      seeds=[int(seed)])[0]
    ref = z["sampled_tokens"]
    assert len(toks) == len(ref)
    agree = int(np.argmin(np.append(toks == ref, False)))
    assert agree >= min(len(ref), 8), f"sampled stream diverged after {agree} tokens"
    print(f"{name}: sampled stream identical for {agree}/{len(ref)} tokens")


def test_streams_are_independent(small):
    """A stream's tokens do not depend on which other streams share its batch."""
    name, d, z, s = small
    rng = np.random.default_rng(5)
    plen = len(z["prompt"])
    prompts = np.stack([z["prompt"]] + [rng.integers(0, d.vocab, plen).astype(np.int32) for _ in range(3)])
    batch = s.generate(prompts, 16)
    for b in range(4):
        alone = s.generate(prompts[b], 16)[0]
        assert np.array_equal(batch[b], alone)


def test_causal_invariance(small):
    """Logits of row i do not change when later tokens change."""
    name, d, z, s = small
    ids = np.array(z["prompt"]).copy()
    a = s.forward(ids, all_rows=True)[0]
    ids2 = ids.copy()
    ids2[-1] = (ids2[-1] + 1) % d.vocab
    b = s.forward(ids2, all_rows=True)[0]
    assert np.array_equal(a[:-1], b[:-1])
    assert not np.array_equal(a[-1], b[-1])


def test_inspect_probabilities(small):
    name, d, z, s = small
    p = s.inspect(z["prompt"])[0]
    row = z["logits"][-1].astype(np.float64)
    want = np.exp(row - row.max())
    want /= want.sum()
    np.testing.assert_allclose(p, want, rtol=2e-3, atol=1e-7)
    assert abs(float(p.sum()) - 1.0) < 1e-5
    assert int(np.argmax(p)) == int(np.argmax(z["logits"][-1]))


def test_bad_token_id_is_reported_not_fatal(small):
    name, d, z, s = small
    bad = np.array(z["prompt"]).copy()
    bad[0] = d.vocab + 3
    with pytest.raises(RuntimeError, match="out of range"):
        s.forward(bad)
    ok = s.forward(z["prompt"])[0]  # the session stays usable
    assert rel_err(ok[None], z["logits"][-1:]) < LOGIT_RTOL


def test_config2_shape_against_reference_fixture():
    z = np.load(os.path.join(GOLDEN, "c2_prefix.npz"))
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, int(z["arena_seed"][0]))
    if hashlib.sha256(arena.tobytes()).digest() != z["arena_sha256"].tobytes():
        pytest.skip("numpy's generator stream changed; the seeded arena no longer matches the fixture")
    with Session(d, 1) as s:
        s.load_params(arena)
        got = s.forward(z["prompt"], all_rows=True)[0]
    assert rel_err(got, z["logits"]) < LOGIT_RTOL


@pytest.mark.parametrize("seq", [1, 63, 64, 65, 200])
def test_config2_shape_against_oracle(oracle, seq):
    """Ragged context lengths around the 64-row attention tile."""
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002, bias_std=0.02)
    ids = formats.zipf_prompt(d.vocab, seq, 4000 + seq)
    want = oracle.forward(d, arena, ids)
    with Session(d, 2) as s:
        s.load_params(arena)
        got = s.forward(np.stack([ids, ids[::-1].copy()]), all_rows=True)
        want2 = oracle.forward(d, arena, ids[::-1].copy())
    assert rel_err(got[0], want) < LOGIT_RTOL
    assert rel_err(got[1], want2) < LOGIT_RTOL
    assert int(np.argmax(got[0][-1])) == int(np.argmax(want[-1])) or \
        np.sort(want[-1])[-1] - np.sort(want[-1])[-2] < NEAR_TIE


def test_config2_greedy_decode_matches_oracle(oracle):
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    prompt = formats.zipf_prompt(d.vocab, 32, 4001)
    ref_t, ref_l = oracle.generate(d, arena, prompt, 24, want_logits=True)
    with Session(d, 1) as s:
        s.load_params(arena)
        s.keep_step_logits(True)
        toks = s.generate(prompt, 24)[0]
        lg = s.read_step_logits(len(toks), 1)[:, 0, :]
    n = assert_greedy_identity(toks, ref_t, ref_l)
    assert rel_err(lg[:n], ref_l[:n]) < LOGIT_RTOL


def test_large_vocab_head_and_sampler(oracle):
    """vocab 32000 (the config-4/5 head): output head as a few-row product,
    greedy argmax and top-k sampling on identical logits."""
    d = formats.ModelDims(1, 2, 64, 128, 32000, 32)
    arena = formats.make_param_arena(d, 31)
    ids = formats.zipf_prompt(d.vocab, 9, 77)
    want = oracle.forward(d, arena, ids, only_last=True)
    with Session(d, 3) as s:
        s.load_params(arena)
        got = s.forward(np.stack([ids, ids, ids]))
        assert rel_err(got, np.stack([want] * 3)) < LOGIT_RTOL
        toks = s.generate(ids, 4)[0]
        ref_t, ref_l = oracle.generate(d, arena, ids, 4, want_logits=True)
        assert_greedy_identity(toks, ref_t, ref_l)
        # sampler alone, on the oracle's logits: indices must be identical
        rows = np.stack([want, want * 0.5, want[::-1].copy()])
        for (temp, k, p) in [(0.8, 40, 0.95), (1.0, 0, 0.9), (1.3, 5000, 1.0), (0.7, 3, 1.0)]:
            dev = s.sample_logits(rows, temp, k, p, seeds=[11, 12, 13], draws=6)
            for r in range(3):
                smp = oracle.Sampler(11 + r)
                ref = [smp.pick(rows[r], temp, k, p)[0] for _ in range(6)]
                assert list(dev[r]) == ref, (temp, k, p, r)


def test_sampler_matches_host_selector_small_vocab(oracle):
    d = formats.CONFIG_DIMS["c3"]
    rng = np.random.default_rng(3)
    rows = (rng.standard_normal((8, d.vocab)) * 2).astype(np.float32)
    with Session(formats.ModelDims(1, 2, 64, 128, d.vocab, 16), 8) as s:
        for (temp, k, p) in [(0.8, 40, 0.95), (1.0, 0, 1.0), (0.5, 0, 0.5), (0.0, 0, 1.0), (1.0, 1, 1.0)]:
            seeds = list(range(3000, 3008))
            dev = s.sample_logits(rows, temp, k, p, seeds=seeds, draws=16)
            for r in range(8):
                smp = oracle.Sampler(seeds[r])
                ref = [smp.pick(rows[r], temp, k, p)[0] for _ in range(16)]
                assert list(dev[r]) == ref, (temp, k, p, r)
