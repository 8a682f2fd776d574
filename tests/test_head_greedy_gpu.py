"""The one-launch tail of a greedy step (final norm, output head, first-max
selection, append, state advance) against the reference's fixtures, the oracle
and the five-launch tail it replaces, through the C ABI's token loop."""
import os

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import Session
from conftest import load_small
from test_native_loop_gpu import assert_greedy_identity

pytestmark = pytest.mark.gpu


class separate_tail:
    """Sessions created inside this block end a step with the separate kernels."""

    def __enter__(self):
        self.old = os.environ.get("LITNICE_B200_FUSED_TAIL")
        os.environ["LITNICE_B200_FUSED_TAIL"] = "0"

    def __exit__(self, *exc):
        if self.old is None:
            del os.environ["LITNICE_B200_FUSED_TAIL"]
        else:
            os.environ["LITNICE_B200_FUSED_TAIL"] = self.old


@pytest.mark.parametrize("name", ["c1", "abcdef"])
def test_fused_tail_matches_reference_fixture(name):
    d, z = load_small(name)
    with Session(d, 2) as s:
        s.load_params(z["arena"])
        toks = s.generate(z["prompt"], 128)[0]
    assert_greedy_identity(toks, z["greedy_tokens"], z["greedy_step_logits"])
    assert len(toks) == min(128, d.max_seq - len(z["prompt"]))


@pytest.mark.parametrize("streams", [1, 3, 8])
def test_fused_tail_equals_separate_kernels(streams):
    d = formats.ModelDims(2, 2, 128, 256, 96, 512)
    arena = formats.make_param_arena(d, 77, bias_std=0.02)
    prompts = np.stack([formats.zipf_prompt(d.vocab, 40, 600 + b) for b in range(streams)])
    with Session(d, streams) as s:
        s.load_params(arena)
        first = s.generate(prompts, 50)
        again = s.generate(prompts, 50)
    with separate_tail():
        with Session(d, streams) as s:
            s.load_params(arena)
            ref = s.generate(prompts, 50)
    assert first.shape == (streams, 50)
    assert np.array_equal(first, again)
    # both tails sum the head's products in fp32, in different orders: a token may
    # differ only where the two largest logits are within rounding of each other
    for b in range(streams):
        diff = np.flatnonzero(first[b] != ref[b])
        assert diff.size == 0 or diff[0] > 8, f"stream {b} diverges at step {diff[:1]}"
    assert (first == ref).mean() > 0.9


def test_fused_tail_config2_shape_matches_oracle(oracle):
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    prompt = formats.zipf_prompt(d.vocab, 32, 4001)
    ref_t, ref_l = oracle.generate(d, arena, prompt, 24, want_logits=True)
    with Session(d, 2) as s:
        s.load_params(arena)
        toks = s.generate(np.stack([prompt, prompt]), 24)
    assert np.array_equal(toks[0], toks[1])
    assert_greedy_identity(toks[0], ref_t, ref_l)


def test_fused_tail_resumes_without_graphs():
    """Direct launches (no graph replay): the state the last CTA advances is the one
    the next step's kernels read."""
    d, z = load_small("abcdef")
    old = os.environ.get("LITNICE_B200_GRAPHS")
    os.environ["LITNICE_B200_GRAPHS"] = "0"
    try:
        with Session(d, 1) as s:
            s.load_params(z["arena"])
            toks = s.generate(z["prompt"], 40)[0]
    finally:
        if old is None:
            del os.environ["LITNICE_B200_GRAPHS"]
        else:
            os.environ["LITNICE_B200_GRAPHS"] = old
    assert_greedy_identity(toks, z["greedy_tokens"][:40], z["greedy_step_logits"][:40])
