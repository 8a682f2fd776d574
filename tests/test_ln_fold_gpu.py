"""LayerNorm folded into the QKV and W1 projections (row statistics from the
producing kernels, correction in the epilogue) against the oracle and against
the stand-alone LayerNorm kernels, with non-trivial gamma / beta and with rows
whose mean dwarfs their spread (the case in which the folded form cancels)."""
import os

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import Session

pytestmark = pytest.mark.gpu

LOGIT_RTOL = 1e-3


def rel_err(got, want):
    scale = np.maximum(np.abs(want).max(axis=-1, keepdims=True), 1e-6)
    return float((np.abs(got - want) / scale).max())


class env:
    def __init__(self, name, value):
        self.name, self.value = name, value

    def __enter__(self):
        self.old = os.environ.get(self.name)
        os.environ[self.name] = self.value

    def __exit__(self, *exc):
        if self.old is None:
            del os.environ[self.name]
        else:
            os.environ[self.name] = self.old


CASES = [
    # L, H, D, F, V, S; head dimension 64 (tensor-core attention) and 32 (SIMT attention)
    formats.ModelDims(2, 2, 128, 256, 96, 512),
    formats.ModelDims(2, 4, 128, 384, 50, 300),
    formats.ModelDims(1, 8, 512, 2048, 96, 700),
]


@pytest.mark.parametrize("dims", CASES, ids=lambda d: f"D{d.d_model}H{d.n_heads}")
@pytest.mark.parametrize("seq", [5, 130, 257])
def test_folded_layernorm_matches_oracle_and_plain_kernels(oracle, dims, seq):
    arena = formats.make_param_arena(dims, 77, bias_std=0.05, ln_std=0.3)
    ids = np.stack([formats.zipf_prompt(dims.vocab, seq, 600 + b) for b in range(2)])
    want = [oracle.forward(dims, arena, ids[b]) for b in range(2)]
    with Session(dims, 2) as s:
        s.load_params(arena)
        folded = s.forward(ids, all_rows=True)
    with env("LITNICE_B200_LN_FOLD", "0"):
        with Session(dims, 2) as s:
            s.load_params(arena)
            plain = s.forward(ids, all_rows=True)
    for b in range(2):
        assert rel_err(folded[b], want[b]) < LOGIT_RTOL
        assert rel_err(plain[b], want[b]) < LOGIT_RTOL
    print(f"folded vs oracle {rel_err(folded[0], want[0]):.2e}, plain vs oracle {rel_err(plain[0], want[0]):.2e}")


def test_rows_with_large_mean(oracle):
    """Embeddings shifted by 25 standard deviations: x W' and mean * u nearly cancel."""
    dims = formats.ModelDims(2, 2, 128, 256, 96, 256)
    arena = formats.make_param_arena(dims, 78, bias_std=0.05, ln_std=0.2)
    lay = formats.ParamLayout.build(dims)
    lay.view(arena, "tok_embedding")[...] += 0.5
    ids = formats.zipf_prompt(dims.vocab, 200, 9)
    want = oracle.forward(dims, arena, ids)
    with Session(dims, 1) as s:
        s.load_params(arena)
        got = s.forward(ids, all_rows=True)[0]
    assert rel_err(got, want) < LOGIT_RTOL
    print(f"large-mean rows: {rel_err(got, want):.2e}")
