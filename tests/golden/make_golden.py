"""Generates the golden fixtures of tests/golden/ from the reference itself.

Run in a container that holds the litnicelm reference sources:

    make -C oracle            # builds oracle/_ref/ from /root/reference
    python tests/golden/make_golden.py

Every expected value below is produced by oracle/_ref/ref_driver, i.e. by the
reference's own Transformer::forward, CPU backend and (restated, file-local)
token selectors; nothing comes from the C restatement or from the GPU code.
The reference ships no golden vectors of its own, so these files are the pin.

Fixtures
  small_<cfg>.npz   parameter arena, prompt ids, all-row logits, greedy tokens
                    with per-step last-row logits, sampled tokens
  c2_prefix.npz     config-2 shape: sha256 of the seeded arena (78 MB, not
                    stored), prompt ids, all-row logits at s=24
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from litnicelm_b200 import formats  # noqa: E402
from oracle import binding as ob  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def small(name: str, seed: int, prompt: np.ndarray, bias_std: float):
    d = formats.CONFIG_DIMS[name]
    arena = formats.make_param_arena(d, seed, bias_std=bias_std)
    logits, _ = ob.ref_run(d, arena, prompt)
    g_tok, g_log, _, _ = ob.ref_run(d, arena, prompt, mode="generate", max_new=128, want_logits=True)
    s_tok, _, _, _ = ob.ref_run(d, arena, prompt, mode="generate", max_new=128, temp=0.8, top_k=5,
                                top_p=0.95, seed=3001)
    f_log, _ = ob.ref_run(d, arena, prompt, attention="fused_inplace", ffn="inplace_fused_bias_relu")
    assert np.array_equal(f_log, logits), "reference attention/ffn variants disagree"
    np.savez_compressed(os.path.join(HERE, f"small_{name}.npz"), arena=arena, prompt=prompt,
                        logits=logits, greedy_tokens=g_tok, greedy_step_logits=g_log,
                        sampled_tokens=s_tok, sampled_params=np.array([0.8, 5, 0.95, 3001]),
                        dims=np.array([d.n_layers, d.n_heads, d.d_model, d.d_ff, d.vocab, d.max_seq,
                                       d.alignment]))
    print(name, "greedy", len(g_tok), "sampled", len(s_tok))


def main():
    if not ob.have_ref():
        raise SystemExit("oracle/_ref is missing: run `make -C oracle` where the reference sources are")
    # prompt "a b c " under the vocabulary order [a, ' ', b, c, d, e, f, '\n']
    abc = np.array([0, 1, 2, 1, 3, 1], dtype=np.int32)
    small("c1", 1001, abc, bias_std=0.02)
    small("abcdef", 1000, abc, bias_std=0.02)

    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    ids = formats.zipf_prompt(d.vocab, 24, 2000 * 2 + 0)
    logits, _ = ob.ref_run(d, arena, ids)
    np.savez_compressed(os.path.join(HERE, "c2_prefix.npz"), prompt=ids, logits=logits,
                        arena_sha256=np.frombuffer(hashlib.sha256(arena.tobytes()).digest(), np.uint8),
                        arena_seed=np.array([1002]))
    print("c2_prefix", logits.shape)


if __name__ == "__main__":
    main()
