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

Fixtures of the benchmark workloads themselves (`python tests/golden/make_golden.py
workloads`, about an hour of CPU time). The reference's CPU backend takes about a
minute per token at these sizes, so the token sequences come from the C
restatement (oracle/liboracle.so, which test_oracle_pin.py pins bit-for-bit to
the reference) and the reference itself then confirms them where one forward is
affordable: ref_driver runs one forward over the finished sequence, its logits
must equal the restatement's bit for bit, and the first maximum of row
prompt_len-1+i must be token i, which is what the reference's own greedy loop
would have picked (inference.cpp:188-198,265-296).
  c2_full.npz       the default bench workload: prompt (seed 4000), all 768
                    greedy tokens, all-row logits at s=1023 (row 255+i is the
                    last-row logits of step i), top-2 gap of every step
  c5_dims.npz       config-4/5 model: last-row logits at s=64 and s=256 of
                    stream 0's prompt and 8 greedy tokens from s=256
  c3_streams.npz    config 3: streams 0, 1, 31, 63 of the 64, 64 sampled tokens
                    each with the bench's per-stream seeds
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


def _sha(arena: np.ndarray) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(arena.tobytes()).digest(), np.uint8)


def _top2_gap(rows: np.ndarray) -> np.ndarray:
    srt = np.sort(rows.astype(np.float64), axis=1)
    return (srt[:, -1] - srt[:, -2]).astype(np.float32)


def c2_full(confirm_with_reference: bool = True):
    """The default bench workload (config 2): arena seed 1002, prompt seed
    2000*2+0, 256-token prompt, 768 greedy tokens."""
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    prompt = formats.zipf_prompt(d.vocab, 256, 2000 * 2 + 0)
    toks, step_logits = ob.generate(d, arena, prompt, 768, want_logits=True)
    assert len(toks) == 768
    ids = np.concatenate([prompt, toks[:-1]])          # 1023 ids: the context of the last step
    logits_all = ob.forward(d, arena, ids)
    assert np.array_equal(logits_all[255:], step_logits), "causal rows must equal the step logits"
    assert np.array_equal(np.argmax(logits_all[255:], axis=1), toks)
    confirmed = 0
    if confirm_with_reference and ob.have_ref():
        ref_logits, _ = ob.ref_run(d, arena, ids, attention="fused_inplace", ffn="inplace_fused_bias_relu")
        assert np.array_equal(ref_logits, logits_all), "restatement differs from the reference at s=1023"
        confirmed = 1
    np.savez_compressed(os.path.join(HERE, "c2_full.npz"), prompt=prompt, greedy_tokens=toks,
                        logits_all=logits_all, top2_gap=_top2_gap(step_logits),
                        arena_sha256=_sha(arena), arena_seed=np.array([1002]),
                        confirmed_by_reference=np.array([confirmed]))
    print("c2_full", toks[:8], "min top-2 gap", float(_top2_gap(step_logits).min()), "confirmed", confirmed)


def c5_dims(confirm_with_reference: bool = True):
    """Config-4/5 model (arena seed 1005, the bench's c5 weights), stream 0's
    256-token prompt (seed 2000*5+0)."""
    d = formats.CONFIG_DIMS["c5"]
    arena = formats.make_param_arena(d, 1005)
    prompt = formats.zipf_prompt(d.vocab, 256, 2000 * 5 + 0)
    last64 = ob.forward(d, arena, prompt[:64], only_last=True)
    toks, step_logits = ob.generate(d, arena, prompt, 8, want_logits=True)
    confirmed = 0
    if confirm_with_reference and ob.have_ref():
        ref_logits, _ = ob.ref_run(d, arena, prompt[:64], attention="fused_inplace",
                                   ffn="inplace_fused_bias_relu")
        assert np.array_equal(ref_logits[-1], last64), "restatement differs from the reference at s=64"
        confirmed = 1
    np.savez_compressed(os.path.join(HERE, "c5_dims.npz"), prompt=prompt, last_logits_s64=last64,
                        greedy_tokens=toks, step_logits=step_logits, top2_gap=_top2_gap(step_logits),
                        arena_sha256=_sha(arena), arena_seed=np.array([1005]),
                        confirmed_by_reference=np.array([confirmed]))
    print("c5_dims", toks, "gaps", _top2_gap(step_logits), "confirmed", confirmed)


def c3_streams():
    """Config 3 (arena seed 1003): four of the bench's 64 streams, 128-token
    prompts (seed 2000*3+i), 64 tokens sampled with temp 0.8, top_k 40,
    top_p 0.95 and seed 3000+i."""
    d = formats.CONFIG_DIMS["c3"]
    arena = formats.make_param_arena(d, 1003)
    which = np.array([0, 1, 31, 63], dtype=np.int32)
    prompts = np.stack([formats.zipf_prompt(d.vocab, 128, 2000 * 3 + int(i)) for i in which])
    toks, logits = [], []
    for i, p in zip(which, prompts):
        t, lg = ob.generate(d, arena, p, 64, temp=0.8, top_k=40, top_p=0.95, seed=3000 + int(i),
                            want_logits=True)
        toks.append(t)
        logits.append(lg)
    np.savez_compressed(os.path.join(HERE, "c3_streams.npz"), streams=which, prompts=prompts,
                        sampled_tokens=np.stack(toks), step_logits=np.stack(logits),
                        sampled_params=np.array([0.8, 40, 0.95]), seeds=3000 + which,
                        arena_sha256=_sha(arena), arena_seed=np.array([1003]))
    print("c3_streams", np.stack(toks)[:, :8])


def c4_prefill(confirm_with_reference: bool = False):
    """Config 4 (arena seed 1004, the bench's prefill batch): sequences 0 and 31
    of rank 0 (prompt seeds 2000*4+i), all 2048 tokens: the last row's logits,
    i.e. the next-token distribution the prefill step returns."""
    d = formats.CONFIG_DIMS["c5"]
    arena = formats.make_param_arena(d, 1004)
    which = np.array([0, 31], dtype=np.int32)
    prompts = np.stack([formats.zipf_prompt(d.vocab, d.max_seq, 2000 * 4 + int(i)) for i in which])
    rows = np.stack([ob.forward(d, arena, p, only_last=True) for p in prompts])
    confirmed = 0
    if confirm_with_reference and ob.have_ref():      # about an hour of the reference's single thread
        ref_logits, _ = ob.ref_run(d, arena, prompts[0], attention="fused_inplace", ffn="inplace_fused_bias_relu")
        assert np.array_equal(ref_logits[-1], rows[0]), "restatement differs from the reference at s=2048"
        confirmed = 1
    np.savez_compressed(os.path.join(HERE, "c4_prefill.npz"), sequences=which, prompts=prompts,
                        last_logits=rows, top2_gap=_top2_gap(rows), arena_sha256=_sha(arena),
                        arena_seed=np.array([1004]), confirmed_by_reference=np.array([confirmed]))
    print("c4_prefill", rows.argmax(axis=1), "gaps", _top2_gap(rows), "confirmed", confirmed)


if __name__ == "__main__":
    what = sys.argv[1:] or ["small"]
    for w in what:
        if w == "small":
            main()
        elif w == "workloads":
            c3_streams()
            c5_dims()
            c2_full()
            c4_prefill()
        else:
            {"c2_full": c2_full, "c5_dims": c5_dims, "c3_streams": c3_streams, "c4_prefill": c4_prefill}[w]()
