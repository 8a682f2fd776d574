"""Drop-in check: the reference's own host code runs on the B200 plugin.

oracle/_ref holds the unmodified reference compiled from its sources: its
`litnicelm` binary and a driver that feeds explicit token ids to the
reference's Transformer::forward. Both load the plugin named by
`backend.library` exactly as the reference always does, so these tests prove
that the exported table is accepted by the reference loader and that every
operator the model code calls behaves like the CPU backend.
"""
import os
import re
import subprocess

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import LIB_PATH
from conftest import load_small

pytestmark = pytest.mark.gpu

ATTENTION = ["reference", "fused_inplace", "fused_inplace_multistream"]
FFN = ["reference", "fused_bias_relu", "inplace_fused_bias_relu"]


@pytest.fixture(scope="module")
def ref(oracle):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not present")
    return oracle


@pytest.mark.parametrize("attention", ATTENTION)
@pytest.mark.parametrize("ffn", FFN)
def test_reference_model_code_on_plugin_all_algo_variants(ref, attention, ffn):
    d, z = load_small("c1")
    got, _ = ref.ref_run(d, z["arena"], z["prompt"], backend_library=LIB_PATH, attention=attention, ffn=ffn)
    want = z["logits"]
    scale = np.abs(want).max(axis=-1, keepdims=True)
    assert float((np.abs(got - want) / scale).max()) < 1e-3


@pytest.mark.parametrize("name", ["c1", "abcdef"])
def test_reference_generation_on_plugin(ref, name):
    d, z = load_small(name)
    toks, logits, _, _ = ref.ref_run(d, z["arena"], z["prompt"], mode="generate", max_new=128,
                                     backend_library=LIB_PATH, attention="fused_inplace",
                                     ffn="inplace_fused_bias_relu", want_logits=True)
    want = z["greedy_tokens"]
    assert len(toks) == len(want)
    for i, (a, b) in enumerate(zip(toks, want)):
        if a != b:
            top2 = np.sort(z["greedy_step_logits"][i])[-2:]
            assert top2[1] - top2[0] < 1e-4, f"token {i} differs without a near-tie"
            break


def test_unmodified_litnicelm_cli_infer_on_plugin(ref, tmp_path):
    """`litnicelm infer` itself, text prompt, character tokenizer, plugin vs CPU plugin."""
    d = formats.ModelDims(2, 2, 64, 256, 128, 48)
    arena = formats.make_param_arena(d, 4242, bias_std=0.02)
    ckpt = str(tmp_path / "m.ckpt")
    formats.write_checkpoint(ckpt, d, arena)
    binf = str(tmp_path / "tok.bin")
    formats.write_dataset_header(binf, d.vocab)
    outs = {}
    for tag, lib in (("cpu", ref.REF_CPU_PLUGIN), ("b200", LIB_PATH)):
        yaml = str(tmp_path / f"{tag}.yaml")
        formats.write_yaml(yaml, d, backend_library=lib, checkpoint=ckpt, dataset_bin=binf,
                           tokenizer_type="character", attention="fused_inplace",
                           ffn="inplace_fused_bias_relu", max_new=24, temp=0.0)
        p = subprocess.run([ref.REF_CLI, "infer", "--config", yaml, "--prompt", "a b c ", "--temp", "0"],
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:] + p.stdout[-2000:]
        outs[tag] = re.findall(r"Generated token id=(\d+)", p.stdout)
        assert len(outs[tag]) == 24
    assert "Loaded backend library" in p.stdout
    assert outs["cpu"] == outs["b200"]


@pytest.mark.parametrize("attention", ATTENTION)
@pytest.mark.parametrize("ffn", FFN)
def test_deferred_operator_queue_changes_nothing(ref, attention, ffn):
    """The plugin records the host's per-head attention calls and projection + bias pairs and issues
    them merged (three launches for all heads, one per projection). With the queue off every call is
    issued at once. Both must leave bit-identical logits: merging changes launch counts, not values."""
    d = formats.ModelDims(2, 4, 64, 128, 40, 48)
    arena = formats.make_param_arena(d, 77, bias_std=0.02, ln_std=0.1)
    ids = formats.zipf_prompt(d.vocab, 37, 5)
    merged, _ = ref.ref_run(d, arena, ids, backend_library=LIB_PATH, attention=attention, ffn=ffn)
    plain, _ = ref.ref_run(d, arena, ids, backend_library=LIB_PATH, attention=attention, ffn=ffn,
                           threads_env={"LITNICE_B200_ABI_QUEUE": "0"})
    assert np.array_equal(merged, plain)
    want, _ = ref.ref_run(d, arena, ids)        # the reference CPU plugin
    scale = np.abs(want).max(axis=-1, keepdims=True)
    assert float((np.abs(merged - want) / scale).max()) < 1e-3


def test_reference_token_loop_on_plugin_config2_shape(ref):
    """The reference's own loop (whole-context forward, one copy_device2host per
    logits row, host-side argmax) at the config-2 shape on the plugin: same
    tokens with and without the plugin's read-ahead for row-by-row read-back,
    and the per-token times of both, for the record."""
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    prompt = formats.zipf_prompt(d.vocab, 200, 4002)
    runs = {}
    for tag, env in (("read-ahead", {}), ("row copies", {"LITNICE_B200_READ_AHEAD": "0"}),
                     ("read-ahead, every call issued at once", {"LITNICE_B200_ABI_QUEUE": "0"})):
        toks, _, secs, _ = ref.ref_run(d, arena, prompt, mode="generate", max_new=24, backend_library=LIB_PATH,
                                       attention="fused_inplace", ffn="inplace_fused_bias_relu", threads_env=env)
        runs[tag] = (toks, float(np.median(secs[2:])))
    assert np.array_equal(runs["read-ahead"][0], runs["row copies"][0])
    assert np.array_equal(runs["read-ahead"][0], runs["read-ahead, every call issued at once"][0])
    assert len(runs["read-ahead"][0]) == 24
    for tag, (_, t) in runs.items():
        print(f"reference host loop on the plugin, context ~212, {tag}: {1e3 * t:.2f} ms per token")
