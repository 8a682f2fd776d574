"""The reference's own `litnicelm train` on the B200 plugin.

The unmodified reference binary (oracle/_ref/litnicelm) runs the flow of its
scripts/try_cpu.sh (tokenizer_training, encode, train for one epoch, infer) twice
on the same corpus and configuration: once with its CPU plugin, once with
`backend.library` pointing at this plugin. Every training entry of the table
(backward products, LayerNorm / softmax / ReLU backward, cross entropy,
embedding gradients, gradient-norm, AdamW) is on that path. The two runs start
from the same deterministic initialisation and see the same batches, so their
final losses and parameters must agree to the rounding that 383 optimiser
steps accumulate.
"""
import os
import re
import subprocess

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import LIB_PATH

pytestmark = pytest.mark.gpu

ATTENTION_FFN = [("reference", "reference"), ("fused_inplace", "inplace_fused_bias_relu"),
                 ("fused_inplace_multistream", "fused_bias_relu")]


def run_flow(ref, root, lib, attention, ffn):
    os.makedirs(root, exist_ok=True)
    corpus = os.path.join(root, "abc.txt")
    with open(corpus, "w") as f:
        f.write("a b c a b c a b c a b c\n" * 128)
    d = formats.ModelDims(2, 2, 32, 64, 128, 8)
    ckpt = os.path.join(root, "best.ckpt")
    yaml = os.path.join(root, "cfg.yaml")
    formats.write_yaml(yaml, d, backend_library=lib, checkpoint=ckpt, corpus=corpus,
                       dataset_bin=os.path.join(root, "art", "tokenized_dataset.bin"),
                       tokenizer_type="only_seen_chars", artifacts_dir=os.path.join(root, "art"),
                       attention=attention, ffn=ffn, max_new=16, temp=0.0, prompt="a b c ")
    outs = {}
    for step in (["tokenizer_training"], ["encode"], ["train", "--incremental=false", "--epochs", "1"],
                 ["infer", "--prompt", "a b ", "--max_new", "3", "--temp", "0"]):
        p = subprocess.run([ref.REF_CLI, step[0], "--config", yaml] + step[1:], capture_output=True, text=True,
                           timeout=900)
        assert p.returncode == 0, f"{step[0]} on {lib}: {p.stderr[-1500:]}{p.stdout[-1500:]}"
        outs[step[0]] = p.stdout
    journal = open(ckpt + ".journal").read()
    loss = float(re.search(r"Best loss: ([0-9.eE+-]+)", journal).group(1))
    steps = int(re.search(r"Global step: (\d+)", journal).group(1))
    dims, arena = formats.read_checkpoint(ckpt)
    tokens = re.findall(r"Generated token id=(\d+)", outs["infer"])
    return loss, steps, dims, arena.view(np.float32), tokens, outs["train"]


@pytest.mark.parametrize("attention,ffn", ATTENTION_FFN)
def test_one_training_epoch_on_the_plugin_matches_the_cpu_backend(oracle, tmp_path, attention, ffn):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not present")
    cpu = run_flow(oracle, str(tmp_path / "cpu"), oracle.REF_CPU_PLUGIN, "reference", "reference")
    gpu = run_flow(oracle, str(tmp_path / "b200"), LIB_PATH, attention, ffn)
    assert "Loaded backend library: " + LIB_PATH in gpu[5]
    assert cpu[1] == gpu[1] == 383
    assert cpu[2] == gpu[2]
    print(f"{attention}/{ffn}: final loss CPU {cpu[0]:.6f}, B200 {gpu[0]:.6f}; "
          f"largest parameter difference {float(np.abs(cpu[3] - gpu[3]).max()):.2e}")
    assert abs(cpu[0] - gpu[0]) <= 2e-3 * max(abs(cpu[0]), 1e-3)
    assert float(np.abs(cpu[3] - gpu[3]).max()) <= 5e-3
    assert np.all(np.isfinite(gpu[3]))
    assert cpu[4] == gpu[4]
