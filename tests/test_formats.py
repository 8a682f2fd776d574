"""Host-side data formats: checkpoint, dataset header, YAML, prompts."""
import os
import subprocess

import numpy as np
import pytest

from litnicelm_b200 import formats


def test_checkpoint_round_trip(tmp_path):
    d = formats.CONFIG_DIMS["c1"]
    arena = formats.make_param_arena(d, 3, bias_std=0.01)
    path = str(tmp_path / "a.ckpt")
    formats.write_checkpoint(path, d, arena)
    lay = formats.ParamLayout.build(d)
    # 136-byte header + parameter arena + optimiser arena of twice the size
    assert os.path.getsize(path) == 136 + 3 * lay.total_bytes
    d2, arena2 = formats.read_checkpoint(path)
    assert d2 == d and np.array_equal(arena, arena2)


def test_layout_zones_and_alignment():
    d = formats.CONFIG_DIMS["c1"]
    lay = formats.ParamLayout.build(d)
    for name, (off, shape) in lay.slices.items():
        assert off % d.alignment == 0
        decay = shape[0] != 1
        assert (off < lay.decay_bytes) == decay, name
    assert list(lay.slices)[0] == "tok_embedding"
    arena = formats.make_param_arena(d, 1)
    assert np.all(lay.view(arena, "layer0.ln1_gamma") == 1.0)
    assert np.all(lay.view(arena, "layer1.ffn_b1") == 0.0)
    assert abs(float(lay.view(arena, "layer0.attn_qkv_w").std()) - 0.02) < 2e-3


def test_zipf_prompt_is_seeded_and_in_range():
    a = formats.zipf_prompt(96, 256, 7)
    b = formats.zipf_prompt(96, 256, 7)
    assert np.array_equal(a, b) and a.dtype == np.int32
    assert a.min() >= 0 and a.max() < 96
    counts = np.bincount(a, minlength=96)
    assert counts[0] > counts[10:].max()  # rank 1 dominates


def test_reference_accepts_generated_files(tmp_path, have_ref):
    """The unmodified reference loads the YAML, dataset header and checkpoint
    this package writes (only where the reference is compiled)."""
    if not have_ref:
        pytest.skip("oracle/_ref not built here")
    from oracle import binding as ob
    d = formats.ModelDims(1, 2, 32, 64, 128, 16)
    arena = formats.make_param_arena(d, 5)
    ckpt = str(tmp_path / "m.ckpt")
    formats.write_checkpoint(ckpt, d, arena)
    binf = str(tmp_path / "t.bin")
    formats.write_dataset_header(binf, d.vocab)
    yaml = str(tmp_path / "c.yaml")
    formats.write_yaml(yaml, d, backend_library=ob.REF_CPU_PLUGIN, checkpoint=ckpt, dataset_bin=binf,
                       max_new=4)
    p = subprocess.run([ob.REF_CLI, "infer", "--config", yaml, "--prompt", "ab", "--temp", "0"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-1500:]
    assert p.stdout.count("Generated token id=") == 4
