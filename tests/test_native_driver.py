"""litnice_b200_run, the host driver of the native loop.

CPU part: its split of the streams over the GPUs is the one the Python side
uses. GPU part: `infer` prints the same [INFERENCE] token lines as the
reference's own `litnicelm infer` (generate_text, inference.cpp:277-294) on
the same checkpoint and prompt, `inspect` names the same argmax, and a run
over two GPUs returns the tokens of the one-GPU run.
"""
import os
import re
import subprocess

import numpy as np
import pytest

from litnicelm_b200 import formats
from litnicelm_b200.plugin import LIB_PATH
from litnicelm_b200.streams import partition_streams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "litnicelm_b200", "litnice_b200_run")


@pytest.fixture(scope="module")
def driver():
    if not os.path.exists(DRIVER):
        import __graft_entry__
        __graft_entry__.build()
    return DRIVER


@pytest.mark.parametrize("total,gpus", [(512, 8), (512, 3), (7, 2), (3, 8), (0, 4), (64, 1)])
def test_driver_partition_matches_the_python_split(driver, total, gpus):
    p = subprocess.run([driver, "partition", "--streams", str(total), "--gpus", str(gpus)],
                       capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stderr
    got = [tuple(int(v) for v in re.findall(r"-?\d+", ln)) for ln in p.stdout.splitlines()]
    want = [(g,) + partition_streams(total, gpus, g) for g in range(gpus)]
    assert got == want


def test_driver_rejects_bad_usage(driver, tmp_path):
    assert subprocess.run([driver], capture_output=True).returncode == 1
    p = subprocess.run([driver, "infer", "--config", str(tmp_path / "absent.yaml")], capture_output=True, text=True)
    assert p.returncode == 1 and "cannot open config" in p.stderr
    p = subprocess.run([driver, "partition", "--streams", "4", "--gpus", "0"], capture_output=True, text=True)
    assert p.returncode == 1


def _write_model(tmp_path, d, seed, lib):
    arena = formats.make_param_arena(d, seed, bias_std=0.02)
    ckpt = str(tmp_path / "m.ckpt")
    formats.write_checkpoint(ckpt, d, arena)
    binf = str(tmp_path / "tok.bin")
    formats.write_dataset_header(binf, d.vocab)
    yaml = str(tmp_path / f"{os.path.basename(lib)}.yaml")
    formats.write_yaml(yaml, d, backend_library=lib, checkpoint=ckpt, dataset_bin=binf,
                       tokenizer_type="character", attention="fused_inplace",
                       ffn="inplace_fused_bias_relu", max_new=24, temp=0.0, prompt="a b c ")
    return arena, yaml


@pytest.mark.gpu
def test_infer_prints_the_reference_token_lines(driver, oracle, tmp_path):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref (the compiled reference) is not present")
    d = formats.ModelDims(2, 2, 64, 256, 128, 48)
    _, yaml_ref = _write_model(tmp_path, d, 4242, oracle.REF_CPU_PLUGIN)
    _, yaml_b200 = _write_model(tmp_path, d, 4242, LIB_PATH)
    ref = subprocess.run([oracle.REF_CLI, "infer", "--config", yaml_ref, "--prompt", "a b c ", "--temp", "0"],
                         capture_output=True, text=True, timeout=600)
    got = subprocess.run([driver, "infer", "--config", yaml_b200, "--prompt", "a b c ", "--temp", "0"],
                         capture_output=True, text=True, timeout=600)
    assert ref.returncode == 0 and got.returncode == 0, got.stderr[-2000:]
    pick = lambda text: [ln for ln in text.splitlines() if "[INFERENCE][TOKEN_GEN] step=" in ln and "Generated token" in ln]
    assert len(pick(ref.stdout)) == 24
    assert pick(got.stdout) == pick(ref.stdout)
    # the closing line carries the whole text: prompt + generated characters
    last = lambda text: [ln for ln in text.splitlines() if ln.startswith("[INFERENCE][TOKEN_GEN] step=0")][-1]
    assert last(got.stdout) == last(ref.stdout)
    assert "[INFERENCE][START]" in got.stdout and "[INFERENCE][END]" in got.stdout


@pytest.mark.gpu
def test_inspect_names_the_reference_argmax(driver, oracle, tmp_path):
    d = formats.ModelDims(2, 2, 64, 256, 128, 48)
    arena, yaml = _write_model(tmp_path, d, 4243, LIB_PATH)
    got = subprocess.run([driver, "inspect", "--config", yaml, "--prompt", "hello"], capture_output=True, text=True,
                         timeout=600)
    assert got.returncode == 0, got.stderr[-2000:]
    ids = np.frombuffer(b"hello", np.uint8).astype(np.int32)
    row = oracle.forward(d, arena, ids, only_last=True).astype(np.float64)
    p = np.exp(row - row.max())
    p /= p.sum()
    m = re.search(r"Argmax: id=(\d+)", got.stdout)
    assert m and int(m.group(1)) == int(np.argmax(p))
    ent = float(re.search(r"Entropy: ([0-9.]+)", got.stdout).group(1))
    assert abs(ent - float(-(p[p > 0] * np.log(p[p > 0])).sum())) < 1e-3
    top = re.findall(r"^\d\. id=(\d+) .* prob=([0-9.]+)", got.stdout, flags=re.M)
    assert [int(t[0]) for t in top] == [int(i) for i in np.argsort(-p, kind="stable")[:5]]


@pytest.mark.gpu
def test_two_gpu_run_returns_the_one_gpu_tokens(driver, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    d = formats.ModelDims(2, 2, 64, 256, 128, 48)
    _, yaml = _write_model(tmp_path, d, 4244, LIB_PATH)
    ids = np.stack([formats.zipf_prompt(d.vocab, 12, 100 + i) for i in range(5)])
    idf = str(tmp_path / "ids.i32")
    ids.astype(np.int32).tofile(idf)
    outs = {}
    for gpus in (1, 2):
        of = str(tmp_path / f"out{gpus}.i32")
        p = subprocess.run([driver, "infer", "--config", yaml, "--ids-file", idf, "--streams", "5", "--gpus", str(gpus),
                            "--max_new", "16", "--temp", "0.8", "--top_k", "40", "--top_p", "0.95", "--seed", "77",
                            "--out-ids-file", of], capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        outs[gpus] = np.fromfile(of, np.int32).reshape(5, 16)
    assert np.array_equal(outs[1], outs[2])
