"""Host-side mirror of the litnicelm data formats the inference path reads.

Everything here is byte-level bookkeeping on the host: where each parameter
lives inside the parameter arena, how a version-6 checkpoint file is laid out,
what the tokenised-dataset header looks like and which YAML keys the reference
configuration loader insists on. The functions cite the reference files they
mirror (paths inside the litnicelm tree).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Tuple

import numpy as np

CKPT_MAGIC = 0x4C474354  # checkpoint.cpp:98-116
CKPT_VERSION = 6
CKPT_ALGO_VERSION = 1
CKPT_HEADER_BYTES = 136
DATASET_MAGIC = 0x4C4E4750  # dataset.cpp:16-19


@dataclass(frozen=True)
class ModelDims:
    """model.* and memory.alignment_bytes of a litnicelm YAML (types.hpp:134-146)."""

    n_layers: int
    n_heads: int
    d_model: int
    d_ff: int
    vocab: int
    max_seq: int
    alignment: int = 64

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads


# The five benchmark shapes (vocab, max_seq_len, layers, heads, d_model, d_ff).
CONFIG_DIMS: Dict[str, ModelDims] = {
    "c1": ModelDims(2, 2, 64, 256, 8, 64),
    "c2": ModelDims(6, 8, 512, 2048, 96, 1024),
    "c3": ModelDims(6, 8, 512, 2048, 96, 1024),
    "c4": ModelDims(12, 16, 1024, 4096, 32000, 2048),
    "c5": ModelDims(12, 16, 1024, 4096, 32000, 2048),
    # the one YAML the reference ships for CPU (conf/char_book_abcdef_cpu.yaml:33-38)
    "abcdef": ModelDims(2, 2, 32, 64, 8, 8),
}


def _align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class ParamLayout:
    """Byte offset and shape of every parameter (named_layout.cpp:40-161).

    Parameters that take weight decay (embeddings and matrices) are packed
    first in declaration order, each aligned; that zone is padded to the
    alignment; LayerNorm vectors and biases follow in declaration order.
    """

    dims: ModelDims
    slices: Dict[str, Tuple[int, Tuple[int, int]]] = field(default_factory=dict)
    decay_bytes: int = 0
    total_bytes: int = 0

    @staticmethod
    def build(d: ModelDims) -> "ParamLayout":
        D, F, V, S, A = d.d_model, d.d_ff, d.vocab, d.max_seq, d.alignment
        specs: List[Tuple[str, Tuple[int, int], bool]] = [
            ("tok_embedding", (V, D), True),
            ("pos_embedding", (S, D), True),
        ]
        for l in range(d.n_layers):
            p = f"layer{l}."
            specs += [
                (p + "ln1_gamma", (1, D), False), (p + "ln1_beta", (1, D), False),
                (p + "attn_qkv_w", (D, 3 * D), True), (p + "attn_qkv_b", (1, 3 * D), False),
                (p + "attn_out_w", (D, D), True), (p + "attn_out_b", (1, D), False),
                (p + "ln2_gamma", (1, D), False), (p + "ln2_beta", (1, D), False),
                (p + "ffn_w1", (D, F), True), (p + "ffn_b1", (1, F), False),
                (p + "ffn_w2", (F, D), True), (p + "ffn_b2", (1, D), False),
            ]
        specs += [("lnf_gamma", (1, D), False), ("lnf_beta", (1, D), False),
                  ("lm_head_w", (D, V), True)]
        out = ParamLayout(d)
        cur = 0
        for name, shape, decay in specs:
            if decay:
                cur = _align_up(cur, A)
                out.slices[name] = (cur, shape)
                cur += 4 * shape[0] * shape[1]
        out.decay_bytes = _align_up(cur, A)
        cur = out.decay_bytes
        for name, shape, decay in specs:
            if not decay:
                cur = _align_up(cur, A)
                out.slices[name] = (cur, shape)
                cur += 4 * shape[0] * shape[1]
        out.total_bytes = _align_up(cur, A)
        return out

    def view(self, arena: np.ndarray, name: str) -> np.ndarray:
        """Float32 view of one parameter inside a uint8 arena image."""
        off, shape = self.slices[name]
        n = shape[0] * shape[1]
        return arena[off:off + 4 * n].view(np.float32).reshape(shape)


def make_param_arena(d: ModelDims, seed: int, bias_std: float = 0.0, ln_std: float = 0.0) -> np.ndarray:
    """Seeded synthetic weights as a parameter-arena image (uint8).

    Matrices and embeddings are N(0, 0.02); LayerNorm gamma 1, beta 0; biases 0
    (or N(0, bias_std) for the harder variant; ln_std > 0 also draws gamma from
    1 + N(0, ln_std) and beta from N(0, ln_std), from a generator of their own
    so that the other values do not change). The reference has no seeded
    initialiser of its own for inference (it loads a checkpoint,
    inference.cpp:73-91), so both sides read the same image.
    """
    lay = ParamLayout.build(d)
    arena = np.zeros(lay.total_bytes, dtype=np.uint8)
    rng = np.random.default_rng(seed)
    ln_rng = np.random.default_rng(seed + 7919)
    for name, (off, shape) in lay.slices.items():
        v = lay.view(arena, name)
        base = name.split(".")[-1]
        if base.endswith("gamma"):
            v[...] = 1.0
            if ln_std > 0:
                v[...] += ln_rng.normal(0.0, ln_std, size=shape).astype(np.float32)
        elif base.endswith("beta"):
            v[...] = 0.0
            if ln_std > 0:
                v[...] = ln_rng.normal(0.0, ln_std, size=shape).astype(np.float32)
        elif shape[0] == 1:  # biases
            if bias_std > 0:
                v[...] = rng.normal(0.0, bias_std, size=shape).astype(np.float32)
        else:
            v[...] = rng.normal(0.0, 0.02, size=shape).astype(np.float32)
    return arena


def write_checkpoint(path: str, d: ModelDims, arena: np.ndarray, conf_version: str = "1") -> None:
    """Version-6 checkpoint: 136-byte header, parameter arena, optimiser arena
    of twice the size (zeros) (checkpoint.cpp:98-116, 244-298, 588-652)."""
    lay = ParamLayout.build(d)
    assert arena.nbytes == lay.total_bytes
    cv = conf_version.encode()[:31].ljust(32, b"\0")
    hdr = struct.pack("<III32sIIIIII4xQQIIQQffIIII",
                      CKPT_MAGIC, CKPT_VERSION, CKPT_ALGO_VERSION, cv,
                      d.n_layers, d.n_heads, d.d_model, d.d_ff, d.vocab, d.max_seq,
                      d.alignment, 0, 0, 0, lay.total_bytes, 2 * lay.total_bytes,
                      0.0, -1.0, 0, 0, 0, 0)
    assert len(hdr) == CKPT_HEADER_BYTES, len(hdr)
    with open(path, "wb") as f:
        f.write(hdr)
        f.write(arena.tobytes())
        zeros = bytes(1 << 20)
        left = 2 * lay.total_bytes
        while left > 0:
            n = min(left, len(zeros))
            f.write(zeros[:n])
            left -= n


def read_checkpoint(path: str) -> Tuple[ModelDims, np.ndarray]:
    """Header dims and the parameter-arena image of a version-6 checkpoint."""
    with open(path, "rb") as f:
        hdr = f.read(CKPT_HEADER_BYTES)
        (magic, ver, _algo, _cv, L, H, D, F, V, S, align, _step, _epoch, _res, data_bytes,
         _adam) = struct.unpack("<III32sIIIIII4xQQIIQQ", hdr[:112])
        if magic != CKPT_MAGIC or ver != CKPT_VERSION:
            raise ValueError(f"{path}: not a version-6 litnicelm checkpoint")
        arena = np.frombuffer(f.read(data_bytes), dtype=np.uint8).copy()
    if arena.nbytes != data_bytes:
        raise ValueError(f"{path}: truncated parameter arena")
    return ModelDims(L, H, D, F, V, S, align), arena


def write_dataset_header(path: str, vocab: int) -> None:
    """Header-only tokenised dataset: magic, version 1, vocab (dataset.cpp:87-124).
    Inference reads nothing else from it (inference.cpp:28-41)."""
    with open(path, "wb") as f:
        f.write(struct.pack("<III", DATASET_MAGIC, 1, vocab))


def write_char_seen(artifacts_dir: str, vocab_chars: Iterable[str]) -> None:
    """Vocabulary file of the only_seen_chars tokenizer: id = position in the
    list (only_seen_chars_tokenizer_plugin.cpp:126-160,249-262)."""
    os.makedirs(artifacts_dir, exist_ok=True)
    with open(os.path.join(artifacts_dir, "char_seen.json"), "w") as f:
        json.dump({"vocab": list(vocab_chars)}, f)


def write_yaml(path: str, d: ModelDims, *, backend_library: str, checkpoint: str,
               dataset_bin: str = "unused.bin", tokenizer_type: str = "character",
               artifacts_dir: str = "", attention: str = "reference", ffn: str = "reference",
               prompt: str = "", max_new: int = 64, temp: float = 0.0, top_k: int = 0,
               top_p: float = 1.0, seed: int = 12345, corpus: str = "unused.txt",
               train_seq_len: int = 4, batch_size: int = 2) -> None:
    """A litnicelm YAML holding every key the loader requires
    (config_mapper.cpp:124-189) and none it does not know (:713-716)."""
    text = f"""conf:
  version: "1"

transformer_layers: 0
parameter_bytes: 0
optimizer_bytes: 0
arena_alignment: {d.alignment}
max_steps: 1

backend:
  library: "{backend_library}"

tokenizer:
  type: "{tokenizer_type}"
  target_vocab_size: {d.vocab}
  training_corpus: "{corpus}"
  inter_file_boundary: "\\n"
  artifacts_dir: "{artifacts_dir}"
  bpe_vocab_file: ""
  bpe_merges_file: ""
  bpe_validation_num_threads: 1
  bpe_validation_sample_rate: 50
  run_validation: false

tokenization:
  input_corpus: "{corpus}"
  output_binary: "{dataset_bin}"
  chunk_size_mb: 16

memory:
  alignment_bytes: {d.alignment}

model:
  n_layers: {d.n_layers}
  n_heads: {d.n_heads}
  d_model: {d.d_model}
  d_ff: {d.d_ff}
  max_seq_len: {d.max_seq}

model_algo:
  attention: "{attention}"
  ffn: "{ffn}"

training:
  learning_rate: 0.002
  beta1: 0.9
  beta2: 0.999
  eps: 0.00000001
  weight_decay: 0.01
  incremental: false
  dry_run: false
  num_epochs_train: 1
  num_epochs_dry_run: 1
  save_interval_epochs: 1
  grad_clip: 1.0
  train_seq_len: {train_seq_len}
  window_stride: {train_seq_len}
  batch_size: {batch_size}
  target_loss: -1.0
  min_delta: 0.0
  patience_epochs: 0
  min_epochs: 0
  stop_on_nonfinite_loss: true

paths:
  model_file_latest: "{checkpoint}.latest"
  model_file_best: "{checkpoint}"
  journal_file: "{checkpoint}.journal"

inference:
  prompt: "{prompt}"
  max_new: {max_new}
  temp: {temp}
  top_k: {top_k}
  top_p: {top_p}
  seed: {seed}

logging:
  show_bpe: false
  show_train: false
  show_inference: true
  report_every_n_steps: 1
  epoch_report_every: 1

reporting:
  verbose_epoch_index: [-1, 0]
  verbose_init: false
"""
    with open(path, "w") as f:
        f.write(text)


def zipf_prompt(vocab: int, length: int, seed: int, s: float = 1.1) -> np.ndarray:
    """i.i.d. Zipf(s) token ids over ranks 1..vocab, id = rank-1, by inverse CDF
    on seeded uniforms. Stands in for corpus text the reference was run on."""
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    u = np.random.default_rng(seed).random(length)
    return np.minimum(np.searchsorted(cdf, u, side="left"), vocab - 1).astype(np.int32)
