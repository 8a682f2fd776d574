"""Small fixed cases that launch every kernel family of the library once or a few
times, for one profiler capture that ends by itself:

    python -m litnicelm_b200.profile_kernels [--only head|loop|abi|cached|training]

  head      the few-row product of the output head at the config-4/5 shape
            (1024 x 32000 fp32, 131 MB per matrix, a ring of copies larger than
            the L2) with 1 and 8 rows, and the config-2 layer shapes
  loop      the native loop on the config-2 model at context 640: a greedy step
            (one-launch tail), a sampled step (final norm, head, sampler, state
            advance), inspect (probabilities in double); a vocabulary-32000
            model for the large-vocabulary sampler
  abi       operators of the plugin table on config-2 sized views: LayerNorm,
            softmax (plain and scaled-causal), row-wise family, causal mask,
            embedding, transpose, copy
  cached    two steps of the cached mode at context 640
  training  the training entries on 2048 x 512 rows

Prints one JSON line with what ran. Everything goes through the C ABI.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import formats
from .plugin import Backend, DevTensor, Session, gemv_time


def _dense(be, arr, dtype=0):
    arr = np.ascontiguousarray(arr)
    ptr = be.alloc(max(arr.nbytes, 4))
    be.upload(ptr, arr)
    strides, acc = [], 4
    for n in reversed(arr.shape):
        strides.insert(0, acc)
        acc *= n
    return DevTensor(ptr, tuple(arr.shape), tuple(strides), dtype, be.device)


def run_head(out):
    for m in (1, 8):
        us, nl = gemv_time(m, 1024, 32000, 3, 2)
        out[f"head_m{m}_us"] = us
    for (k, n) in ((512, 1536), (2048, 512), (1024, 4096)):
        us, nl = gemv_time(1, k, n, 3, 0)
        out[f"layer_{k}x{n}_us"] = us


def run_loop(out):
    d = formats.CONFIG_DIMS["c2"]
    arena = formats.make_param_arena(d, 1002)
    ids = formats.zipf_prompt(d.vocab, 640, 4000)
    with Session(d, 1) as s:
        s.load_params(arena)
        s.generate(ids, 2)                                        # greedy: one-launch tail
        s.generate(ids, 2, temp=0.8, top_k=40, top_p=0.95, seeds=[3000])  # sampled: norm, head, sampler, advance
        s.inspect(ids)
        out["loop_launches_last_call"] = int(s.stats().kernel_launches)
    dv = formats.ModelDims(1, 2, 64, 128, 32000, 32)
    with Session(dv, 4) as s:
        s.load_params(formats.make_param_arena(dv, 31))
        p = np.stack([formats.zipf_prompt(dv.vocab, 9, 70 + i) for i in range(4)])
        s.generate(p, 2, temp=0.8, top_k=40, top_p=0.95, seeds=[1, 2, 3, 4])
        s.generate(p, 2, temp=1.0, top_k=0, top_p=0.9, seeds=[1, 2, 3, 4])      # full-vocabulary sort
        s.generate(p, 2)


def run_abi(out):
    rng = np.random.default_rng(0)
    S, D, V = 640, 512, 96
    with Backend() as be:
        x = _dense(be, rng.standard_normal((1, S, D)).astype(np.float32))
        y = _dense(be, rng.standard_normal((1, S, D)).astype(np.float32))
        o = _dense(be, np.zeros((1, S, D), np.float32))
        g = _dense(be, np.ones((1, D), np.float32))
        b = _dense(be, np.zeros((1, D), np.float32))
        sc = _dense(be, rng.standard_normal((1, S, S)).astype(np.float32))
        so = _dense(be, np.zeros((1, S, S), np.float32))
        table = _dense(be, rng.standard_normal((V, D)).astype(np.float32))
        ids = _dense(be, rng.integers(0, V, size=(1, S)).astype(np.int32), dtype=1)
        t = _dense(be, np.zeros((D, S), np.float32))
        x2 = DevTensor(x.ptr, (S, D), (D * 4, 4), 0, be.device)
        for _ in range(2):
            be.call("layernorm_forward", x, g, b, o)
            be.call("softmax_rows", sc, so)
            be.call("scaled_causal_softmax_rows", sc, 0.125, so)
            be.call("apply_causal_mask_inplace", so, -1e9)
            be.call("add", x, y, o)
            be.call("add_bias_rowwise", x, b, o)
            be.call("add_bias_relu_rowwise", x, b, o)
            be.call("relu", x, o)
            be.call("mul_scalar", x, 0.125, o)
            be.call("fill", o, 0.0)
            be.call("copy", x, o)
            be.call("embedding_lookup", table, ids, o)
            be.call("transpose", x2, t)
        be.download(o.ptr, 16)
    out["abi"] = "ok"


def run_cached(out):
    os.environ["LITNICE_B200_KV_CACHE"] = "1"
    try:
        d = formats.CONFIG_DIMS["c2"]
        with Session(d, 1) as s:
            s.load_params(formats.make_param_arena(d, 1002))
            s.generate(formats.zipf_prompt(d.vocab, 638, 4000), 3)
            out["cached_launches"] = int(s.stats().kernel_launches)
    finally:
        del os.environ["LITNICE_B200_KV_CACHE"]


def run_training(out):
    rng = np.random.default_rng(1)
    B, S, D, V = 8, 256, 512, 96
    with Backend() as be:
        x = _dense(be, rng.standard_normal((B, S, D)).astype(np.float32))
        dy = _dense(be, rng.standard_normal((B, S, D)).astype(np.float32))
        dx = _dense(be, np.zeros((B, S, D), np.float32))
        g = _dense(be, np.ones((1, D), np.float32))
        dg = _dense(be, np.zeros((1, D), np.float32))
        db = _dense(be, np.zeros((1, D), np.float32))
        w = _dense(be, (rng.standard_normal((D, D)) * 0.02).astype(np.float32))
        dw = _dense(be, np.zeros((D, D), np.float32))
        logits = _dense(be, rng.standard_normal((B, S, V)).astype(np.float32))
        targets = _dense(be, rng.integers(0, V, size=(B, S)).astype(np.int32), dtype=1)
        loss = _dense(be, np.zeros((1, 1), np.float32))
        ids = _dense(be, rng.integers(0, V, size=(B, S)).astype(np.int32), dtype=1)
        tok = _dense(be, np.zeros((V, D), np.float32))
        pos = _dense(be, np.zeros((S, D), np.float32))
        sm = _dense(be, np.full((B, S, S), 1.0 / S, np.float32))
        ds = _dense(be, rng.standard_normal((B, S, S)).astype(np.float32))
        do = _dense(be, np.zeros((B, S, S), np.float32))
        p = _dense(be, rng.standard_normal((D, D)).astype(np.float32))
        m = _dense(be, np.zeros((D, D), np.float32))
        v = _dense(be, np.zeros((D, D), np.float32))
        be.call("layernorm_backward", x, g, dy, dx, dg, db)
        be.call("row_sum", dy, db)
        be.call("relu_backward", x, dy, dx)
        be.call("gemm_ranked_matrix_rhs_t", dy, w, dx)
        be.call("gemm_ranked_reduce_lhs_t", x, dy, dw)
        be.call("cross_entropy_mean_backward_inplace", logits, targets, loss)
        be.call("accumulate_embedding_grads", ids, dy, tok, pos)
        be.call("softmax_backward_rows", sm, ds, do)
        be.call("softmax_backward_causal_rows", sm, ds, do)
        be.call("adamw_step", p, dw, m, v, 1, 0.002, 0.9, 0.999, 0.01, 1)
        out["grad_sum_squares"] = float(be.call("sum_squares_f32", dw))
        out["loss"] = float(be.call("read_scalar_f32", loss))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", choices=["", "head", "loop", "abi", "cached", "training"])
    args = ap.parse_args()
    out = {}
    for name, fn in (("head", run_head), ("loop", run_loop), ("abi", run_abi), ("cached", run_cached),
                     ("training", run_training)):
        if args.only in ("", name):
            fn(out)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
