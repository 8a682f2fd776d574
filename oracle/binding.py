"""Test infrastructure, not product code.

ctypes binding of oracle/liboracle.so (the C restatement of the litnicelm
inference path) and helpers that run the reference itself, compiled under
oracle/_ref/, on explicit token ids. Only tests/, the smoke check and the CPU
baseline leg of bench.py may import this module.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
import tempfile
from typing import Optional, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_CPU_PLUGIN = os.path.join(REF_DIR, "liblitnice_backend_cpu.so")
REF_DRIVER = os.path.join(REF_DIR, "ref_driver")
REF_CLI = os.path.join(REF_DIR, "litnicelm")


class LoDims(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_heads", C.c_int32), ("d_model", C.c_int32),
                ("d_ff", C.c_int32), ("vocab", C.c_int32), ("max_seq", C.c_int32),
                ("alignment", C.c_int64)]


class LoMt(C.Structure):
    _fields_ = [("mt", C.c_uint32 * 624), ("idx", C.c_int32)]


_lib = None


def build() -> None:
    subprocess.run(["make", "-C", HERE, "-s"], check=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-C", HERE, "-s", "port"], check=True)
        _lib = C.CDLL(path)
        f32p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_int32)
        _lib.lo_forward.argtypes = [C.POINTER(LoDims), C.c_void_p, i32p, C.c_int32, f32p, C.c_int]
        _lib.lo_forward.restype = C.c_int
        _lib.lo_greedy.argtypes = [f32p, C.c_int32]
        _lib.lo_greedy.restype = C.c_int32
        _lib.lo_mt_seed.argtypes = [C.POINTER(LoMt), C.c_uint32]
        _lib.lo_mt_next.argtypes = [C.POINTER(LoMt)]
        _lib.lo_mt_next.restype = C.c_uint32
        _lib.lo_sample_ex.argtypes = [f32p, C.c_int32, C.c_float, C.c_uint32, C.c_float,
                                      C.POINTER(LoMt), i32p]
        _lib.lo_sample_ex.restype = C.c_int32
        _lib.lo_generate.argtypes = [C.POINTER(LoDims), C.c_void_p, i32p, C.c_int32, C.c_int32,
                                     C.c_float, C.c_uint32, C.c_float, C.c_uint32, i32p, f32p]
        _lib.lo_generate.restype = C.c_int32
        i64 = C.c_int64
        _lib.lo_gemm_strided.argtypes = [f32p, i64, f32p, i64, f32p, i64, i64, i64, i64]
        _lib.lo_gemm_rhs_t.argtypes = [f32p, i64, f32p, i64, f32p, i64, i64, i64, i64]
        _lib.lo_layernorm.argtypes = [f32p, f32p, f32p, f32p, i64, i64]
        _lib.lo_softmax_rows.argtypes = [f32p, f32p, i64, i64]
        _lib.lo_scaled_causal_softmax_rows.argtypes = [f32p, C.c_float, f32p, i64, i64]
    return _lib


def _f32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _dims(d) -> LoDims:
    return LoDims(d.n_layers, d.n_heads, d.d_model, d.d_ff, d.vocab, d.max_seq, d.alignment)


def forward(d, arena: np.ndarray, ids: np.ndarray, only_last: bool = False) -> np.ndarray:
    """Logits [s, V] (or [V] for the last row) of one stream."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    s = int(ids.shape[0])
    out = np.empty((d.vocab,) if only_last else (s, d.vocab), dtype=np.float32)
    rc = lib().lo_forward(C.byref(_dims(d)), arena.ctypes.data, _i32(ids), s, _f32(out),
                          1 if only_last else 0)
    if rc != 0:
        raise RuntimeError(f"lo_forward failed rc={rc}")
    return out


def generate(d, arena: np.ndarray, prompt: np.ndarray, max_new: int, temp: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = 12345,
             want_logits: bool = False) -> Tuple[np.ndarray, Optional[np.ndarray]]:
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    out = np.empty(max_new, dtype=np.int32)
    lg = np.empty((max_new, d.vocab), dtype=np.float32) if want_logits else None
    n = lib().lo_generate(C.byref(_dims(d)), arena.ctypes.data, _i32(prompt), len(prompt),
                          max_new, temp, top_k, top_p, seed, _i32(out),
                          _f32(lg) if want_logits else None)
    if n < 0:
        raise RuntimeError("lo_generate failed")
    return out[:n].copy(), (lg[:n].copy() if want_logits else None)


def gemm(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), np.float32)
    lib().lo_gemm_strided(_f32(a), k, _f32(b), n, _f32(out), n, m, k, n)
    return out


def gemm_rhs_t(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    m, k = a.shape
    n = b.shape[0]
    out = np.empty((m, n), np.float32)
    lib().lo_gemm_rhs_t(_f32(a), k, _f32(b), k, _f32(out), n, m, k, n)
    return out


def layernorm(x: np.ndarray, g: np.ndarray, b: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    g = np.ascontiguousarray(g, np.float32).ravel()
    b = np.ascontiguousarray(b, np.float32).ravel()
    out = np.empty_like(x)
    lib().lo_layernorm(_f32(x), _f32(g), _f32(b), _f32(out), x.shape[0], x.shape[1])
    return out


def softmax_rows(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().lo_softmax_rows(_f32(x), _f32(out), x.shape[0], x.shape[1])
    return out


def scaled_causal_softmax_rows(x: np.ndarray, scale: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().lo_scaled_causal_softmax_rows(_f32(x), scale, _f32(out), x.shape[0], x.shape[1])
    return out


class Sampler:
    """One generation's selector state: std::mt19937(seed) shared across steps."""

    def __init__(self, seed: int):
        self.g = LoMt()
        lib().lo_mt_seed(C.byref(self.g), seed)

    def next_u32(self) -> int:
        return int(lib().lo_mt_next(C.byref(self.g)))

    def pick(self, row: np.ndarray, temp: float, top_k: int, top_p: float) -> Tuple[int, int]:
        row = np.ascontiguousarray(row, np.float32)
        kept = C.c_int32(0)
        tok = lib().lo_sample_ex(_f32(row), len(row), temp, top_k, top_p, C.byref(self.g),
                                 C.byref(kept))
        return int(tok), int(kept.value)


def greedy(row: np.ndarray) -> int:
    row = np.ascontiguousarray(row, np.float32)
    return int(lib().lo_greedy(_f32(row), len(row)))


# ---- the reference itself (oracle/_ref) ------------------------------------

def have_ref() -> bool:
    return os.path.exists(REF_DRIVER) and os.path.exists(REF_CPU_PLUGIN)


def ref_run(d, arena: np.ndarray, ids: np.ndarray, *, mode: str = "forward",
            backend_library: Optional[str] = None, attention: str = "reference",
            ffn: str = "reference", max_new: int = 0, temp: float = 0.0, top_k: int = 0,
            top_p: float = 1.0, seed: int = 12345, want_logits: bool = False,
            workdir: Optional[str] = None, threads_env: Optional[dict] = None):
    """Run the reference's own model code (ref_driver) on explicit ids through
    the plugin `backend_library` (default: the reference CPU plugin).

    forward  -> (logits [s,V], info)
    generate -> (tokens, last-row logits per step or None, per-step seconds, info)
    """
    from litnicelm_b200 import formats

    lib_path = backend_library or REF_CPU_PLUGIN
    with tempfile.TemporaryDirectory(dir=workdir) as tmp:
        ckpt = os.path.join(tmp, "model.ckpt")
        formats.write_checkpoint(ckpt, d, arena)
        yaml = os.path.join(tmp, "cfg.yaml")
        formats.write_yaml(yaml, d, backend_library=lib_path, checkpoint=ckpt,
                           attention=attention, ffn=ffn)
        ids_path = os.path.join(tmp, "ids.i32")
        np.ascontiguousarray(ids, np.int32).tofile(ids_path)
        out = os.path.join(tmp, "out.bin")
        cmd = [REF_DRIVER, "--config", yaml, "--vocab", str(d.vocab), "--ids", ids_path,
               "--mode", mode, "--out", out]
        lg = os.path.join(tmp, "lg.f32")
        tm = os.path.join(tmp, "t.f64")
        if mode == "generate":
            cmd += ["--max-new", str(max_new), "--temp", repr(float(temp)), "--top-k", str(top_k),
                    "--top-p", repr(float(top_p)), "--seed", str(seed), "--times-out", tm]
            if want_logits:
                cmd += ["--logits-out", lg]
        env = dict(os.environ)
        if threads_env:
            env.update(threads_env)
        p = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if p.returncode != 0:
            raise RuntimeError(f"ref_driver failed: {p.stderr[-2000:]}\n{p.stdout[-500:]}")
        info = {}
        for line in p.stdout.splitlines():
            if line.startswith("{"):
                info = json.loads(line)
        if mode == "forward":
            return np.fromfile(out, np.float32).reshape(-1, d.vocab), info
        toks = np.fromfile(out, np.int32)
        logits = np.fromfile(lg, np.float32).reshape(-1, d.vocab) if want_logits else None
        return toks, logits, np.fromfile(tm, np.float64), info
