"""ctypes access to liblitnice_backend_b200.so.

Two thin layers over the C ABI declared in include/litnice_backend_b200.h:

* ``Backend`` drives the litnicelm plugin table (BackendApiV1) the way the
  reference's DynamicLibraryBackend does (src/model/backend/device_backend.cpp:
  180-654): create(GPU), alloc, host<->device copies, one call per operator with
  byte-strided views. It works with any library exporting
  ``litnice_backend_get_api`` (the reference CPU plugin included), which is how
  the tests compare two plugins on identical views.
* ``Session`` drives the native token loop (litnice_b200_*).

There is no fallback: if the shared library is missing or no CUDA device is
present, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

from .formats import ModelDims

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblitnice_backend_b200.so")
MAX_RANK = 6


class BackendTensorView(C.Structure):
    _fields_ = [("device", C.c_uint32), ("dtype", C.c_uint32), ("data", C.c_void_p),
                ("rank", C.c_uint32), ("rows", C.c_int64), ("cols", C.c_int64),
                ("stride_r_bytes", C.c_int64), ("stride_c_bytes", C.c_int64),
                ("dims", C.c_int64 * MAX_RANK), ("strides_bytes", C.c_int64 * MAX_RANK)]


class BackendMemoryInfo(C.Structure):
    _fields_ = [("available", C.c_uint32), ("free_bytes", C.c_uint64), ("total_bytes", C.c_uint64)]


_V = C.POINTER(BackendTensorView)
_H = C.c_void_p


def _fn(res, *args):
    return C.CFUNCTYPE(res, *args)


# Order of backend_plugin_api.hpp:26-162.
_API_FIELDS = [
    ("abi_version", C.c_uint32),
    ("create", _fn(C.c_void_p, C.c_uint32)),
    ("destroy", _fn(None, _H)),
    ("device", _fn(C.c_uint32, _H)),
    ("alloc", _fn(C.c_void_p, _H, C.c_uint64, C.c_uint32)),
    ("free", _fn(None, _H, C.c_void_p)),
    ("copy_host2device", _fn(None, _H, C.c_void_p, C.c_void_p, C.c_uint64)),
    ("copy_device2host", _fn(None, _H, C.c_void_p, C.c_void_p, C.c_uint64)),
    ("copy", _fn(None, _H, _V, _V)),
    ("fill", _fn(None, _H, _V, C.c_float)),
    ("add", _fn(None, _H, _V, _V, _V)),
    ("add_inplace", _fn(None, _H, _V, _V)),
    ("add_bias_rowwise", _fn(None, _H, _V, _V, _V)),
    ("add_bias_relu_rowwise", _fn(None, _H, _V, _V, _V)),
    ("add_bias_relu_rowwise_inplace", _fn(None, _H, _V, _V)),
    ("mul_scalar", _fn(None, _H, _V, C.c_float, _V)),
    ("sum_squares_f32", _fn(C.c_float, _H, _V)),
    ("relu", _fn(None, _H, _V, _V)),
    ("relu_backward", _fn(None, _H, _V, _V, _V)),
    ("relu_backward_inplace", _fn(None, _H, _V, _V)),
    ("row_sum", _fn(None, _H, _V, _V)),
    ("gemm", _fn(None, _H, _V, _V, _V)),
    ("gemm_ranked_matrix_rhs", _fn(None, _H, _V, _V, _V)),
    ("gemm_ranked_matrix_rhs_t", _fn(None, _H, _V, _V, _V)),
    ("gemm_ranked_reduce_lhs_t", _fn(None, _H, _V, _V, _V)),
    ("gemm_batched", _fn(None, _H, _V, _V, _V)),
    ("gemm_batched_lhs_t", _fn(None, _H, _V, _V, _V)),
    ("gemm_batched_rhs_t", _fn(None, _H, _V, _V, _V)),
    ("transpose", _fn(None, _H, _V, _V)),
    ("layernorm_forward", _fn(None, _H, _V, _V, _V, _V)),
    ("layernorm_backward", _fn(None, _H, _V, _V, _V, _V, _V, _V)),
    ("embedding_lookup", _fn(None, _H, _V, _V, _V)),
    ("accumulate_embedding_grads", _fn(None, _H, _V, _V, _V, _V)),
    ("cross_entropy_mean", _fn(None, _H, _V, _V, _V)),
    ("cross_entropy_mean_backward_inplace", _fn(None, _H, _V, _V, _V)),
    ("read_scalar_f32", _fn(C.c_float, _H, _V)),
    ("backward_from_logits_targets", _fn(None, _H, _V, _V)),
    ("softmax_rows", _fn(None, _H, _V, _V)),
    ("softmax_backward_rows", _fn(None, _H, _V, _V, _V)),
    ("scaled_causal_softmax_rows", _fn(None, _H, _V, C.c_float, _V)),
    ("supports_exec_context_iteration", _fn(C.c_uint32, _H)),
    ("start_exec_context_iteration", _fn(None, _H)),
    ("finish_exec_context_iteration", _fn(None, _H)),
    ("start_exec_context_group", _fn(None, _H)),
    ("finish_exec_context_group", _fn(None, _H)),
    ("gemm_batched_exec_context", _fn(None, _H, _V, _V, _V)),
    ("gemm_batched_lhs_t_exec_context", _fn(None, _H, _V, _V, _V)),
    ("gemm_batched_rhs_t_exec_context", _fn(None, _H, _V, _V, _V)),
    ("scaled_causal_softmax_rows_exec_context", _fn(None, _H, _V, C.c_float, _V)),
    ("softmax_backward_causal_rows_exec_context", _fn(None, _H, _V, _V, _V)),
    ("softmax_backward_causal_rows", _fn(None, _H, _V, _V, _V)),
    ("apply_causal_mask_inplace", _fn(None, _H, _V, C.c_float)),
    ("adamw_step", _fn(None, _H, _V, _V, _V, _V, C.c_uint64, C.c_float, C.c_float, C.c_float,
                       C.c_float, C.c_uint32)),
    ("is_file2device_read_supported", _fn(C.c_uint32, _H)),
    ("read_file2device", _fn(None, _H, C.c_char_p, C.c_void_p, C.c_uint64, C.c_uint64)),
    ("memory_info", _fn(BackendMemoryInfo, _H)),
]


class BackendApiV1(C.Structure):
    _fields_ = _API_FIELDS


API_ENTRY_NAMES = [name for name, _ in _API_FIELDS[1:]]

# What a host of the native loop binds (the diagnostics of the header's third section are
# left out on purpose).
NATIVE_SYMBOLS = [
    "litnice_b200_session_create", "litnice_b200_session_create_on", "litnice_b200_session_destroy",
    "litnice_b200_last_error",
    "litnice_b200_load_params", "litnice_b200_load_checkpoint", "litnice_b200_generate",
    "litnice_b200_upload_prompts", "litnice_b200_run", "litnice_b200_download_tokens",
    "litnice_b200_keep_step_logits", "litnice_b200_read_step_logits", "litnice_b200_forward",
    "litnice_b200_inspect", "litnice_b200_sample_logits", "litnice_b200_get_stats",
    "litnice_b200_gemv_noalloc",
]


def load_library(path: Optional[str] = None) -> C.CDLL:
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `make -C litnicelm_b200/csrc` "
                           "(there is no CPU fallback)")
    return C.CDLL(path)


def get_api(lib: C.CDLL) -> BackendApiV1:
    lib.litnice_backend_get_api.restype = C.POINTER(BackendApiV1)
    api = lib.litnice_backend_get_api()
    if not api or api.contents.abi_version != 16:
        raise RuntimeError("backend ABI mismatch")
    return api.contents


def projection_time(m: int, k: int, n: int, repeats: int = 20, engine: int = 1,
                    lib: Optional[C.CDLL] = None) -> float:
    """Average device time in microseconds of one C[m,n] = A[m,k]·W[k,n] on the
    tensor-core (engine 1) or SIMT (engine 0) projection kernel, warm, launched
    back to back (litnice_b200_projection_time)."""
    lib = lib or load_library()
    f32p = C.POINTER(C.c_float)
    fn = lib.litnice_b200_projection_time
    fn.argtypes = [C.c_int32, f32p, C.c_int32, C.c_int32, f32p, C.c_int32, f32p, C.c_int32, C.POINTER(C.c_double)]
    fn.restype = C.c_int
    rng = np.random.default_rng(0)
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = (rng.standard_normal((k, n), dtype=np.float32) * 0.02).astype(np.float32)
    c = np.empty((m, n), np.float32)
    us = C.c_double(0)
    rc = fn(engine, a.ctypes.data_as(f32p), m, k, w.ctypes.data_as(f32p), n, c.ctypes.data_as(f32p), repeats,
            C.byref(us))
    if rc != 0:
        raise RuntimeError(f"litnice_b200_projection_time failed with status {rc}")
    return us.value


def gemv_host(x: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray] = None,
              residual: Optional[np.ndarray] = None, relu: bool = False,
              ln: Optional[Tuple[np.ndarray, np.ndarray]] = None,
              lib: Optional[C.CDLL] = None) -> np.ndarray:
    """out[m, n] = x[m, k] . W[k, n] (+ bias) (+ residual) (ReLU) for m <= 8 on the few-row
    kernels of the output head (litnice_b200_gemv_host: host buffers in, host buffer out)."""
    lib = lib or load_library()
    f32p = C.POINTER(C.c_float)
    fn = lib.litnice_b200_gemv_host
    fn.argtypes = [f32p, C.c_int32, f32p, C.c_int32, C.c_int32, f32p, f32p, C.c_int32, f32p, f32p, f32p]
    fn.restype = C.c_int
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    m, k = x.shape
    n = w.shape[1]
    out = np.empty((m, n), np.float32)
    b = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, np.float32).ravel()
        b = bias.ctypes.data_as(f32p)
    r = None
    if residual is not None:
        residual = np.ascontiguousarray(residual, np.float32)
        r = residual.ctypes.data_as(f32p)
    g = be = None
    if ln is not None:   # (gamma, beta): the rows of x pass through LayerNorm inside the kernel
        gamma = np.ascontiguousarray(ln[0], np.float32).ravel()
        beta = np.ascontiguousarray(ln[1], np.float32).ravel()
        g, be = gamma.ctypes.data_as(f32p), beta.ctypes.data_as(f32p)
    rc = fn(x.ctypes.data_as(f32p), m, w.ctypes.data_as(f32p), k, n, b, r, 1 if relu else 0, g, be,
            out.ctypes.data_as(f32p))
    if rc != 0:
        raise RuntimeError(f"litnice_b200_gemv_host failed with status {rc}")
    return out


def gemv_time(m: int, k: int, n: int, repeats: int = 50, cold_l2: int = 2, force_tn: int = 0,
              force_splits: int = 0, lib: Optional[C.CDLL] = None) -> Tuple[float, int]:
    """(mean device microseconds, kernels per call) of the few-row product. cold_l2 = 2:
    `repeats` calls back to back between one pair of CUDA events, each on the next of a
    ring of weight copies larger than three times the L2 (every call reads HBM);
    1: events around each call, a 256 MB buffer written before it; 0: the same matrix
    every call (L2-resident when it fits)."""
    lib = lib or load_library()
    fn = lib.litnice_b200_gemv_time
    fn.argtypes = [C.c_int32] * 7 + [C.POINTER(C.c_double), C.POINTER(C.c_int32)]
    fn.restype = C.c_int
    us, nl = C.c_double(0), C.c_int32(0)
    rc = fn(m, k, n, repeats, int(cold_l2), force_tn, force_splits, C.byref(us), C.byref(nl))
    if rc != 0:
        raise RuntimeError(f"litnice_b200_gemv_time failed with status {rc}")
    return us.value, nl.value


@dataclass
class DevTensor:
    """A byte-strided view into plugin-allocated memory (TensorView of the
    reference, src/model/tensor.hpp:121-323)."""
    ptr: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]  # bytes
    dtype: int = 0            # 0 f32, 1 i32
    device: int = 1

    def view(self) -> BackendTensorView:
        v = BackendTensorView()
        v.device, v.dtype, v.data, v.rank = self.device, self.dtype, self.ptr, len(self.shape)
        v.rows = self.shape[0]
        v.cols = self.shape[1] if len(self.shape) > 1 else 0
        v.stride_r_bytes = self.strides[-2] if len(self.shape) >= 2 else 0
        v.stride_c_bytes = self.strides[-1]
        for i, (d, s) in enumerate(zip(self.shape, self.strides)):
            v.dims[i], v.strides_bytes[i] = d, s
        return v


class Backend:
    """One plugin instance, driven as the reference host drives it."""

    def __init__(self, lib_path: Optional[str] = None, device_kinds: Sequence[int] = (1, 0)):
        self.lib = load_library(lib_path)
        self.api = get_api(self.lib)
        self.h = None
        for kind in device_kinds:  # device_backend.cpp:208-220
            self.h = self.api.create(kind)
            if self.h:
                break
        if not self.h:
            raise RuntimeError("backend create failed")
        self.device = int(self.api.device(self.h))
        self._allocs = []

    def close(self):
        if self.h:
            for p in self._allocs:
                self.api.free(self.h, p)
            self._allocs = []
            self.api.destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def alloc(self, nbytes: int, alignment: int = 64) -> int:
        p = self.api.alloc(self.h, nbytes, alignment)
        if not p:
            raise MemoryError("plugin alloc returned null")
        self._allocs.append(p)
        return int(p)

    def upload(self, ptr: int, arr: np.ndarray, offset: int = 0):
        arr = np.ascontiguousarray(arr)
        self.api.copy_host2device(self.h, ptr + offset, arr.ctypes.data, arr.nbytes)

    def download(self, ptr: int, nbytes: int, offset: int = 0) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        self.api.copy_device2host(self.h, out.ctypes.data, ptr + offset, nbytes)
        return out

    def put(self, buffer_ptr: int, t: DevTensor, values: np.ndarray, buffer_bytes: int):
        """Scatter `values` (logical shape of t) into the strided view t by
        rewriting the whole backing buffer from the host."""
        host = self.download(buffer_ptr, buffer_bytes)
        dt = np.float32 if t.dtype == 0 else np.int32
        view = np.lib.stride_tricks.as_strided(
            host[t.ptr - buffer_ptr:].view(dt), shape=t.shape, strides=t.strides, writeable=True)
        view[...] = values
        self.upload(buffer_ptr, host)

    def get(self, buffer_ptr: int, t: DevTensor, buffer_bytes: int) -> np.ndarray:
        host = self.download(buffer_ptr, buffer_bytes)
        dt = np.float32 if t.dtype == 0 else np.int32
        return np.lib.stride_tricks.as_strided(host[t.ptr - buffer_ptr:].view(dt), shape=t.shape,
                                               strides=t.strides).copy()

    def call(self, name: str, *args):
        """Invoke a table entry; DevTensor arguments become view pointers."""
        conv = []
        keep = []
        for a in args:
            if isinstance(a, DevTensor):
                v = a.view()
                keep.append(v)
                conv.append(C.byref(v))
            else:
                conv.append(a)
        return getattr(self.api, name)(self.h, *conv)


class B200Dims(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_heads", C.c_int32), ("d_model", C.c_int32),
                ("d_ff", C.c_int32), ("vocab_size", C.c_int32), ("max_seq_len", C.c_int32),
                ("alignment_bytes", C.c_uint64)]


class B200Sampling(C.Structure):
    _fields_ = [("temp", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float)]


class B200Stats(C.Structure):
    _fields_ = [("device_ms", C.c_double), ("kernel_launches", C.c_int64), ("tokens", C.c_int64),
                ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64), ("gemm_ms", C.c_double),
                ("gemm_launches", C.c_int64), ("gemm_flops", C.c_double), ("attn_ms", C.c_double),
                ("attn_launches", C.c_int64), ("gemm_span_ms", C.c_double), ("gemm_span_launches", C.c_int64),
                ("gemm_span_flops", C.c_double), ("attn_span_ms", C.c_double), ("attn_span_launches", C.c_int64),
                ("step_span_ms", C.c_double)]


class NativeError(RuntimeError):
    pass


class Session:
    """Native token loop: generate_text of the reference (inference.cpp:265-296)
    for n independent streams in lockstep, entirely on the GPU."""

    def __init__(self, dims: ModelDims, max_streams: int = 1, lib_path: Optional[str] = None,
                 device: Optional[int] = None):
        self.lib = load_library(lib_path)
        L = self.lib
        i32p, f32p, u32p = C.POINTER(C.c_int32), C.POINTER(C.c_float), C.POINTER(C.c_uint32)
        L.litnice_b200_session_create.argtypes = [C.POINTER(B200Dims), C.c_int32, C.POINTER(C.c_void_p)]
        L.litnice_b200_session_destroy.argtypes = [C.c_void_p]
        L.litnice_b200_session_destroy.restype = None
        L.litnice_b200_last_error.argtypes = [C.c_void_p]
        L.litnice_b200_last_error.restype = C.c_char_p
        L.litnice_b200_load_params.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.litnice_b200_load_checkpoint.argtypes = [C.c_void_p, C.c_char_p]
        L.litnice_b200_generate.argtypes = [C.c_void_p, i32p, C.c_int32, C.c_int32, C.c_int32,
                                            C.POINTER(B200Sampling), u32p, i32p, i32p]
        L.litnice_b200_upload_prompts.argtypes = [C.c_void_p, i32p, C.c_int32, C.c_int32, u32p]
        L.litnice_b200_run.argtypes = [C.c_void_p, C.c_int32, C.POINTER(B200Sampling), i32p]
        L.litnice_b200_download_tokens.argtypes = [C.c_void_p, i32p, C.c_int32]
        L.litnice_b200_keep_step_logits.argtypes = [C.c_void_p, C.c_int32]
        L.litnice_b200_read_step_logits.argtypes = [C.c_void_p, f32p, C.c_int64]
        L.litnice_b200_forward.argtypes = [C.c_void_p, i32p, C.c_int32, C.c_int32, C.c_int32, f32p]
        L.litnice_b200_inspect.argtypes = [C.c_void_p, i32p, C.c_int32, C.c_int32, f32p]
        L.litnice_b200_sample_logits.argtypes = [C.c_void_p, f32p, C.c_int32, C.POINTER(B200Sampling),
                                                 u32p, C.c_int32, i32p]
        L.litnice_b200_get_stats.argtypes = [C.c_void_p, C.POINTER(B200Stats)]
        L.litnice_b200_profile_step.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]
        self.dims = dims
        self.max_streams = max_streams
        cd = B200Dims(dims.n_layers, dims.n_heads, dims.d_model, dims.d_ff, dims.vocab, dims.max_seq,
                      dims.alignment)
        self.h = C.c_void_p()
        if device is None:
            rc = L.litnice_b200_session_create(C.byref(cd), max_streams, C.byref(self.h))
        else:
            L.litnice_b200_session_create_on.argtypes = [C.POINTER(B200Dims), C.c_int32, C.c_int32,
                                                         C.POINTER(C.c_void_p)]
            rc = L.litnice_b200_session_create_on(C.byref(cd), max_streams, device, C.byref(self.h))
        if rc != 0:
            msg = L.litnice_b200_last_error(self.h).decode() if self.h else "no session"
            if self.h:
                L.litnice_b200_session_destroy(self.h)
                self.h = None
            raise NativeError(f"session_create failed ({rc}): {msg}")

    def close(self):
        if self.h:
            self.lib.litnice_b200_session_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise NativeError(f"{what} failed ({rc}): {self.lib.litnice_b200_last_error(self.h).decode()}")

    @staticmethod
    def _i32(a):
        return a.ctypes.data_as(C.POINTER(C.c_int32))

    @staticmethod
    def _f32(a):
        return a.ctypes.data_as(C.POINTER(C.c_float))

    def load_params(self, arena: np.ndarray):
        arena = np.ascontiguousarray(arena)
        self._check(self.lib.litnice_b200_load_params(self.h, arena.ctypes.data, arena.nbytes), "load_params")

    def load_checkpoint(self, path: str):
        self._check(self.lib.litnice_b200_load_checkpoint(self.h, path.encode()), "load_checkpoint")

    def keep_step_logits(self, enable: bool):
        self._check(self.lib.litnice_b200_keep_step_logits(self.h, 1 if enable else 0), "keep_step_logits")

    def _seeds(self, seeds, n):
        if seeds is None:
            return None, None
        arr = np.ascontiguousarray(seeds, dtype=np.uint32)
        assert arr.shape == (n,)
        return arr, arr.ctypes.data_as(C.POINTER(C.c_uint32))

    def generate(self, prompts: np.ndarray, max_new: int, temp: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, seeds=None) -> np.ndarray:
        """prompts [n_streams, prompt_len] int32 -> tokens [n_streams, produced]."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int32)
        if prompts.ndim == 1:
            prompts = prompts[None, :]
        n, plen = prompts.shape
        out = np.zeros((n, max(1, max_new)), dtype=np.int32)
        count = C.c_int32(0)
        sp = B200Sampling(temp, top_k, top_p)
        keep, sptr = self._seeds(seeds, n)
        self._check(self.lib.litnice_b200_generate(self.h, self._i32(prompts), n, plen, max_new,
                                                   C.byref(sp), sptr, self._i32(out), C.byref(count)),
                    "generate")
        return out[:, :count.value].copy()

    def upload_prompts(self, prompts: np.ndarray, seeds=None):
        prompts = np.ascontiguousarray(prompts, dtype=np.int32)
        if prompts.ndim == 1:
            prompts = prompts[None, :]
        n, plen = prompts.shape
        keep, sptr = self._seeds(seeds, n)
        self._check(self.lib.litnice_b200_upload_prompts(self.h, self._i32(prompts), n, plen, sptr),
                    "upload_prompts")
        self._n = n

    def run(self, max_new: int, temp: float = 0.0, top_k: int = 0, top_p: float = 1.0) -> int:
        sp = B200Sampling(temp, top_k, top_p)
        count = C.c_int32(0)
        self._check(self.lib.litnice_b200_run(self.h, max_new, C.byref(sp), C.byref(count)), "run")
        return count.value

    def download_tokens(self, count: int) -> np.ndarray:
        out = np.zeros((self._n, max(1, count)), dtype=np.int32)
        self._check(self.lib.litnice_b200_download_tokens(self.h, self._i32(out), max(1, count)),
                    "download_tokens")
        return out[:, :count]

    def read_step_logits(self, steps: int, n_streams: int) -> np.ndarray:
        out = np.empty((steps, n_streams, self.dims.vocab), dtype=np.float32)
        self._check(self.lib.litnice_b200_read_step_logits(self.h, self._f32(out), out.size), "read_step_logits")
        return out

    def forward(self, ids: np.ndarray, all_rows: bool = False) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.ndim == 1:
            ids = ids[None, :]
        n, s = ids.shape
        out = np.empty((n, s, self.dims.vocab) if all_rows else (n, self.dims.vocab), dtype=np.float32)
        self._check(self.lib.litnice_b200_forward(self.h, self._i32(ids), n, s, 1 if all_rows else 0,
                                                  self._f32(out)), "forward")
        return out

    def inspect(self, ids: np.ndarray) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.ndim == 1:
            ids = ids[None, :]
        n, s = ids.shape
        out = np.empty((n, self.dims.vocab), dtype=np.float32)
        self._check(self.lib.litnice_b200_inspect(self.h, self._i32(ids), n, s, self._f32(out)), "inspect")
        return out

    def sample_logits(self, logits: np.ndarray, temp: float, top_k: int, top_p: float, seeds,
                      draws: int = 1) -> np.ndarray:
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        n = logits.shape[0]
        out = np.empty((n, draws), dtype=np.int32)
        sp = B200Sampling(temp, top_k, top_p)
        keep, sptr = self._seeds(seeds, n)
        self._check(self.lib.litnice_b200_sample_logits(self.h, self._f32(logits), n, C.byref(sp), sptr,
                                                        draws, self._i32(out)), "sample_logits")
        return out

    def stats(self) -> B200Stats:
        st = B200Stats()
        self._check(self.lib.litnice_b200_get_stats(self.h, C.byref(st)), "get_stats")
        return st

    def profile_step(self, n_streams: int, seq_len: int, repeats: int = 3) -> B200Stats:
        self._check(self.lib.litnice_b200_profile_step(self.h, n_streams, seq_len, repeats), "profile_step")
        return self.stats()
