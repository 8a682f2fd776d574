"""Helpers for driving a litnicelm backend plugin through its C ABI from tests."""
from __future__ import annotations

import numpy as np

from litnicelm_b200.plugin import Backend, DevTensor


class Buffer:
    """A plugin allocation with a host mirror; views are byte-strided windows."""

    def __init__(self, be: Backend, nbytes: int, rng=None, fill=None):
        self.be = be
        self.nbytes = nbytes
        self.ptr = be.alloc(nbytes, 64)
        self.host = np.zeros(nbytes, np.uint8)
        if rng is not None:
            self.host.view(np.float32)[:] = rng.standard_normal(nbytes // 4).astype(np.float32)
        if fill is not None:
            self.host.view(np.float32)[:] = fill
        self.push()

    def push(self):
        self.be.upload(self.ptr, self.host)

    def pull(self):
        self.host = self.be.download(self.ptr, self.nbytes)
        return self.host

    def view(self, shape, strides=None, offset=0, dtype=0) -> DevTensor:
        if strides is None:
            strides, acc = [], 4
            for d in reversed(shape):
                strides.insert(0, acc)
                acc *= d
        return DevTensor(self.ptr + offset, tuple(shape), tuple(strides), dtype, self.be.device)

    def np_view(self, t: DevTensor) -> np.ndarray:
        dt = np.float32 if t.dtype == 0 else np.int32
        return np.lib.stride_tricks.as_strided(self.host[t.ptr - self.ptr:].view(dt), shape=t.shape,
                                               strides=t.strides)


def prefix_slice_view(buf: Buffer, full_shape, s, axis=1, offset=0):
    """View [.., s, ..] of a dense tensor of full_shape: strides of the full
    tensor, extent s on `axis` (the inference temp views of the reference,
    tensor_store.cpp:708-744)."""
    strides, acc = [], 4
    for d in reversed(full_shape):
        strides.insert(0, acc)
        acc *= d
    shape = list(full_shape)
    shape[axis] = s
    return buf.view(shape, strides, offset)
