"""Runs one training operator of a litnicelm backend plugin on numpy inputs through the C ABI."""
from __future__ import annotations

import numpy as np

from abi_util import Buffer, prefix_slice_view


def dense(be, arr, dtype=0):
    """A plugin buffer holding arr, and its dense view."""
    arr = np.ascontiguousarray(arr)
    buf = Buffer(be, max(arr.nbytes, 4))
    buf.host[:arr.nbytes] = arr.view(np.uint8).reshape(-1)
    buf.push()
    return buf, buf.view(arr.shape, dtype=dtype)


def sliced(be, arr, full_rows):
    """arr [B, s, C] stored as the first s rows of a [B, full_rows, C] buffer: the prefix
    slices the reference's training temporaries are (tensor_store.cpp:708-744)."""
    b, s, c = arr.shape
    buf = Buffer(be, b * full_rows * c * 4, fill=-5.0)
    view = prefix_slice_view(buf, (b, full_rows, c), s)
    buf.np_view(view)[...] = arr
    buf.push()
    return buf, view


def read(buf, view):
    buf.pull()
    return buf.np_view(view).copy()


def child_raises(snippet: str, message: str, timeout: int = 300):
    """Runs `snippet` (Python source; `be` is an open Backend of the B200 plugin, `np`, `dense`
    and `Buffer` are in scope) in a child process and checks that a C++ exception carrying
    `message` left the plugin. The table reports failures as C++ exceptions (the contract of the
    reference loader, main.cpp:37-40); a ctypes caller cannot catch those, so the child ends in
    std::terminate, which prints what()."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    code = ("import sys\nsys.path[:0] = [%r, %r]\nimport numpy as np\n"
            "from litnicelm_b200.plugin import Backend\nfrom abi_util import Buffer\n"
            "from training_util import dense\nbe = Backend()\n" % (root, here)) + snippet + "\nprint('NO EXCEPTION')\n"
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout)
    assert "NO EXCEPTION" not in p.stdout, "the call returned normally"
    assert p.returncode != 0
    assert message in p.stderr, p.stderr[-1500:]
