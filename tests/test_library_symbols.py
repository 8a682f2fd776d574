"""The shared library loads without a GPU and exports what include/*.h declares."""
import ctypes as C
import os
import re

import pytest

from litnicelm_b200 import plugin

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "litnice_backend_b200.h")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(plugin.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return plugin.load_library()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(litnice_b200_[a-z0-9_]+)\s*\(", text))
    names.add("litnice_backend_get_api")
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert set(plugin.NATIVE_SYMBOLS) <= set(names)


def test_plugin_table_layout_and_version(lib):
    # backend_plugin_api.hpp: BackendTensorView is 152 bytes, the table is
    # abi_version + 55 pointers = 448 bytes on x86-64, version 16.
    assert C.sizeof(plugin.BackendTensorView) == 152
    assert C.sizeof(plugin.BackendApiV1) == 448
    api = plugin.get_api(lib)
    assert api.abi_version == 16
    assert len(plugin.API_ENTRY_NAMES) == 55
    for name in plugin.API_ENTRY_NAMES:
        assert C.cast(getattr(api, name), C.c_void_p).value, f"table entry {name} is null"


def test_native_api_rejects_bad_arguments_without_a_gpu(lib):
    lib.litnice_b200_session_create.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)]
    h = C.c_void_p()
    assert lib.litnice_b200_session_create(None, 1, C.byref(h)) == -1
    bad = plugin.B200Dims(2, 3, 64, 256, 8, 64, 64)  # 64 % 3 != 0
    assert lib.litnice_b200_session_create(C.byref(bad), 1, C.byref(h)) == -1
    lib.litnice_b200_last_error.restype = C.c_char_p
    lib.litnice_b200_last_error.argtypes = [C.c_void_p]
    assert lib.litnice_b200_last_error(None) == b"null session"


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        plugin.load_library(str(tmp_path / "absent.so"))
